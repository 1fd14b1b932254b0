// Decode-step driver 3: ONE WARP PER PROGRAM, operands streamed from global memory straight into registers.
//
// A program (row n, value head hv) is small -- about 37 KB read, ~3 000 warp instructions -- but it is a chain of short
// dependent phases.  Run by a multi-warp group out of a shared-memory stage, that chain costs ~4 000 cycles of latency
// per program and shared memory limits the SM to two programs computing at a time.  Here every warp owns a whole
// program: no block barrier, no shared-memory staging (only ~1.6 KB of per-warp scratch), so an SM keeps 16 programs
// in flight and the scheduler hides one warp's latency behind the others.  Loads are 16-byte, coalesced (a warp-wide
// load covers four whole 128-byte rows) and kept 8 deep per warp.
//
// Lane mapping (lane = 8 g + l8): for the tile and the key rows, row group g takes row 4 pass + g and lane l8 owns the
// 16 columns 16 l8 ..; for the value-side epilogue lane owns the four values 4 lane .. 4 lane + 3.
#pragma once
// (included from lq_step.cu inside namespace lq, after the shared helpers)

constexpr int WK_WARPS = 4;                        // warps per CTA of the warp-per-program driver
constexpr int WK_SCRATCH = 72 * 8 + 128 * 8;       // per warp: wd[72] float2, mqy[128] float2

__device__ __forceinline__ uint4 ldg16(const void* p) { return ldg_stream(p); }
__device__ __forceinline__ uint2 ldg8(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

template <int R>
__global__ void __launch_bounds__(32 * WK_WARPS, 4) step_warp_gdn_kernel(StepParams P) {
    __shared__ __align__(16) char wk_smem[WK_WARPS * WK_SCRATCH];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, l8 = lane & 7, g = lane >> 3;
    float2* wd = reinterpret_cast<float2*>(wk_smem + wib * WK_SCRATCH);
    float2* mqy = wd + 72;
    const int HV = P.d.HV, H = P.d.H, L = P.d.L;
    const int nprog = P.N * HV;
    const int nwarps = gridDim.x * WK_WARPS;
    const int MIX = 2 * H * KD + HV * VD;
    const int gqa = HV / H;

    for (int p = blockIdx.x * WK_WARPS + wib; p < nprog; p += nwarps) {
        const int n = p / HV, hv = p - n * HV;
        const ProgScalars sc = load_scalars(P, n, hv, false);        // uniform loads: every lane gets the same values
        uint32_t* orow = reinterpret_cast<uint32_t*>(P.o) + int64_t(p) * 64;
        if (!prog_live(sc, L)) {
            reinterpret_cast<uint2*>(orow)[lane] = make_uint2(0u, 0u);
            continue;
        }
        const int h = sc.h;
        const int64_t sh = int64_t(sc.slot) * HV + hv;
        const char* base = head_base(P.ssm, P.d.SS, sc.slot, hv);
        const char* mrow = reinterpret_cast<const char*>(P.mixed + int64_t(n) * MIX);
        const int hk = hv / gqa;
        const char* kb = reinterpret_cast<const char*>(P.Kbuf + sh * L * KD);
        const char* ub = reinterpret_cast<const char*>(P.Ubuf + sh * L * VD);

        // ---- loads that everything else waits for, issued first: tile rows 0..31, q, k, Sk, Sv ----
        uint4 tb[8];
        const char* trow = base + CK_CODES + g * KD + l8 * 16;      // + 512 per pass
#pragma unroll
        for (int it = 0; it < 8; ++it) tb[it] = ldg16(trow + it * 512);
        const uint4 q0 = ldg16(mrow + hk * 256 + l8 * 32), q1 = ldg16(mrow + hk * 256 + l8 * 32 + 16);
        const uint4 k0 = ldg16(mrow + (H + hk) * 256 + l8 * 32), k1 = ldg16(mrow + (H + hk) * 256 + l8 * 32 + 16);
        float4 sk4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) sk4[i] = *reinterpret_cast<const float4*>(base + CK_SK + l8 * 64 + i * 16);
        float svr[4];                                                // Sv of the four rows this lane ends up owning
#pragma unroll
        for (int b = 0; b < 4; ++b) svr[b] = reinterpret_cast<const float*>(base + CK_SV)[32 * b + 4 * l8 + g];

        // ---- l2 norms over this lane's 16 columns, reduced over the row group ----
        float2 kn[8], qn[8];
        float kq;
        {
            const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            const uint32_t kw[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
            float sq = 0.f, sk = 0.f, skq = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                qn[i] = bf16x2_to_f2(qw[i]);
                kn[i] = bf16x2_to_f2(kw[i]);
                sq = fmaf(qn[i].x, qn[i].x, sq); sq = fmaf(qn[i].y, qn[i].y, sq);
                sk = fmaf(kn[i].x, kn[i].x, sk); sk = fmaf(kn[i].y, kn[i].y, sk);
                skq = fmaf(kn[i].x, qn[i].x, skq); skq = fmaf(kn[i].y, qn[i].y, skq);
            }
            sq = oct_sum(sq); sk = oct_sum(sk); skq = oct_sum(skq);
            const float inq = rsqrtf(sq + 1e-6f) * P.scale, ink = rsqrtf(sk + 1e-6f);
            kq = skq * inq * ink;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                qn[i] = __fmul2_rn(qn[i], make_float2(inq, inq));
                kn[i] = __fmul2_rn(kn[i], make_float2(ink, ink));
            }
        }
        if (g == 0) {                                                // append k_hat (bf16): row group 0 holds all 128 columns
            uint4 a0, a1;
            a0.x = f2_to_bf16x2(kn[0].x, kn[0].y); a0.y = f2_to_bf16x2(kn[1].x, kn[1].y);
            a0.z = f2_to_bf16x2(kn[2].x, kn[2].y); a0.w = f2_to_bf16x2(kn[3].x, kn[3].y);
            a1.x = f2_to_bf16x2(kn[4].x, kn[4].y); a1.y = f2_to_bf16x2(kn[5].x, kn[5].y);
            a1.z = f2_to_bf16x2(kn[6].x, kn[6].y); a1.w = f2_to_bf16x2(kn[7].x, kn[7].y);
            uint4* dst = reinterpret_cast<uint4*>(P.Kbuf + (sh * L + h) * KD) + l8 * 2;
            dst[0] = a0;
            dst[1] = a1;
        }

        // ---- window dots: row j = 4 ch + g; two passes in flight ----
        const int nch = (h + 3) >> 2;
        for (int ch = 0; ch < nch; ch += 2) {
            const int ja = 4 * ch + g, jb = ja + 4;
            const bool la = ja < h, lb = jb < h;
            const char* ra = kb + (la ? ja : 0) * 256 + l8 * 32;
            const char* rb = kb + (lb ? jb : 0) * 256 + l8 * 32;
            const uint4 a0 = ldg16(ra), a1 = ldg16(ra + 16), b0 = ldg16(rb), b1 = ldg16(rb + 16);
            const float wa = la ? P.Wbuf[sh * L + ja] : 0.f, wb = lb ? P.Wbuf[sh * L + jb] : 0.f;
            const uint32_t xa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const uint32_t xb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            float2 aka = make_float2(0.f, 0.f), aqa = aka, akb = aka, aqb = aka;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 fa = bf16x2_to_f2(xa[i]), fb = bf16x2_to_f2(xb[i]);
                aka = __ffma2_rn(fa, kn[i], aka);
                aqa = __ffma2_rn(fa, qn[i], aqa);
                akb = __ffma2_rn(fb, kn[i], akb);
                aqb = __ffma2_rn(fb, qn[i], aqb);
            }
            float dka = aka.x + aka.y, dqa = aqa.x + aqa.y, dkb = akb.x + akb.y, dqb = aqb.x + aqb.y;
#pragma unroll
            for (int o = 1; o <= 4; o <<= 1) {
                dka += __shfl_xor_sync(0xffffffffu, dka, o);
                dqa += __shfl_xor_sync(0xffffffffu, dqa, o);
                dkb += __shfl_xor_sync(0xffffffffu, dkb, o);
                dqb += __shfl_xor_sync(0xffffffffu, dqb, o);
            }
            if (l8 == 0) {
                if (la) { const float wj = wa * sc.alpha; P.Wbuf[sh * L + ja] = wj; wd[ja] = make_float2(wj * dka, wj * dqa); }
                if (lb) { const float wj = wb * sc.alpha; P.Wbuf[sh * L + jb] = wj; wd[jb] = make_float2(wj * dkb, wj * dqb); }
            }
        }
        // ---- factor dots: row group g takes factors g, g + 4 ----
#pragma unroll
        for (int cr = 0; cr < R / 4; ++cr) {
            const int r = 4 * cr + g;
            const char* up = base + CK_UQ + r * 512 + l8 * 32;
            const uint4 r0 = ldg16(up), r1 = ldg16(up + 16);
            const uint32_t ww[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            float2 ak = make_float2(0.f, 0.f), aq = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 x = f16x2_to_f2(ww[i]);
                ak = __ffma2_rn(x, kn[i], ak);
                aq = __ffma2_rn(x, qn[i], aq);
            }
            const float dk = oct_sum(ak.x + ak.y), dq = oct_sum(aq.x + aq.y);
            if (l8 == 0) wd[64 + r] = make_float2(dk, dq);
        }

        // ---- checkpoint matvec: operands k_hat Sk / 127, q_hat Sk / 127; 32 passes, 8 loads in flight ----
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 sa = make_float2(sk4[i].x * (1.0f / QMAX), sk4[i].y * (1.0f / QMAX));
            const float2 sb = make_float2(sk4[i].z * (1.0f / QMAX), sk4[i].w * (1.0f / QMAX));
            kn[2 * i] = __fmul2_rn(kn[2 * i], sa);
            qn[2 * i] = __fmul2_rn(qn[2 * i], sa);
            kn[2 * i + 1] = __fmul2_rn(kn[2 * i + 1], sb);
            qn[2 * i + 1] = __fmul2_rn(qn[2 * i + 1], sb);
        }
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
            float pk[8], pq[8];
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const uint4 cw = tb[it];
                if (blk < 3) tb[it] = ldg16(trow + ((blk + 1) * 8 + it) * 512);      // refill the slot: pass + 8
                const uint32_t ww[4] = {cw.x, cw.y, cw.z, cw.w};
                float2 ak = make_float2(0.f, 0.f), aq = make_float2(0.f, 0.f);
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    float2 xa, xb;
                    s8x4_to_f2x2(ww[m], xa, xb);
                    ak = __ffma2_rn(xa, kn[2 * m], ak);
                    aq = __ffma2_rn(xa, qn[2 * m], aq);
                    ak = __ffma2_rn(xb, kn[2 * m + 1], ak);
                    aq = __ffma2_rn(xb, qn[2 * m + 1], aq);
                }
                pk[it] = ak.x + ak.y;
                pq[it] = aq.x + aq.y;
            }
            const float mqr = pass_transpose_sum(pk, l8), yqr = pass_transpose_sum(pq, l8);
            mqy[32 * blk + 4 * l8 + g] = make_float2(mqr * svr[blk], yqr * svr[blk]);
        }
        __syncwarp();

        // ---- value side: lane owns values 4 lane .. 4 lane + 3 ----
        float2 ck0 = make_float2(0.f, 0.f), ck1 = ck0, cq0 = ck0, cq1 = ck0;
        {
            const char* up = ub + lane * 8;
            int j = 0;
            for (; j + 4 <= h; j += 4) {
                uint2 u[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) u[i] = ldg8(up + (j + i) * 256);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 w2 = wd[j + i];
                    const float2 wk = make_float2(w2.x, w2.x), wq = make_float2(w2.y, w2.y);
                    const float2 ua = bf16x2_to_f2(u[i].x), ubv = bf16x2_to_f2(u[i].y);
                    ck0 = __ffma2_rn(ua, wk, ck0); ck1 = __ffma2_rn(ubv, wk, ck1);
                    cq0 = __ffma2_rn(ua, wq, cq0); cq1 = __ffma2_rn(ubv, wq, cq1);
                }
            }
            for (; j < h; ++j) {
                const uint2 u = ldg8(up + j * 256);
                const float2 w2 = wd[j];
                const float2 wk = make_float2(w2.x, w2.x), wq = make_float2(w2.y, w2.y);
                const float2 ua = bf16x2_to_f2(u.x), ubv = bf16x2_to_f2(u.y);
                ck0 = __ffma2_rn(ua, wk, ck0); ck1 = __ffma2_rn(ubv, wk, ck1);
                cq0 = __ffma2_rn(ua, wq, cq0); cq1 = __ffma2_rn(ubv, wq, cq1);
            }
        }
        float2 rk0 = make_float2(0.f, 0.f), rk1 = rk0, rq0 = rk0, rq1 = rk0;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint2 qv = ldg8(base + CK_UQ + r * 512 + 256 + lane * 8);
            const float2 dd = wd[64 + r];
            const float2 dk = make_float2(dd.x, dd.x), dq = make_float2(dd.y, dd.y);
            const float2 qa = f16x2_to_f2(qv.x), qb = f16x2_to_f2(qv.y);
            rk0 = __ffma2_rn(qa, dk, rk0); rk1 = __ffma2_rn(qb, dk, rk1);
            rq0 = __ffma2_rn(qa, dq, rq0); rq1 = __ffma2_rn(qb, dq, rq1);
        }
        const uint2 vw = ldg8(mrow + (2 * H + hv) * 256 + lane * 8);
        const float4 ma = *reinterpret_cast<const float4*>(mqy + 4 * lane);          // (mq, yq) of values 4 lane, 4 lane + 1
        const float4 mb = *reinterpret_cast<const float4*>(mqy + 4 * lane + 2);      // ... + 2, + 3
        const float2 va = bf16x2_to_f2(vw.x), vb = bf16x2_to_f2(vw.y);
        const float pn = sc.pold * sc.alpha, beta = sc.beta;
        const float u0 = beta * (va.x - (pn * (ma.x + rk0.x) + ck0.x));
        const float u1 = beta * (va.y - (pn * (ma.z + rk0.y) + ck0.y));
        const float u2 = beta * (vb.x - (pn * (mb.x + rk1.x) + ck1.x));
        const float u3 = beta * (vb.y - (pn * (mb.z + rk1.y) + ck1.y));
        const float y0 = pn * (ma.y + rq0.x) + cq0.x + kq * u0;
        const float y1 = pn * (ma.w + rq0.y) + cq0.y + kq * u1;
        const float y2 = pn * (mb.y + rq1.x) + cq1.x + kq * u2;
        const float y3 = pn * (mb.w + rq1.y) + cq1.y + kq * u3;
        reinterpret_cast<uint2*>(orow)[lane] = make_uint2(f2_to_bf16x2(y0, y1), f2_to_bf16x2(y2, y3));
        reinterpret_cast<uint2*>(P.Ubuf + (sh * L + h) * VD)[lane] = make_uint2(f2_to_bf16x2(u0, u1), f2_to_bf16x2(u2, u3));
        if (lane == 0) {
            P.Pbuf[sh] = pn;
            P.Wbuf[sh * L + h] = 1.f;
            P.hcnt[sh] = h + 1;
        }
        __syncwarp();                                                // wd / mqy are reused by this warp's next program
    }
}

