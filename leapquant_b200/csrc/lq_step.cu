// GDN / KDA decode-step kernels (sm_100a).
//
// One "program" is one (row n, value head hv): it streams the head's INT8 checkpoint (codes, scales, factors) and the
// h live entries of its window buffer, and appends the new token.  A program is executed by a group of 128 threads
// working out of a shared-memory stage; the same body serves the two drivers in this file:
//   * step_direct_kernel    : one CTA per program, cooperative 16-byte global loads into the stage;
//   * step_pipelined_kernel : persistent CTAs, a producer warp filling a ring of stages with bulk asynchronous
//                             copies (cp.async.bulk + mbarrier) while the consumer groups compute.
//
// Thread mapping of the matvec: eight lanes share a row of the 128 x 128 INT8 tile; lane l8 = lane & 7 owns the
// 16 columns 16 l8 .. 16 l8 + 15, so a warp-wide 16-byte load covers four whole 128-byte rows and the operand
// vectors k_hat * Sk / 127 and q_hat * Sk / 127 for those columns stay in registers for the whole tile.
#include <string.h>

#include "lq_common.cuh"

namespace lq {

constexpr int GT = 128;                   // threads of one consumer group

// ---- stage layout (bytes); the checkpoint part mirrors the packed slot so that it is ONE contiguous copy ----
struct StageLayout {
    int kb, ub, w, q, k, v, gb, pb, a, dtb, sc, bytes;
};
__host__ __device__ inline StageLayout stage_layout(int L, int R, bool kda) {
    StageLayout s;
    int o = ck_bytes(R);
    s.kb = o; o += L * 256;
    s.ub = o; o += L * 256;
    s.w = o; o += 256;
    s.q = o; o += 256;
    s.k = o; o += 256;
    s.v = o; o += 256;
    s.gb = s.pb = s.a = s.dtb = 0;
    if (kda) {
        s.gb = o; o += L * 256;
        s.pb = o; o += 512;
        s.a = o; o += 256;
        s.dtb = o; o += 512;
    }
    s.sc = o; o += 32;                      // ProgScalars written by the producer warp (pipelined driver)
    s.bytes = (o + 127) & ~127;
    return s;
}

struct StepParams {
    lq_dims d;
    char* ssm;
    uint16_t* Kbuf;
    uint16_t* Ubuf;
    float* Wbuf;
    float* Pbuf;
    uint16_t* Gbuf;
    int32_t* hcnt;
    const uint16_t* mixed;
    const uint16_t* a;
    const uint16_t* b;
    const float* A_log;
    const float* dt_bias;
    const int32_t* idx;
    uint16_t* o;
    int N;
    float scale;
    float glb;
};

// per-program scalars, produced once and read by the whole group
struct ProgScalars {
    int slot, h, n, hv;
    float alpha, beta, pold, ea;
};

// per-group scratch in shared memory
struct GroupScratch {
    float2* wd;      // [64 + 8]  (w_j dk_j, w_j dq_j) for j < L, then (dU_r . k, dU_r . q) at 64 + r
    float2* mqy;     // [128]     (mq, yq) per row
    float4* part;    // [64][2]   partial contribution sums of the odd-j half
    float* pcs;      // [128]     KDA: pc per column
    float* ens;      // [128]     KDA: en per column
};
constexpr int SCRATCH_BYTES = (72 * 8) + 128 * 8 + 64 * 32 + 128 * 4 + 128 * 4;   // 4672

__device__ __forceinline__ GroupScratch carve_scratch(char* p) {
    GroupScratch g;
    g.wd = reinterpret_cast<float2*>(p); p += 72 * 8;
    g.mqy = reinterpret_cast<float2*>(p); p += 128 * 8;
    g.part = reinterpret_cast<float4*>(p); p += 64 * 32;
    g.pcs = reinterpret_cast<float*>(p); p += 128 * 4;
    g.ens = reinterpret_cast<float*>(p);
    return g;
}

__device__ __forceinline__ ProgScalars load_scalars(const StepParams& P, int n, int hv, bool kda) {
    ProgScalars s;
    s.n = n; s.hv = hv;
    s.slot = P.idx[n];
    s.h = 0; s.alpha = 1.f; s.beta = 0.f; s.pold = 1.f; s.ea = 1.f;
    if (s.slot > 0 && s.slot < P.d.NS) {
        const int64_t sh = int64_t(s.slot) * P.d.HV + hv;
        s.h = P.hcnt[sh];
        s.ea = expf(P.A_log[hv]);
        s.beta = round_bf16(sigmoidf_(bf16_to_f(P.b[int64_t(n) * P.d.HV + hv])));
        if (!kda) {
            const float xg = bf16_to_f(P.a[int64_t(n) * P.d.HV + hv]) + P.dt_bias[hv];
            s.alpha = expf(-s.ea * softplus_thr(xg));
            s.pold = P.Pbuf[sh];
        }
    } else {
        s.slot = 0;
    }
    return s;
}

// Transposed reduction: every lane holds eight partial sums x[0..7] (one per tile pass); the eight lanes of a row group
// add them up so that lane l8 ends with the total of pass l8.  7 shuffles instead of 24.
__device__ __forceinline__ float oct_transpose_sum(const float (&x)[8], int l8) {
    float y[4];
    const bool b2 = l8 & 4;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float keep = b2 ? x[4 + k] : x[k];
        const float send = b2 ? x[k] : x[4 + k];
        y[k] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    float z[2];
    const bool b1 = l8 & 2;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const float keep = b1 ? y[2 + k] : y[k];
        const float send = b1 ? y[k] : y[2 + k];
        z[k] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
    const bool b0 = l8 & 1;
    const float keep = b0 ? z[1] : z[0];
    const float send = b0 ? z[0] : z[1];
    return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

// ------------------------------------------------------------------------------------------------------------------
// the program body: 128 threads, operands in the shared-memory stage `st`
// ------------------------------------------------------------------------------------------------------------------
template <int R, bool KDA>
__device__ __forceinline__ void step_body(const StepParams& P, const ProgScalars& sc, char* st, const StageLayout& lay,
                                          const GroupScratch& gs, int t, int bar) {
    const int w = t >> 5, lane = t & 31, l8 = lane & 7, g = lane >> 3;
    const int L = P.d.L, h = sc.h;
    const int64_t sh = int64_t(sc.slot) * P.d.HV + sc.hv;
    const float alpha = sc.alpha;

    // ---- KDA pre-pass (thread per key channel): gate, cumulative log gate, decayed window keys ----
    if (KDA) {
        const int c = t;
        const float xg = bf16_to_f(reinterpret_cast<const uint16_t*>(st + lay.a)[c]) + reinterpret_cast<const float*>(st + lay.dtb)[c];
        float gl;
        if (P.glb != 0.f) gl = P.glb * (1.0f / (1.0f + __expf(-sc.ea * xg)));
        else gl = -sc.ea * (xg <= SOFTPLUS_THRESHOLD ? __logf(1.0f + __expf(xg)) : xg);
        const float gn = reinterpret_cast<const float*>(st + lay.pb)[c] + gl;
        const float en = __expf(gl);
        gs.pcs[c] = __expf(gn);
        gs.ens[c] = en;
        P.Pbuf[sh * KD + c] = gn;
        P.Gbuf[(sh * L + h) * KD + c] = f_to_f16(en);
        uint16_t* kb = reinterpret_cast<uint16_t*>(st + lay.kb);
        const uint16_t* gb = reinterpret_cast<const uint16_t*>(st + lay.gb);
        float dcur = en;
        for (int j = h - 1; j >= 0; --j) {
            kb[j * KD + c] = f_to_bf16(bf16_to_f(kb[j * KD + c]) * dcur);
            dcur *= f16_to_f(gb[j * KD + c]);
        }
        named_bar(bar, GT);
    }

    // ---- l2 norms of q and k over this lane's 16 columns, reduced over the 8 lanes of the row group ----
    float2 kn[8], qn[8];
    float kq;
    {
        const uint4 q0 = reinterpret_cast<const uint4*>(st + lay.q)[l8 * 2], q1 = reinterpret_cast<const uint4*>(st + lay.q)[l8 * 2 + 1];
        const uint4 k0 = reinterpret_cast<const uint4*>(st + lay.k)[l8 * 2], k1 = reinterpret_cast<const uint4*>(st + lay.k)[l8 * 2 + 1];
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
    // append k_hat (bf16) to the window: warp 0, row group 0 holds all 128 columns
    if (w == 0 && g == 0) {
        uint4 a0, a1;
        a0.x = f2_to_bf16x2(kn[0].x, kn[0].y); a0.y = f2_to_bf16x2(kn[1].x, kn[1].y);
        a0.z = f2_to_bf16x2(kn[2].x, kn[2].y); a0.w = f2_to_bf16x2(kn[3].x, kn[3].y);
        a1.x = f2_to_bf16x2(kn[4].x, kn[4].y); a1.y = f2_to_bf16x2(kn[5].x, kn[5].y);
        a1.z = f2_to_bf16x2(kn[6].x, kn[6].y); a1.w = f2_to_bf16x2(kn[7].x, kn[7].y);
        uint4* dst = reinterpret_cast<uint4*>(P.Kbuf + (sh * L + h) * KD) + l8 * 2;
        dst[0] = a0;
        dst[1] = a1;
    }

    // ---- window dots dk_j = K_j . k_hat, dq_j = K_j . q_hat: four rows per warp pass, passes dealt round-robin to the warps ----
    const int nch = (h + 3) >> 2;
    for (int ch = w; ch < nch; ch += 4) {
        const int j = 4 * ch + g;
        const bool live = j < h;
        const int jj = live ? j : 0;
        const uint4 r0 = reinterpret_cast<const uint4*>(st + lay.kb + jj * 256)[l8 * 2];
        const uint4 r1 = reinterpret_cast<const uint4*>(st + lay.kb + jj * 256)[l8 * 2 + 1];
        const uint32_t ww[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        float2 ak = make_float2(0.f, 0.f), aq = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 x = bf16x2_to_f2(ww[i]);
            ak = __ffma2_rn(x, kn[i], ak);
            aq = __ffma2_rn(x, qn[i], aq);
        }
        const float dk = oct_sum(ak.x + ak.y), dq = oct_sum(aq.x + aq.y);
        if (live && l8 == 0) {
            float wj = reinterpret_cast<const float*>(st + lay.w)[j];
            if (!KDA) {
                wj *= alpha;
                P.Wbuf[sh * L + j] = wj;
            }
            gs.wd[j] = make_float2(wj * dk, wj * dq);
        }
    }
    // ---- factor dots dU_r . k_hat, dU_r . q_hat (KDA: U_r[c] pc[c]) ----
#pragma unroll
    for (int cr = 0; cr < R / 4; ++cr) {
        if (((nch + cr) & 3) == w) {
            const int r = 4 * cr + g;
            const uint4 r0 = reinterpret_cast<const uint4*>(st + CK_UQ + r * 512)[l8 * 2];
            const uint4 r1 = reinterpret_cast<const uint4*>(st + CK_UQ + r * 512)[l8 * 2 + 1];
            const uint32_t ww[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            float2 ak = make_float2(0.f, 0.f), aq = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float2 x = f16x2_to_f2(ww[i]);
                if (KDA) x = __fmul2_rn(x, *reinterpret_cast<const float2*>(gs.pcs + l8 * 16 + 2 * i));
                ak = __ffma2_rn(x, kn[i], ak);
                aq = __ffma2_rn(x, qn[i], aq);
            }
            const float dk = oct_sum(ak.x + ak.y), dq = oct_sum(aq.x + aq.y);
            if (l8 == 0) gs.wd[64 + r] = make_float2(dk, dq);
        }
    }

    // ---- checkpoint matvec: operands k_hat Sk / 127 (pc), q_hat Sk / 127 (pc) for this lane's columns ----
    {
        const float4* skp = reinterpret_cast<const float4*>(st + CK_SK) + l8 * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 s4 = skp[i];
            if (KDA) {
                const float4 p4 = reinterpret_cast<const float4*>(gs.pcs)[l8 * 4 + i];
                s4.x *= p4.x; s4.y *= p4.y; s4.z *= p4.z; s4.w *= p4.w;
            }
            const float2 sa = make_float2(s4.x * (1.0f / QMAX), s4.y * (1.0f / QMAX));
            const float2 sb = make_float2(s4.z * (1.0f / QMAX), s4.w * (1.0f / QMAX));
            kn[2 * i] = __fmul2_rn(kn[2 * i], sa);
            qn[2 * i] = __fmul2_rn(qn[2 * i], sa);
            kn[2 * i + 1] = __fmul2_rn(kn[2 * i + 1], sb);
            qn[2 * i + 1] = __fmul2_rn(qn[2 * i + 1], sb);
        }
    }
    float pk[8], pq[8];
    {
        const uint4* tile = reinterpret_cast<const uint4*>(st + CK_CODES);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int row = 32 * w + 4 * it + g;
            const uint4 cw = tile[row * 8 + l8];
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
    }
    {
        const float mqr = oct_transpose_sum(pk, l8), yqr = oct_transpose_sum(pq, l8);
        const int row = 32 * w + 4 * l8 + g;
        const float svv = reinterpret_cast<const float*>(st + CK_SV)[row];
        gs.mqy[row] = make_float2(mqr * svv, yqr * svv);
    }
    named_bar(bar, GT);

    // ---- contribution of the window and of the rank-R part: thread = (value pair vp, parity of j) ----
    const int vp = t & 63, jh = t >> 6;
    float2 ck = make_float2(0.f, 0.f), cq = make_float2(0.f, 0.f), rk = make_float2(0.f, 0.f), rq = make_float2(0.f, 0.f);
    {
        const uint32_t* ub = reinterpret_cast<const uint32_t*>(st + lay.ub);
#pragma unroll 4
        for (int j = jh; j < h; j += 2) {
            const float2 u2 = bf16x2_to_f2(ub[j * 64 + vp]);
            const float2 wd = gs.wd[j];
            ck = __ffma2_rn(u2, make_float2(wd.x, wd.x), ck);
            cq = __ffma2_rn(u2, make_float2(wd.y, wd.y), cq);
        }
        const uint32_t* uq = reinterpret_cast<const uint32_t*>(st + CK_UQ);
#pragma unroll
        for (int r = jh; r < R; r += 2) {
            const float2 q2 = f16x2_to_f2(uq[r * 128 + 64 + vp]);
            const float2 dd = gs.wd[64 + r];
            rk = __ffma2_rn(q2, make_float2(dd.x, dd.x), rk);
            rq = __ffma2_rn(q2, make_float2(dd.y, dd.y), rq);
        }
    }
    if (jh == 1) {
        gs.part[vp * 2] = make_float4(ck.x, ck.y, cq.x, cq.y);
        gs.part[vp * 2 + 1] = make_float4(rk.x, rk.y, rq.x, rq.y);
    }
    named_bar(bar, GT);
    if (jh == 0) {
        const float4 pa = gs.part[vp * 2], pb = gs.part[vp * 2 + 1];
        ck.x += pa.x; ck.y += pa.y; cq.x += pa.z; cq.y += pa.w;
        rk.x += pb.x; rk.y += pb.y; rq.x += pb.z; rq.y += pb.w;
        const float2 m0 = gs.mqy[2 * vp], m1 = gs.mqy[2 * vp + 1];
        const float2 vv = bf16x2_to_f2(reinterpret_cast<const uint32_t*>(st + lay.v)[vp]);
        const float beta = sc.beta;
        float u0, u1, y0, y1;
        if (KDA) {
            u0 = beta * (vv.x - (m0.x + rk.x + ck.x));
            u1 = beta * (vv.y - (m1.x + rk.y + ck.y));
            y0 = m0.y + rq.x + cq.x + kq * u0;
            y1 = m1.y + rq.y + cq.y + kq * u1;
        } else {
            const float pn = sc.pold * alpha;
            u0 = beta * (vv.x - (pn * (m0.x + rk.x) + ck.x));
            u1 = beta * (vv.y - (pn * (m1.x + rk.y) + ck.y));
            y0 = pn * (m0.y + rq.x) + cq.x + kq * u0;
            y1 = pn * (m1.y + rq.y) + cq.y + kq * u1;
            if (t == 0) P.Pbuf[sh] = pn;
        }
        reinterpret_cast<uint32_t*>(P.o)[(int64_t(sc.n) * P.d.HV + sc.hv) * 64 + vp] = f2_to_bf16x2(y0, y1);
        reinterpret_cast<uint32_t*>(P.Ubuf)[(sh * L + h) * 64 + vp] = f2_to_bf16x2(u0, u1);
        if (t == 0) {
            P.Wbuf[sh * L + h] = 1.f;
            P.hcnt[sh] = h + 1;
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// driver 1: one CTA per program, plain 16-byte loads
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void copy16(char* dst, const char* src, int bytes, int t, int nthreads) {
    const int n16 = bytes >> 4;
    int i = t;
    for (; i + 3 * nthreads < n16; i += 4 * nthreads) {
        const uint4 a = ldg_stream(src + 16 * i), b = ldg_stream(src + 16 * (i + nthreads));
        const uint4 c = ldg_stream(src + 16 * (i + 2 * nthreads)), d = ldg_stream(src + 16 * (i + 3 * nthreads));
        reinterpret_cast<uint4*>(dst)[i] = a;
        reinterpret_cast<uint4*>(dst)[i + nthreads] = b;
        reinterpret_cast<uint4*>(dst)[i + 2 * nthreads] = c;
        reinterpret_cast<uint4*>(dst)[i + 3 * nthreads] = d;
    }
    for (; i < n16; i += nthreads) reinterpret_cast<uint4*>(dst)[i] = ldg_stream(src + 16 * i);
}

template <int R, bool KDA>
__global__ void __launch_bounds__(GT, 4) step_direct_kernel(StepParams P) {
    extern __shared__ __align__(128) char stage_smem[];
    __shared__ ProgScalars s_sc;
    const int t = threadIdx.x;
    const int prog = blockIdx.x;
    const int n = prog / P.d.HV, hv = prog - n * P.d.HV;
    const StageLayout lay = stage_layout(P.d.L, R, KDA);
    if (t == 0) s_sc = load_scalars(P, n, hv, KDA);
    __syncthreads();
    const ProgScalars sc = s_sc;
    if (sc.slot <= 0 || sc.h >= P.d.L || sc.h < 0) {
        if (t < 64) reinterpret_cast<uint32_t*>(P.o)[(int64_t(n) * P.d.HV + hv) * 64 + t] = 0u;
        return;
    }
    const int L = P.d.L, H = P.d.H, HV = P.d.HV, h = sc.h;
    const int hk = hv / (HV / H);
    const int64_t sh = int64_t(sc.slot) * HV + hv;
    const int MIX = 2 * H * KD + HV * VD;
    char* st = stage_smem;
    copy16(st, head_base(P.ssm, P.d.SS, sc.slot, hv), ck_bytes(R), t, GT);
    copy16(st + lay.kb, reinterpret_cast<const char*>(P.Kbuf + sh * L * KD), h * 256, t, GT);
    copy16(st + lay.ub, reinterpret_cast<const char*>(P.Ubuf + sh * L * VD), h * 256, t, GT);
    copy16(st + lay.w, reinterpret_cast<const char*>(P.Wbuf + sh * L), L * 4, t, GT);
    const char* mrow = reinterpret_cast<const char*>(P.mixed + int64_t(n) * MIX);
    if (t < 16) reinterpret_cast<uint4*>(st + lay.q)[t] = ldg_stream(mrow + hk * 256 + 16 * t);
    else if (t < 32) reinterpret_cast<uint4*>(st + lay.k)[t - 16] = ldg_stream(mrow + (H + hk) * 256 + 16 * (t - 16));
    else if (t < 48) reinterpret_cast<uint4*>(st + lay.v)[t - 32] = ldg_stream(mrow + 2 * H * 256 + hv * 256 + 16 * (t - 32));
    if (KDA) {
        copy16(st + lay.gb, reinterpret_cast<const char*>(P.Gbuf + sh * L * KD), h * 256, t, GT);
        copy16(st + lay.pb, reinterpret_cast<const char*>(P.Pbuf + sh * KD), 512, t, GT);
        copy16(st + lay.a, reinterpret_cast<const char*>(P.a + (int64_t(n) * HV + hv) * KD), 256, t, GT);
        copy16(st + lay.dtb, reinterpret_cast<const char*>(P.dt_bias + int64_t(hv) * KD), 512, t, GT);
    }
    __syncthreads();
    const GroupScratch gs = carve_scratch(stage_smem + lay.bytes);
    step_body<R, KDA>(P, sc, st, lay, gs, t, 1);
}

// ------------------------------------------------------------------------------------------------------------------
// driver 2: persistent CTAs, producer warp + bulk asynchronous copies into a ring of stages
// ------------------------------------------------------------------------------------------------------------------
constexpr uint32_t WAIT_LIMIT = 1u << 22;      // bounded spin: ~seconds at worst, then the kernel records a status and leaves
constexpr int ST_PRODUCER_TIMEOUT = 1, ST_CONSUMER_TIMEOUT = 2;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)
        : "memory");
    return ok != 0;
}
// waits for the phase with the given parity; gives up after WAIT_LIMIT polls
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// bulk asynchronous copy global -> this CTA's shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// group-wide AND of a predicate over a named barrier (also a barrier)
__device__ __forceinline__ bool group_all(int bar, int nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %3, 0;\n"
        "barrier.cta.red.and.pred p, %1, %2, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r)
        : "r"(bar), "r"(nthreads), "r"(uint32_t(pred))
        : "memory");
    return r != 0;
}

template <int R, bool KDA, int NG>
__global__ void __launch_bounds__(32 + NG * GT, 1) step_pipelined_kernel(StepParams P, int nstages) {
    extern __shared__ __align__(128) char stage_smem[];
    const StageLayout lay = stage_layout(P.d.L, R, KDA);
    char* scratch0 = stage_smem + size_t(nstages) * lay.bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(scratch0 + NG * SCRATCH_BYTES);
    uint64_t* empty = full + nstages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int HV = P.d.HV, H = P.d.H, L = P.d.L;
    const int nprog = P.N * HV;
    const int grid = gridDim.x, bid = blockIdx.x;
    const int nit = (nprog - bid + grid - 1) / grid;

    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, GT);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    __syncthreads();

    if (warp == 0) {
        // ================= producer: scalars of 32 programs per batch, then one stage fill per program =================
        const int MIX = 2 * H * KD + HV * VD;
        const int gqa = HV / H;
        ProgScalars cur, nxt;
        auto fetch = [&](int i) {
            ProgScalars r;
            r.slot = 0; r.h = 0; r.n = 0; r.hv = 0; r.alpha = 1.f; r.beta = 0.f; r.pold = 1.f; r.ea = 1.f;
            if (i < nit) {
                const int p = bid + i * grid;
                const int n = p / HV;
                r = load_scalars(P, n, p - n * HV, KDA);
            }
            return r;
        };
        nxt = fetch(lane);
        bool ok = true;
        for (int base = 0; base < nit && ok; base += 32) {
            cur = nxt;
            nxt = fetch(base + 32 + lane);
            const int cnt = min(32, nit - base);
            for (int j = 0; j < cnt; ++j) {
                const int i = base + j;
                const int s = i % nstages;
                const uint32_t u = uint32_t(i / nstages);
                ProgScalars sc;
                sc.slot = __shfl_sync(0xffffffffu, cur.slot, j);
                sc.h = __shfl_sync(0xffffffffu, cur.h, j);
                sc.n = __shfl_sync(0xffffffffu, cur.n, j);
                sc.hv = __shfl_sync(0xffffffffu, cur.hv, j);
                sc.alpha = __shfl_sync(0xffffffffu, cur.alpha, j);
                sc.beta = __shfl_sync(0xffffffffu, cur.beta, j);
                sc.pold = __shfl_sync(0xffffffffu, cur.pold, j);
                sc.ea = __shfl_sync(0xffffffffu, cur.ea, j);
                int good = 1;
                if (lane == 0) good = mbar_wait_bounded(empty + s, (u & 1u) ^ 1u) ? 1 : 0;
                good = __shfl_sync(0xffffffffu, good, 0);
                if (!good) {
                    if (lane == 0) atomicOr(&g_status, ST_PRODUCER_TIMEOUT);
                    ok = false;
                    break;
                }
                char* st = stage_smem + size_t(s) * lay.bytes;
                const bool live = sc.slot > 0 && sc.h >= 0 && sc.h < L;
                if (lane == 0) {
                    *reinterpret_cast<ProgScalars*>(st + lay.sc) = sc;
                    if (live) {
                        uint32_t bytes = ck_bytes(R) + 2u * uint32_t(sc.h) * 256u + uint32_t(L) * 4u + 3u * 256u;
                        if (KDA) bytes += uint32_t(sc.h) * 256u + 512u + 256u + 512u;
                        mbar_arrive_expect_tx(full + s, bytes);
                    } else {
                        mbar_arrive(full + s);
                    }
                }
                __syncwarp();
                if (live) {
                    const int64_t sh = int64_t(sc.slot) * HV + sc.hv;
                    const char* mrow = reinterpret_cast<const char*>(P.mixed + int64_t(sc.n) * MIX);
                    const int hk = sc.hv / gqa;
                    const uint32_t hb = uint32_t(sc.h) * 256u;
                    switch (lane) {
                        case 0: bulk_g2s(st, head_base(P.ssm, P.d.SS, sc.slot, sc.hv), ck_bytes(R), full + s); break;
                        case 1: if (hb) bulk_g2s(st + lay.kb, P.Kbuf + sh * L * KD, hb, full + s); break;
                        case 2: if (hb) bulk_g2s(st + lay.ub, P.Ubuf + sh * L * VD, hb, full + s); break;
                        case 3: bulk_g2s(st + lay.w, P.Wbuf + sh * L, uint32_t(L) * 4u, full + s); break;
                        case 4: bulk_g2s(st + lay.q, mrow + hk * 256, 256u, full + s); break;
                        case 5: bulk_g2s(st + lay.k, mrow + (H + hk) * 256, 256u, full + s); break;
                        case 6: bulk_g2s(st + lay.v, mrow + (2 * H + sc.hv) * 256, 256u, full + s); break;
                        case 7: if (KDA && hb) bulk_g2s(st + lay.gb, P.Gbuf + sh * L * KD, hb, full + s); break;
                        case 8: if (KDA) bulk_g2s(st + lay.pb, P.Pbuf + sh * KD, 512u, full + s); break;
                        case 9: if (KDA) bulk_g2s(st + lay.a, P.a + (int64_t(sc.n) * HV + sc.hv) * KD, 256u, full + s); break;
                        case 10: if (KDA) bulk_g2s(st + lay.dtb, P.dt_bias + int64_t(sc.hv) * KD, 512u, full + s); break;
                        default: break;
                    }
                }
            }
        }
        // Leave only after every stage this warp armed has been consumed (bounded): no copy of this CTA is then in flight.
        if (lane == 0) {
            const int last = ok ? nit : 0;
            for (int s = 0; s < nstages && s < last; ++s) {
                const int uses = (last - 1 - s) / nstages + 1;            // fills of stage s
                if (!mbar_wait_bounded(empty + s, uint32_t(uses - 1) & 1u)) {
                    atomicOr(&g_status, ST_PRODUCER_TIMEOUT);
                    break;
                }
            }
        }
        return;
    }

    // ================= consumers: group g takes programs g, g + NG, ... =================
    const int g = (warp - 1) >> 2;
    const int t = tid - 32 - g * GT;
    const int bar = 1 + g;
    const GroupScratch gs = carve_scratch(scratch0 + g * SCRATCH_BYTES);
    for (int i = g; i < nit; i += NG) {
        const int s = i % nstages;
        const uint32_t u = uint32_t(i / nstages);
        const bool got = mbar_wait_bounded(full + s, u & 1u);
        if (!group_all(bar, GT, got)) {                 // uniform decision: nobody enters the body unless all saw the data
            if (t == 0) atomicOr(&g_status, ST_CONSUMER_TIMEOUT);
            return;
        }
        char* st = stage_smem + size_t(s) * lay.bytes;
        const ProgScalars sc = *reinterpret_cast<const ProgScalars*>(st + lay.sc);
        if (sc.slot > 0 && sc.h >= 0 && sc.h < L) {
            step_body<R, KDA>(P, sc, st, lay, gs, t, bar);
        } else {
            const int p = bid + i * grid;
            if (t < 64) reinterpret_cast<uint32_t*>(P.o)[int64_t(p) * 64 + t] = 0u;
        }
        fence_async_smem();                              // generic-proxy accesses to the stage before the next bulk copy lands
        mbar_arrive(empty + s);
    }
}

// 0 = pipelined (default), 1 = direct
static int g_step_impl = 0;

template <int R, bool KDA>
static int launch_step(const StepParams& P, cudaStream_t st) {
    const StageLayout lay = stage_layout(P.d.L, R, KDA);
    if (g_step_impl == 1) {
        const size_t smem = size_t(lay.bytes) + SCRATCH_BYTES;
        int rc = ensure_smem((const void*)step_direct_kernel<R, KDA>, smem);
        if (rc) return rc;
        step_direct_kernel<R, KDA><<<unsigned(P.N) * P.d.HV, GT, smem, st>>>(P);
        return finish_launch();
    }
    constexpr int NG = 2;
    const size_t budget = 227 * 1024;
    const size_t fixed = size_t(NG) * SCRATCH_BYTES + 2 * 16 * sizeof(uint64_t);
    int nstages = int((budget - fixed) / size_t(lay.bytes));
    if (nstages > 16) nstages = 16;
    if (nstages < 2) return LQ_ERR_UNSUPPORTED;
    const size_t smem = size_t(nstages) * lay.bytes + size_t(NG) * SCRATCH_BYTES + 2 * size_t(nstages) * sizeof(uint64_t);
    int rc = ensure_smem((const void*)step_pipelined_kernel<R, KDA, NG>, smem);
    if (rc) return rc;
    const int nprog = P.N * P.d.HV;
    const int grid = nprog < device_sm_count() ? nprog : device_sm_count();
    step_pipelined_kernel<R, KDA, NG><<<grid, 32 + NG * GT, smem, st>>>(P, nstages);
    return finish_launch();
}

static int step_common(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                       int32_t* hcnt, const void* mixed, const void* a, const void* b, const float* A_log,
                       const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale, float glb, bool kda,
                       void* stream) {
    int rc = check_dims(d);
    if (rc) return rc;
    if (!ssm || !Kbuf || !Ubuf || !Wbuf || !Pbuf || !hcnt || !A_log || !dt_bias || (kda && !Gbuf)) return LQ_ERR_NULL;
    if (N < 0) return LQ_ERR_RANGE;
    if (N == 0) return LQ_OK;
    if (!mixed || !a || !b || !idx || !o) return LQ_ERR_NULL;
    const uintptr_t al = reinterpret_cast<uintptr_t>(ssm) | reinterpret_cast<uintptr_t>(Kbuf) | reinterpret_cast<uintptr_t>(Ubuf) |
                         reinterpret_cast<uintptr_t>(Wbuf) | reinterpret_cast<uintptr_t>(mixed) | reinterpret_cast<uintptr_t>(o) |
                         (kda ? (reinterpret_cast<uintptr_t>(Gbuf) | reinterpret_cast<uintptr_t>(Pbuf) |
                                 reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(dt_bias)) : 0);
    if (al & 15) return LQ_ERR_ALIGN;
    StepParams P;
    P.d = *d; P.ssm = (char*)ssm; P.Kbuf = (uint16_t*)Kbuf; P.Ubuf = (uint16_t*)Ubuf; P.Wbuf = Wbuf; P.Pbuf = Pbuf;
    P.Gbuf = (uint16_t*)Gbuf; P.hcnt = hcnt; P.mixed = (const uint16_t*)mixed; P.a = (const uint16_t*)a;
    P.b = (const uint16_t*)b; P.A_log = A_log; P.dt_bias = dt_bias; P.idx = idx; P.o = (uint16_t*)o; P.N = N;
    P.scale = scale > 0.f ? scale : 1.0f / sqrtf(float(d->K));
    P.glb = glb;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (kda) return d->R == 4 ? launch_step<4, true>(P, s) : launch_step<8, true>(P, s);
    return d->R == 4 ? launch_step<4, false>(P, s) : launch_step<8, false>(P, s);
}

}  // namespace lq

extern "C" int lq_set_option(const char* name, int32_t value) {
    if (!name) return LQ_ERR_NULL;
    if (strcmp(name, "step_impl") == 0) {
        if (value != 0 && value != 1) return LQ_ERR_RANGE;
        lq::g_step_impl = value;
        return LQ_OK;
    }
    return LQ_ERR_UNSUPPORTED;
}

extern "C" int lq_gdn_step(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                           const void* mixed, const void* a, const void* b, const float* A_log, const float* dt_bias,
                           const int32_t* idx, void* o, int32_t N, float scale, void* stream) {
    return lq::step_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, nullptr, hcnt, mixed, a, b, A_log, dt_bias, idx, o, N, scale, 0.f,
                           false, stream);
}

extern "C" int lq_kda_step(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                           int32_t* hcnt, const void* mixed, const void* a, const void* b, const float* A_log,
                           const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale,
                           float gate_lower_bound, void* stream) {
    return lq::step_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, idx, o, N, scale,
                           gate_lower_bound, true, stream);
}
