// Window-flush kernel (sm_100a): rebuild -> rank-R subspace iteration -> residual -> smoothing scales -> INT8.
//
// Persistent CTAs of 256 threads.  Every CTA scans the due flags of all (row, head) programs of the call, ranks the
// due ones in a fixed order and keeps the ranks congruent to its block index, so the work is balanced to +-1 head
// per CTA whatever the pattern of full windows, and the launch shape never depends on device data.
// The rebuilt 128 x 128 state B and the residual E stay in shared memory as fp32 for the whole program.
#include "lq_linalg.cuh"

namespace lq {

constexpr int TS = 136;          // row stride (bf16 elements) of the staged window tiles: 272 B keeps ldmatrix rows conflict-free

struct FlushSmem {
    float* B;        // [128][LDB]
    uint16_t* Kt;    // [Lp][TS] window keys, bf16 as stored (rows L.. zero)
    uint16_t* Ut;    // [Lp][TS] window values, bf16 as stored (rows L.. zero)
    float* tab;      // KDA: [L][128] scale of key (j, c): w_j D_j[c]
    float* scr;      // [128][R]   (aliases the window tiles: used after the rebuild only)
    float* colpart;  // [16][128]  (aliases the window tiles)
    float* Uo;       // [R][128] old U^T (KDA: times pc)
    float* Qo;       // [R][128] old Q^T
    float* Un;       // [128][R] P / new U
    float* Qn;       // [128][R] Q
    float* Msm;      // [R][R]
    float* sk;       // [128] column scale operand of the dequant (KDA: Sk pc); later 1 / Sk_new
    float* sv;       // [128]
    float* pc;       // [128]
    float* w;        // [64]
    int* wcnt;       // [8]
    int* dlist;      // [maxd]
};

__host__ __device__ inline int flush_lp(int L) { return (L + 15) & ~15; }
// floats of the region shared by the window tiles (rebuild) and scr + colpart (afterwards)
template <int R>
__host__ __device__ inline int flush_region_floats(int L) {
    const int tiles = flush_lp(L) * TS;                     // two bf16 tiles = Lp * TS floats
    const int later = 128 * R + 16 * 128;
    return tiles > later ? tiles : later;
}
template <int R>
__host__ __device__ inline size_t flush_smem_floats(int L, int maxd, bool kda) {
    return size_t(128) * LDB + flush_region_floats<R>(L) + (kda ? size_t(L) * 128 : 0) + 2 * R * 128 + 2 * 128 * R + 64 +
           3 * 128 + 64 + 8 + maxd;
}

// ---- warp-level tensor-core helpers (legacy mma.sync path; the rebuild is a real 128 x 128 x L product) ----
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = uint32_t(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// x (fp32) ~ hi + lo as two bf16 pieces (16 mantissa bits, relative error 2^-17): the split the reference uses for the
// same operand (reference leapquant/kernels.py:1508-1511).  The tensor pipe bounds the rebuild, so a third piece
// would cost 50 % more time for accuracy far below the INT8 step.
__device__ __forceinline__ void split2(float x, float& hi, float& lo) {
    hi = round_bf16(x);
    lo = round_bf16(x - hi);
}

#ifdef LQ_TRACE
static __device__ long long g_ftrace[320 * 16];
#define LQ_FSTAMP(k) do { if (tid == 0) { const long long tn = clock64(); facc[k] += tn - flast; flast = tn; } } while (0)
#else
#define LQ_FSTAMP(k) do { } while (0)
#endif

template <int R, bool KDA>
__global__ void __launch_bounds__(NT_LA, (R == 4 ? 2 : 1))
flush_kernel(lq_dims d, char* __restrict__ ssm, const uint16_t* __restrict__ Kbuf, const uint16_t* __restrict__ Ubuf,
             float* __restrict__ Wbuf, float* __restrict__ Pbuf, uint16_t* __restrict__ Gbuf, int32_t* __restrict__ hcnt,
             const float* __restrict__ Q0, const int32_t* __restrict__ idx, int N, int iters, int maxd) {
    extern __shared__ __align__(16) float smem[];
    FlushSmem s;
    const int Lp = flush_lp(d.L);
    {
        float* p = smem;
        s.B = p; p += 128 * LDB;
        s.Kt = reinterpret_cast<uint16_t*>(p);
        s.Ut = s.Kt + Lp * TS;
        s.scr = p;
        s.colpart = p + 128 * R;
        p += flush_region_floats<R>(d.L);
        s.tab = p; p += KDA ? d.L * 128 : 0;
        s.Uo = p; p += R * 128;
        s.Qo = p; p += R * 128;
        s.Un = p; p += 128 * R;
        s.Qn = p; p += 128 * R;
        s.Msm = p; p += 64;
        s.sk = p; p += 128;
        s.sv = p; p += 128;
        s.pc = p; p += 128;
        s.w = p; p += 64;
        s.wcnt = reinterpret_cast<int*>(p); p += 8;
        s.dlist = reinterpret_cast<int*>(p);
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, bid = blockIdx.x;
    const int L = d.L, HV = d.HV;

    // ---------------- balanced compaction of the due programs ----------------
    const int total = N * HV;
    const int per_warp = ((total + 7) / 8 + 31) & ~31;
    const int wbeg = warp * per_warp, wend = min(wbeg + per_warp, total);
    auto due_at = [&](int i, int& q) -> bool {
        if (i >= wend) return false;
        const int n = i / HV, hv = i - n * HV;
        const int slot = idx[n];
        if (slot <= 0 || slot >= d.NS) return false;
        q = slot * HV + hv;
        return hcnt[q] == L;
    };
    // counting pass, 16 flags per lane in flight: all slot loads, then all counter loads, then the ballots
    // (a loop of dependent load pairs made a launch that finds nothing due cost ~10 us)
    int cnt = 0;
    constexpr int UN = 16;
    for (int b0 = wbeg; b0 < wend; b0 += 32 * UN) {
        int sl[UN], hc[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int i = b0 + 32 * u + lane;
            sl[u] = (i < wend) ? idx[i / HV] : 0;
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int i = b0 + 32 * u + lane;
            const bool ok = sl[u] > 0 && sl[u] < d.NS;
            hc[u] = ok ? hcnt[sl[u] * HV + (i % HV)] : -1;
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) cnt += __popc(__ballot_sync(0xffffffffu, hc[u] == L));
    }
    if (lane == 0) s.wcnt[warp] = cnt;
    __syncthreads();
    int rank = 0, ndue = 0;
#pragma unroll
    for (int w2 = 0; w2 < 8; ++w2) {
        const int c2 = s.wcnt[w2];
        rank += (w2 < warp) ? c2 : 0;
        ndue += c2;
    }
    if (ndue == 0) return;
    if (cnt > 0) {
        const uint32_t lt = (1u << lane) - 1u;
        for (int b0 = wbeg; b0 < wend; b0 += 32) {
            int q = 0;
            const bool f = due_at(b0 + lane, q);
            const uint32_t m = __ballot_sync(0xffffffffu, f);
            const int r = rank + __popc(m & lt);
            if (f && (r % G) == bid && (r / G) < maxd) s.dlist[r / G] = q;
            rank += __popc(m);
        }
    }
    const int mine = (ndue > bid) ? min((ndue - bid + G - 1) / G, maxd) : 0;
    __syncthreads();

    const int ty = tid >> 4, tx = tid & 15, v0 = ty * 8;
#ifdef LQ_TRACE
    long long facc[16] = {0}, flast = clock64();
#endif

    for (int k = 0; k < mine; ++k) {
        LQ_FSTAMP(0);
        const int q = s.dlist[k];
        const int slot = q / HV, hv = q - slot * HV;
        const int64_t sh = q;
        char* base = head_base(ssm, d.SS, slot, hv);
        float p = 1.f;
        if (!KDA) p = fmaxf(Pbuf[sh], PNMIN);

        // ---- stage A: operands to shared memory ----
        if (tid < L) s.w[tid] = Wbuf[sh * L + tid];
        if (tid < 128) {
            const float pcv = KDA ? expf(Pbuf[sh * KD + tid]) : 1.f;
            s.pc[tid] = pcv;
            s.sk[tid] = reinterpret_cast<const float*>(base + CK_SK)[tid] * pcv;
            s.sv[tid] = reinterpret_cast<const float*>(base + CK_SV)[tid];
        }
        {
            const uint16_t* uq = reinterpret_cast<const uint16_t*>(base + CK_UQ);
            for (int i = tid; i < R * 128; i += NT_LA) {
                const int r = i >> 7, c = i & 127;
                s.Uo[i] = f16_to_f(uq[r * (KD + VD) + c]);
                s.Qo[i] = f16_to_f(uq[r * (KD + VD) + KD + c]);
            }
        }
        LQ_FSTAMP(1);
        // window rows as stored (bf16), 16 bytes at a time into the padded tiles; rows L .. Lp-1 are zero
        {
            const uint4* kb = reinterpret_cast<const uint4*>(Kbuf + sh * L * KD);
            const uint4* ub = reinterpret_cast<const uint4*>(Ubuf + sh * L * VD);
            for (int i = tid; i < Lp * 16; i += NT_LA) {
                const int j = i >> 4, c8 = i & 15;
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(s.Kt + j * TS + c8 * 8) = j < L ? kb[i] : z;
                *reinterpret_cast<uint4*>(s.Ut + j * TS + c8 * 8) = j < L ? ub[i] : z;
            }
        }
        __syncthreads();
        if (KDA && tid < 128) {
            // key scale w_j D_j[c] with D_{L-1} = 1, D_j = D_{j+1} e_{j+1}; old U^T times pc
            float dcur = 1.f;
            const uint16_t* gb = Gbuf + sh * L * KD + tid;
            for (int j = L - 1; j >= 0; --j) {
                s.tab[j * 128 + tid] = s.w[j] * dcur;
                dcur *= f16_to_f(gb[j * KD]);
            }
            const float pcv = s.pc[tid];
#pragma unroll
            for (int r = 0; r < R; ++r) s.Uo[r * 128 + tid] *= pcv;
        }
        if (KDA) __syncthreads();

        LQ_FSTAMP(2);
        // ---- stage B: B = deq(checkpoint) * decay + sum_j (w_j u_j) k_j^T on the tensor cores (mma.sync bf16, fp32 accumulate).
        //      The operand that carries an fp32 scale (GDN: w_j u_j[v]; KDA: w_j D_j[c] k_j[c]) is the A operand, built in
        //      registers as two bf16 pieces (hi + lo, 16 mantissa bits); the other one is bf16 as stored and comes
        //      through ldmatrix.  GDN computes B[v][c] with M = v; KDA computes the transpose with M = c. ----
        {
            const int r = lane >> 2, q2 = (lane & 3) * 2;
            const int m0 = warp * 16;                           // this warp's 16 rows of the product (v for GDN, c for KDA)
            const uint16_t* At = KDA ? s.Kt : s.Ut;             // A source tile [j][m]
            const uint16_t* Bt = KDA ? s.Ut : s.Kt;             // B source tile [j][n]
            float acc[16][4];
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
            // this thread's INT8 codes, fetched now so that their latency hides behind the products:
            // accumulator (nt, hrow) covers (mm, nn), (mm, nn + 1) with mm = m0 + r + 8 hrow, nn = 8 nt + q2
            const uint8_t* cb = reinterpret_cast<const uint8_t*>(base + CK_CODES);
            uint32_t cpre[16];                                 // [nt]: low half hrow 0, high half hrow 1; two codes each
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) {
                uint32_t pk = 0;
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int mm = m0 + r + 8 * hrow, nn = 8 * nt + q2;
                    uint32_t two;
                    if (!KDA) two = *reinterpret_cast<const uint16_t*>(cb + mm * KD + nn);
                    else two = uint32_t(cb[nn * KD + mm]) | (uint32_t(cb[(nn + 1) * KD + mm]) << 8);
                    pk |= two << (16 * hrow);
                }
                cpre[nt] = pk;
            }
            LQ_FSTAMP(14);
            for (int ks = 0; ks < Lp; ks += 16) {
                uint32_t ah[4], al[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {                   // a0: (r, k..k+1)  a1: (r+8, ..)  a2: (r, k+8..)  a3: (r+8, k+8..)
                    const int m = m0 + r + 8 * (e & 1);
                    const int j = ks + q2 + 8 * (e >> 1);
                    float x0 = bf16_to_f(At[j * TS + m]), x1 = bf16_to_f(At[(j + 1) * TS + m]);
                    if (KDA) {
                        x0 *= (j < L) ? s.tab[j * 128 + m] : 0.f;
                        x1 *= (j + 1 < L) ? s.tab[(j + 1) * 128 + m] : 0.f;
                    } else {
                        x0 *= (j < L) ? s.w[j] : 0.f;
                        x1 *= (j + 1 < L) ? s.w[j + 1] : 0.f;
                    }
                    float h0, l0, h1, l1;
                    split2(x0, h0, l0);
                    split2(x1, h1, l1);
                    ah[e] = f2_to_bf16x2(h0, h1);
                    al[e] = f2_to_bf16x2(l0, l1);
                }
                // ldmatrix row address of this lane: matrix lane >> 3 = (k half) + 2 (n-tile of the pair), row lane & 7
                const uint16_t* brow = Bt + (ks + (lane & 7) + 8 * ((lane >> 3) & 1)) * TS + 8 * (lane >> 4);
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    uint32_t bf[4];
                    ldmatrix_x4_trans(bf, brow + np * 16);
                    mma_bf16_16816(acc[2 * np], ah, bf[0], bf[1]);
                    mma_bf16_16816(acc[2 * np], al, bf[0], bf[1]);
                    mma_bf16_16816(acc[2 * np + 1], ah, bf[2], bf[3]);
                    mma_bf16_16816(acc[2 * np + 1], al, bf[2], bf[3]);
                }
            }
            LQ_FSTAMP(13);
            // add the dequantised checkpoint and store B[v][c]; accumulator (e, nt): row m0 + r + 8 (e >> 1), col 8 nt + q2 + (e & 1)
            const float pq = KDA ? (1.0f / QMAX) : (p / QMAX);
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int mm = m0 + r + 8 * hrow, nn = 8 * nt + q2;
                    const uint32_t cw = (cpre[nt] >> (16 * hrow)) & 0xffffu;
                    if (!KDA) {                                 // (v, c) = (mm, nn), (mm, nn + 1): two adjacent codes
                        const float svr = s.sv[mm] * pq;
                        const float f0 = float(int(int8_t(cw & 0xff))), f1 = float(int(int8_t(cw >> 8)));
                        const float o0 = (f0 * svr) * s.sk[nn] + acc[nt][2 * hrow];
                        const float o1 = (f1 * svr) * s.sk[nn + 1] + acc[nt][2 * hrow + 1];
                        *reinterpret_cast<float2*>(s.B + mm * LDB + nn) = make_float2(o0, o1);
                    } else {                                    // (c, v) = (mm, nn), (mm, nn + 1): codes of rows nn, nn + 1
                        const float f0 = float(int(int8_t(cw & 0xff))), f1 = float(int(int8_t(cw >> 8)));
                        const float skc = s.sk[mm];
                        s.B[nn * LDB + mm] = (f0 * (s.sv[nn] * pq)) * skc + acc[nt][2 * hrow];
                        s.B[(nn + 1) * LDB + mm] = (f1 * (s.sv[nn + 1] * pq)) * skc + acc[nt][2 * hrow + 1];
                    }
                }
            }
        }
        __syncthreads();                                        // the window tiles are dead: scr / colpart may use the region
        LQ_FSTAMP(3);
        for (int i = tid; i < 128 * R; i += NT_LA) s.Qn[i] = round_f16(Q0[i]);
        __syncthreads();

        LQ_FSTAMP(4);
        // ---- stage C: subspace iteration on T = B + p Q_old U_old^T ----
        // P = T^T Q  (rounded to fp16 values)
        coldot<R>(s.B, s.Qn, s.Un, s.scr, tid);
        factor_gram<R>(s.Qo, s.Qn, s.Msm, tid);
        factor_apply<R, true>(s.Uo, s.Msm, s.Un, p, tid);
        LQ_FSTAMP(5);
        for (int it = 0; it < iters; ++it) {
            rowdot<R>(s.B, s.Un, s.Qn, s.scr, tid);          // Q = T P
            factor_gram<R>(s.Uo, s.Un, s.Msm, tid);
            factor_apply<R, false>(s.Qo, s.Msm, s.Qn, p, tid);
            LQ_FSTAMP(6);
            cholqr2_f16<R>(s.Qn, tid);
            LQ_FSTAMP(7);
            coldot<R>(s.B, s.Qn, s.Un, s.scr, tid);          // P = T^T Q
            factor_gram<R>(s.Qo, s.Qn, s.Msm, tid);
            factor_apply<R, true>(s.Uo, s.Msm, s.Un, p, tid);
        }

        LQ_FSTAMP(8);
        // ---- stage D: new factors to the checkpoint ----
        {
            uint16_t* uq = reinterpret_cast<uint16_t*>(base + CK_UQ);
            for (int i = tid; i < R * 128; i += NT_LA) {
                const int r = i >> 7, c = i & 127;
                uq[r * (KD + VD) + c] = f_to_f16(s.Un[c * R + r]);
                uq[r * (KD + VD) + KD + c] = f_to_f16(s.Qn[c * R + r]);
            }
        }

        LQ_FSTAMP(9);
        // ---- stage E: residual E = B + p Q_old U_old^T - Q U^T in place, column sums of |E| ----
        {
            float colp[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) colp[c] = 0.f;
            float uo[R][8], un[R][8];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uo[r][c] = s.Uo[r * 128 + 4 * tx + c];
                    uo[r][4 + c] = s.Uo[r * 128 + 64 + 4 * tx + c];
                    un[r][c] = s.Un[(4 * tx + c) * R + r];
                    un[r][4 + c] = s.Un[(64 + 4 * tx + c) * R + r];
                }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float qo[R], qn[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    qo[r] = s.Qo[r * 128 + v0 + i];
                    qn[r] = s.Qn[(v0 + i) * R + r];
                }
                float4 ba = *reinterpret_cast<const float4*>(s.B + (v0 + i) * LDB + 4 * tx);
                float4 bb = *reinterpret_cast<const float4*>(s.B + (v0 + i) * LDB + 64 + 4 * tx);
                float e[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float t1 = 0.f, t2 = 0.f;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        t1 = fmaf(qo[r], uo[r][c], t1);
                        t2 = fmaf(qn[r], un[r][c], t2);
                    }
                    e[c] = fmaf(p, t1, e[c]) - t2;
                    colp[c] += fabsf(e[c]);
                }
                *reinterpret_cast<float4*>(s.B + (v0 + i) * LDB + 4 * tx) = make_float4(e[0], e[1], e[2], e[3]);
                *reinterpret_cast<float4*>(s.B + (v0 + i) * LDB + 64 + 4 * tx) = make_float4(e[4], e[5], e[6], e[7]);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                s.colpart[ty * 128 + 4 * tx + c] = colp[c];
                s.colpart[ty * 128 + 64 + 4 * tx + c] = colp[4 + c];
            }
        }
        __syncthreads();
        if (tid < 128) {
            float m = 0.f;
#pragma unroll
            for (int t2 = 0; t2 < 16; ++t2) m += s.colpart[t2 * 128 + tid];
            m *= (1.0f / float(VD));
            const float skn = fmaxf(sqrtf(m), EPS);
            reinterpret_cast<float*>(base + CK_SK)[tid] = skn;
            s.sk[tid] = 1.0f / skn;                           // reciprocal of the STORED scale
        }
        __syncthreads();

        LQ_FSTAMP(10);
        // ---- stage F: row scales and INT8 codes ----
        {
            const int l8 = lane & 7, g = lane >> 3;
            uint32_t* codes = reinterpret_cast<uint32_t*>(base + CK_CODES);
            float* svg = reinterpret_cast<float*>(base + CK_SV);
            float rk[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 r4 = *reinterpret_cast<const float4*>(s.sk + i * 32 + l8 * 4);
                rk[4 * i + 0] = r4.x; rk[4 * i + 1] = r4.y; rk[4 * i + 2] = r4.z; rk[4 * i + 3] = r4.w;
            }
#pragma unroll 1
            for (int it = 0; it < 4; ++it) {
                const int row = warp * 16 + it * 4 + g;
                float x[16];
                float rmax = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 ev = *reinterpret_cast<const float4*>(s.B + row * LDB + i * 32 + l8 * 4);
                    x[4 * i + 0] = ev.x * rk[4 * i + 0];
                    x[4 * i + 1] = ev.y * rk[4 * i + 1];
                    x[4 * i + 2] = ev.z * rk[4 * i + 2];
                    x[4 * i + 3] = ev.w * rk[4 * i + 3];
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) rmax = fmaxf(rmax, fabsf(x[i]));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 4));
                const float svv = fmaxf(rmax, EPS);
                const float rm = QMAX * __frcp_rn(svv);
                if (l8 == 0) svg[row] = svv;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    codes[row * 32 + i * 8 + l8] = pack4(rne_code(x[4 * i + 0], rm), rne_code(x[4 * i + 1], rm),
                                                         rne_code(x[4 * i + 2], rm), rne_code(x[4 * i + 3], rm));
            }
        }
        LQ_FSTAMP(11);
        // ---- stage G: window reset ----
        if (tid < L) Wbuf[sh * L + tid] = 0.f;
        if (KDA) {
            if (tid < 128) Pbuf[sh * KD + tid] = 0.f;
            uint32_t* g32 = reinterpret_cast<uint32_t*>(Gbuf + sh * L * KD);
            for (int i = tid; i < L * KD / 2; i += NT_LA) g32[i] = 0x3C003C00u;
        } else if (tid == 0) {
            Pbuf[sh] = 1.f;
        }
        if (tid == 0) hcnt[sh] = 0;
        __syncthreads();
        LQ_FSTAMP(12);
    }
#ifdef LQ_TRACE
    if (tid == 0 && blockIdx.x < 320) for (int i = 0; i < 16; ++i) g_ftrace[blockIdx.x * 16 + i] = facc[i];
    if (tid == 0 && blockIdx.x < 320) g_ftrace[blockIdx.x * 16 + 15] = mine;
#endif
}

template <int R, bool KDA>
static int launch_flush(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                        int32_t* hcnt, const float* Q0, const int32_t* idx, int N, int iters, cudaStream_t st) {
    const int total = N * d->HV;
    // two CTAs per SM when the shared memory of one allows it (R = 4): a flush is a chain of short phases, and a second
    // head in flight on the SM hides most of their latency
    int per_sm = 1;
    if (R == 4) {
        const int g2 = min(2 * device_sm_count(), total);
        const size_t s2 = sizeof(float) * flush_smem_floats<R>(d->L, (total + g2 - 1) / g2 + 1, KDA);
        if (s2 <= 113 * 1024) per_sm = 2;
    }
    const int G = min(per_sm * device_sm_count(), total);
    const int maxd = (total + G - 1) / G + 1;
    const size_t smem = sizeof(float) * flush_smem_floats<R>(d->L, maxd, KDA);
    if (smem > 227 * 1024) return LQ_ERR_UNSUPPORTED;
    int rc = ensure_smem((const void*)flush_kernel<R, KDA>, smem);
    if (rc) return rc;
    flush_kernel<R, KDA><<<G, NT_LA, smem, st>>>(*d, (char*)ssm, (const uint16_t*)Kbuf, (const uint16_t*)Ubuf, Wbuf, Pbuf,
                                                 (uint16_t*)Gbuf, hcnt, Q0, idx, N, iters, maxd);
    return finish_launch();
}

}  // namespace lq

using namespace lq;

#ifdef LQ_TRACE
extern "C" int lq_debug_read_ftrace(long long* out, int n) {
    return cudaMemcpyFromSymbol(out, lq::g_ftrace, sizeof(long long) * n) == cudaSuccess ? 0 : -5;
}
#endif

extern "C" int lq_flush(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                        int32_t* hcnt, const float* Q0, const int32_t* idx, int32_t N, int32_t kda, int32_t iters,
                        void* stream) {
    int rc = check_dims(d);
    if (rc) return rc;
    if (!ssm || !Kbuf || !Ubuf || !Wbuf || !Pbuf || !hcnt || !Q0 || (N > 0 && !idx) || (kda && !Gbuf)) return LQ_ERR_NULL;
    if (N < 0 || iters < 0) return LQ_ERR_RANGE;
    if (N == 0) return LQ_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->R == 4)
        return kda ? launch_flush<4, true>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st)
                   : launch_flush<4, false>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st);
    return kda ? launch_flush<8, true>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st)
               : launch_flush<8, false>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st);
}
