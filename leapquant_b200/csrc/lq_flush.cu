// Window-flush kernel (sm_100a): rebuild -> rank-R subspace iteration -> residual -> smoothing scales -> INT8.
//
// Persistent CTAs of 256 threads.  Every CTA scans the due flags of all (row, head) programs of the call, ranks the
// due ones in a fixed order and keeps the ranks congruent to its block index, so the work is balanced to +-1 head
// per CTA whatever the pattern of full windows, and the launch shape never depends on device data.
// The rebuilt 128 x 128 state B and the residual E stay in shared memory as fp32 for the whole program.
#include "lq_linalg.cuh"

namespace lq {

struct FlushSmem {
    float* B;        // [128][LDB]
    float* Kf;       // [L][128] window keys (KDA: times w_j D_j)
    float* WU;       // [L][128] w_j u_j (KDA: u_j)
    float* Uo;       // [R][128] old U^T (KDA: times pc)
    float* Qo;       // [R][128] old Q^T
    float* Un;       // [128][R] P / new U
    float* Qn;       // [128][R] Q
    float* scr;      // [128][R]
    float* Msm;      // [R][R]
    float* sk;       // [128] column scale operand of the dequant (KDA: Sk pc); later 1 / Sk_new
    float* sv;       // [128]
    float* pc;       // [128]
    float* w;        // [64]
    float* colpart;  // [16][128]
    int* wcnt;       // [8]
    int* dlist;      // [maxd]
};

template <int R>
__host__ __device__ inline size_t flush_smem_floats(int L, int maxd) {
    return size_t(128) * LDB + 2 * size_t(L) * 128 + 2 * R * 128 + 3 * 128 * R + 64 + 3 * 128 + 64 + 16 * 128 + 8 + maxd;
}

template <int R, bool KDA>
__global__ void __launch_bounds__(NT_LA, 1)
flush_kernel(lq_dims d, char* __restrict__ ssm, const uint16_t* __restrict__ Kbuf, const uint16_t* __restrict__ Ubuf,
             float* __restrict__ Wbuf, float* __restrict__ Pbuf, uint16_t* __restrict__ Gbuf, int32_t* __restrict__ hcnt,
             const float* __restrict__ Q0, const int32_t* __restrict__ idx, int N, int iters, int maxd) {
    extern __shared__ __align__(16) float smem[];
    FlushSmem s;
    {
        float* p = smem;
        s.B = p; p += 128 * LDB;
        s.Kf = p; p += d.L * 128;
        s.WU = p; p += d.L * 128;
        s.Uo = p; p += R * 128;
        s.Qo = p; p += R * 128;
        s.Un = p; p += 128 * R;
        s.Qn = p; p += 128 * R;
        s.scr = p; p += 128 * R;
        s.Msm = p; p += 64;
        s.sk = p; p += 128;
        s.sv = p; p += 128;
        s.pc = p; p += 128;
        s.w = p; p += 64;
        s.colpart = p; p += 16 * 128;
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
    int cnt = 0;
    for (int b0 = wbeg; b0 < wend; b0 += 32) {
        int q;
        const bool f = due_at(b0 + lane, q);
        cnt += __popc(__ballot_sync(0xffffffffu, f));
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

    for (int k = 0; k < mine; ++k) {
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
        __syncthreads();
        {
            const uint32_t* kb = reinterpret_cast<const uint32_t*>(Kbuf + sh * L * KD);
            const uint32_t* ub = reinterpret_cast<const uint32_t*>(Ubuf + sh * L * VD);
            for (int i = tid; i < L * 64; i += NT_LA) {
                const int j = i >> 6;
                const float2 kk = bf16x2_to_f2(kb[i]);
                const float2 uu = bf16x2_to_f2(ub[i]);
                const float wj = KDA ? 1.f : s.w[j];
                *reinterpret_cast<float2*>(s.Kf + 2 * i) = kk;
                *reinterpret_cast<float2*>(s.WU + 2 * i) = make_float2(wj * uu.x, wj * uu.y);
            }
        }
        __syncthreads();
        if (KDA && tid < 128) {
            // decayed keys w_j D_j k_j with D_{L-1} = 1, D_j = D_{j+1} e_{j+1}; old U^T times pc
            float dcur = 1.f;
            const uint16_t* gb = Gbuf + sh * L * KD + tid;
            for (int j = L - 1; j >= 0; --j) {
                s.Kf[j * 128 + tid] *= s.w[j] * dcur;
                dcur *= f16_to_f(gb[j * KD]);
            }
            const float pcv = s.pc[tid];
#pragma unroll
            for (int r = 0; r < R; ++r) s.Uo[r * 128 + tid] *= pcv;
        }
        if (KDA) __syncthreads();

        // ---- stage B: B = deq(checkpoint) * decay + sum_j (w_j u_j) k_j^T, 8 x 8 outputs per thread ----
        {
            float acc[8][8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[i][c] = 0.f;
#pragma unroll 2
            for (int j = 0; j < L; ++j) {
                const float4 ua = *reinterpret_cast<const float4*>(s.WU + j * 128 + v0);
                const float4 ub = *reinterpret_cast<const float4*>(s.WU + j * 128 + v0 + 4);
                const float4 ka = *reinterpret_cast<const float4*>(s.Kf + j * 128 + 4 * tx);
                const float4 kb = *reinterpret_cast<const float4*>(s.Kf + j * 128 + 64 + 4 * tx);
                const float uu[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
                const float kk[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int c = 0; c < 8; ++c) acc[i][c] = fmaf(uu[i], kk[c], acc[i][c]);
            }
            const uint32_t* cw = reinterpret_cast<const uint32_t*>(base + CK_CODES);
            float skl[8];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                skl[c] = s.sk[4 * tx + c];
                skl[4 + c] = s.sk[64 + 4 * tx + c];
            }
            const float pq = KDA ? (1.0f / QMAX) : (p / QMAX);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float svr = s.sv[v0 + i] * pq;
                float f[8];
                s8x4_to_f4(cw[(v0 + i) * 32 + tx], f[0], f[1], f[2], f[3]);
                s8x4_to_f4(cw[(v0 + i) * 32 + 16 + tx], f[4], f[5], f[6], f[7]);
                float o[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) o[c] = (f[c] * svr) * skl[c] + acc[i][c];
                *reinterpret_cast<float4*>(s.B + (v0 + i) * LDB + 4 * tx) = make_float4(o[0], o[1], o[2], o[3]);
                *reinterpret_cast<float4*>(s.B + (v0 + i) * LDB + 64 + 4 * tx) = make_float4(o[4], o[5], o[6], o[7]);
            }
        }
        for (int i = tid; i < 128 * R; i += NT_LA) s.Qn[i] = round_f16(Q0[i]);
        __syncthreads();

        // ---- stage C: subspace iteration on T = B + p Q_old U_old^T ----
        // P = T^T Q  (rounded to fp16 values)
        coldot<R>(s.B, s.Qn, s.Un, s.scr, tid);
        factor_gram<R>(s.Qo, s.Qn, s.Msm, tid);
        factor_apply<R, true>(s.Uo, s.Msm, s.Un, p, tid);
        for (int it = 0; it < iters; ++it) {
            rowdot<R>(s.B, s.Un, s.Qn, s.scr, tid);          // Q = T P
            factor_gram<R>(s.Uo, s.Un, s.Msm, tid);
            factor_apply<R, false>(s.Qo, s.Msm, s.Qn, p, tid);
            cholqr2_f16<R>(s.Qn, tid);
            coldot<R>(s.B, s.Qn, s.Un, s.scr, tid);          // P = T^T Q
            factor_gram<R>(s.Qo, s.Qn, s.Msm, tid);
            factor_apply<R, true>(s.Uo, s.Msm, s.Un, p, tid);
        }

        // ---- stage D: new factors to the checkpoint ----
        {
            uint16_t* uq = reinterpret_cast<uint16_t*>(base + CK_UQ);
            for (int i = tid; i < R * 128; i += NT_LA) {
                const int r = i >> 7, c = i & 127;
                uq[r * (KD + VD) + c] = f_to_f16(s.Un[c * R + r]);
                uq[r * (KD + VD) + KD + c] = f_to_f16(s.Qn[c * R + r]);
            }
        }

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
    }
}

template <int R, bool KDA>
static int launch_flush(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                        int32_t* hcnt, const float* Q0, const int32_t* idx, int N, int iters, cudaStream_t st) {
    const int total = N * d->HV;
    const int G = min(device_sm_count(), total);
    const int maxd = (total + G - 1) / G + 1;
    const size_t smem = sizeof(float) * flush_smem_floats<R>(d->L, maxd);
    if (smem > 227 * 1024) return LQ_ERR_UNSUPPORTED;
    int rc = ensure_smem((const void*)flush_kernel<R, KDA>, smem);
    if (rc) return rc;
    flush_kernel<R, KDA><<<G, NT_LA, smem, st>>>(*d, (char*)ssm, (const uint16_t*)Kbuf, (const uint16_t*)Ubuf, Wbuf, Pbuf,
                                                 (uint16_t*)Gbuf, hcnt, Q0, idx, N, iters, maxd);
    return finish_launch();
}

}  // namespace lq

using namespace lq;

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
