// Standalone quantize, in-place dequantize and low-rank factorisation kernels (sm_100a).
//
// One CTA of 256 threads per (row, value head); the head's 128 x 128 fp32 tile lives in shared memory for the whole
// kernel, so the in-place rewrite of the slot (fp32 state <-> packed 8-bit checkpoint) never reads what it has
// already overwritten.
#include "lq_linalg.cuh"

namespace lq {

// ------------------------------------------------------------------------------------------------------------------
// shared pieces
// ------------------------------------------------------------------------------------------------------------------
// Row-wise INT8 stage with true divisions: Sv[v] = max(max_c |E / Sk|, EPS); code = clamp(rint(E / (Sk Sv) * 127)).
// Warp w takes rows 16 w .. 16 w + 15, four rows per pass; eight lanes share a row, each lane owns columns
// {32 i + 4 l8 .. + 3 | i = 0..3} so that the eight float4 reads of a row are one contiguous 128-B line.
__device__ __forceinline__ void quant_rows_div(const float* __restrict__ E, const float* __restrict__ sk, char* base,
                                               int tid) {
    const int warp = tid >> 5, lane = tid & 31, l8 = lane & 7, g = lane >> 3;
    uint32_t* codes = reinterpret_cast<uint32_t*>(base + CK_CODES);
    float* svg = reinterpret_cast<float*>(base + CK_SV);
#pragma unroll 1
    for (int it = 0; it < 4; ++it) {
        const int row = warp * 16 + it * 4 + g;
        float e[16], s[16];
        float rmax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 ev = *reinterpret_cast<const float4*>(E + row * LDB + i * 32 + l8 * 4);
            const float4 sv4 = *reinterpret_cast<const float4*>(sk + i * 32 + l8 * 4);
            e[4 * i + 0] = ev.x; e[4 * i + 1] = ev.y; e[4 * i + 2] = ev.z; e[4 * i + 3] = ev.w;
            s[4 * i + 0] = sv4.x; s[4 * i + 1] = sv4.y; s[4 * i + 2] = sv4.z; s[4 * i + 3] = sv4.w;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) rmax = fmaxf(rmax, fabsf(e[i] / s[i]));
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 4));
        const float svv = fmaxf(rmax, EPS);
        if (l8 == 0) svg[row] = svv;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t b[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float c = rintf(e[4 * i + k] / (s[4 * i + k] * svv) * QMAX);
                c = fminf(fmaxf(c, -QMAX), QMAX);
                b[k] = uint32_t(int(c)) & 0xffu;
            }
            codes[row * 32 + i * 8 + l8] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// quantize
// ------------------------------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(NT_LA, 1)
quantize_kernel(lq_dims d, char* __restrict__ ssm, float* __restrict__ Wbuf, float* __restrict__ Pbuf,
                uint16_t* __restrict__ Gbuf, int32_t* __restrict__ hcnt, const float* __restrict__ Q0,
                const int32_t* __restrict__ idx, int kda, int iters) {
    extern __shared__ __align__(16) float smem[];
    float* S = smem;                      // [128][LDB]
    float* Qs = S + 128 * LDB;            // [128][R]
    float* Ps = Qs + 128 * R;             // [128][R]
    float* scr = Ps + 128 * R;            // [128][R]
    float* sk = scr + 128 * R;            // [128]
    float* part = sk + 128;               // [2][128]
    const int tid = threadIdx.x;
    const int n = blockIdx.x / d.HV, hv = blockIdx.x % d.HV;
    const int slot = idx[n];
    if (slot <= 0 || slot >= d.NS) return;
    char* base = head_base(ssm, d.SS, slot, hv);

    for (int i = tid; i < 128 * 32; i += NT_LA) {
        const float4 v = reinterpret_cast<const float4*>(base)[i];
        *reinterpret_cast<float4*>(S + (i >> 5) * LDB + (i & 31) * 4) = v;
    }
    for (int i = tid; i < 128 * R; i += NT_LA) Qs[i] = Q0[i];
    __syncthreads();

    for (int it = 0; it < iters; ++it) {
        coldot<R>(S, Qs, Ps, scr, tid);       // P = S^T Q
        mgs_cols<R>(Ps, tid);
        rowdot<R>(S, Ps, Qs, scr, tid);       // Q = S P
        mgs_cols<R>(Qs, tid);
    }
    coldot<R>(S, Qs, Ps, scr, tid);           // U = S^T Q
    for (int i = tid; i < 128 * R; i += NT_LA) {
        Ps[i] = round_f16(Ps[i]);
        Qs[i] = round_f16(Qs[i]);
    }
    __syncthreads();

    // residual E = S - Q U^T (one factor at a time, fused multiply-add), column sums of |E|
    {
        const int c = tid & 127, half = tid >> 7;
        float u[R];
#pragma unroll
        for (int r = 0; r < R; ++r) u[r] = Ps[c * R + r];
        float cs = 0.f;
#pragma unroll 4
        for (int row = half * 64; row < half * 64 + 64; ++row) {
            float acc = S[row * LDB + c];
#pragma unroll
            for (int r = 0; r < R; ++r) acc = fmaf(-Qs[row * R + r], u[r], acc);
            S[row * LDB + c] = acc;
            cs += fabsf(acc);
        }
        part[half * 128 + c] = cs;
    }
    __syncthreads();
    if (tid < 128) {
        const float skv = fmaxf(sqrtf((part[tid] + part[128 + tid]) / float(VD)), EPS);
        sk[tid] = skv;
        reinterpret_cast<float*>(base + CK_SK)[tid] = skv;
    }
    __syncthreads();
    quant_rows_div(S, sk, base, tid);

    uint16_t* uq = reinterpret_cast<uint16_t*>(base + CK_UQ);
    for (int i = tid; i < R * 128; i += NT_LA) {
        const int r = i >> 7, c = i & 127;
        uq[r * (KD + VD) + c] = f_to_f16(Ps[c * R + r]);
        uq[r * (KD + VD) + KD + c] = f_to_f16(Qs[c * R + r]);
    }
    // window reset
    const int64_t sh = int64_t(slot) * d.HV + hv;
    for (int j = tid; j < d.L; j += NT_LA) Wbuf[sh * d.L + j] = 0.f;
    if (kda) {
        for (int c = tid; c < KD; c += NT_LA) Pbuf[sh * KD + c] = 0.f;
        uint32_t* g32 = reinterpret_cast<uint32_t*>(Gbuf + sh * d.L * KD);
        for (int i = tid; i < d.L * KD / 2; i += NT_LA) g32[i] = 0x3C003C00u;     // fp16 1.0 pairs
    } else if (tid == 0) {
        Pbuf[sh] = 1.f;
    }
    if (tid == 0) hcnt[sh] = 0;
}

// ------------------------------------------------------------------------------------------------------------------
// dequantize in place
// ------------------------------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(NT_LA, 1)
dequant_kernel(lq_dims d, char* __restrict__ ssm, const uint16_t* __restrict__ Kbuf, const uint16_t* __restrict__ Ubuf,
               float* __restrict__ Wbuf, float* __restrict__ Pbuf, const uint16_t* __restrict__ Gbuf,
               int32_t* __restrict__ hcnt, const int32_t* __restrict__ idx, int kda) {
    extern __shared__ __align__(16) float smem[];
    uint32_t* cw = reinterpret_cast<uint32_t*>(smem);     // [128][32] code words
    float* sk = smem + 4096;                              // [128]  (KDA: unscaled)
    float* sv = sk + 128;                                 // [128]
    float* pc = sv + 128;                                 // [128]  per-column decay (GDN: 1)
    float* Uo = pc + 128;                                 // [R][128]
    float* Qo = Uo + R * 128;                             // [R][128]
    float* Kf = Qo + R * 128;                             // [L][128] keys (KDA: decayed)
    float* Uf = Kf + d.L * 128;                           // [L][128] w_j u_j
    float* lut = Uf + d.L * 128;                          // [256] code / 127, indexed by code + 128: the IEEE division the
                                                          // reference's expression asks for, done 256 times per CTA instead of 16 384
    const int tid = threadIdx.x;
    const int n = blockIdx.x / d.HV, hv = blockIdx.x % d.HV;
    const int slot = idx[n];
    if (slot <= 0 || slot >= d.NS) return;
    char* base = head_base(ssm, d.SS, slot, hv);
    const int64_t sh = int64_t(slot) * d.HV + hv;
    const int h = min(max(hcnt[sh], 0), d.L);
    const float p = kda ? 1.f : Pbuf[sh];

    for (int i = tid; i < 4096 / 4; i += NT_LA)
        reinterpret_cast<uint4*>(cw)[i] = reinterpret_cast<const uint4*>(base + CK_CODES)[i];
    lut[tid] = float(tid - 128) / QMAX;
    if (tid < 128) {
        sk[tid] = reinterpret_cast<const float*>(base + CK_SK)[tid];
        sv[tid] = reinterpret_cast<const float*>(base + CK_SV)[tid];
        pc[tid] = kda ? expf(Pbuf[sh * KD + tid]) : 1.f;
    }
    {
        const uint16_t* uq = reinterpret_cast<const uint16_t*>(base + CK_UQ);
        for (int i = tid; i < R * 128; i += NT_LA) {
            const int r = i >> 7, c = i & 127;
            Uo[i] = f16_to_f(uq[r * (KD + VD) + c]);
            Qo[i] = f16_to_f(uq[r * (KD + VD) + KD + c]);
        }
    }
    for (int i = tid; i < h * 128; i += NT_LA) {
        const int j = i >> 7;
        Kf[i] = bf16_to_f(Kbuf[sh * d.L * KD + i]);
        Uf[i] = Wbuf[sh * d.L + j] * bf16_to_f(Ubuf[sh * d.L * VD + i]);
    }
    __syncthreads();
    if (kda && tid < 128) {                    // D_j = prod_{j < i < h} e_i, backward running product per column
        float dcur = 1.f;
        for (int j = h - 1; j >= 0; --j) {
            Kf[j * 128 + tid] *= dcur;
            dcur *= f16_to_f(Gbuf[(sh * d.L + j) * KD + tid]);
        }
    }
    __syncthreads();

    const int ty = tid >> 4, tx = tid & 15, v0 = ty * 8;
    float acc[8][8];
    // checkpoint part: (q / 127) * Sk * Sv + sum_r Q_r[v] U_r[c], then the decay
    {
        float skl[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            skl[k] = sk[4 * tx + k];
            skl[4 + k] = sk[64 + 4 * tx + k];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float svv = sv[v0 + i];
            const uint32_t wa = cw[(v0 + i) * 32 + tx] ^ 0x80808080u, wb = cw[(v0 + i) * 32 + 16 + tx] ^ 0x80808080u;
            const float f[8] = {lut[wa & 255u], lut[(wa >> 8) & 255u], lut[(wa >> 16) & 255u], lut[wa >> 24],
                                lut[wb & 255u], lut[(wb >> 8) & 255u], lut[(wb >> 16) & 255u], lut[wb >> 24]};
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[i][k] = f[k] * skl[k] * svv;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float uu[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uu[k] = Uo[r * 128 + 4 * tx + k];
                uu[4 + k] = Uo[r * 128 + 64 + 4 * tx + k];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float qv = Qo[r * 128 + v0 + i];
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[i][k] = fmaf(qv, uu[k], acc[i][k]);
            }
        }
        float pcl[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            pcl[k] = pc[4 * tx + k];
            pcl[4 + k] = pc[64 + 4 * tx + k];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[i][k] = acc[i][k] * p * pcl[k];
    }
    // live window entries
    for (int j = 0; j < h; ++j) {
        const float4 ua = *reinterpret_cast<const float4*>(Uf + j * 128 + v0);
        const float4 ub = *reinterpret_cast<const float4*>(Uf + j * 128 + v0 + 4);
        const float4 ka = *reinterpret_cast<const float4*>(Kf + j * 128 + 4 * tx);
        const float4 kb = *reinterpret_cast<const float4*>(Kf + j * 128 + 64 + 4 * tx);
        const float uu[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
        const float kk[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[i][k] = fmaf(uu[i], kk[k], acc[i][k]);
    }
    float* out = reinterpret_cast<float*>(base);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        *reinterpret_cast<float4*>(out + (v0 + i) * KD + 4 * tx) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4*>(out + (v0 + i) * KD + 64 + 4 * tx) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
    if (!kda) {
        for (int j = tid; j < d.L; j += NT_LA) Wbuf[sh * d.L + j] = 0.f;
        if (tid == 0) {
            Pbuf[sh] = 1.f;
            hcnt[sh] = 0;
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// low-rank factorisation of x [n][K][V]
// ------------------------------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(NT_LA, 1)
lowrank_kernel(const float* __restrict__ x, const float* __restrict__ Q0, float* __restrict__ U, float* __restrict__ Q,
               int iters) {
    extern __shared__ __align__(16) float smem[];
    float* M = smem;                      // [K][LDB]: row = key index, column = value index
    float* Qs = M + 128 * LDB;            // [V][R]
    float* Ps = Qs + 128 * R;             // [K][R]
    float* scr = Ps + 128 * R;
    const int tid = threadIdx.x;
    const float* xb = x + int64_t(blockIdx.x) * KD * VD;
    for (int i = tid; i < 128 * 32; i += NT_LA) {
        const float4 v = reinterpret_cast<const float4*>(xb)[i];
        *reinterpret_cast<float4*>(M + (i >> 5) * LDB + (i & 31) * 4) = v;
    }
    for (int i = tid; i < 128 * R; i += NT_LA) Qs[i] = Q0[i];
    __syncthreads();
    for (int it = 0; it < iters; ++it) {
        rowdot<R>(M, Qs, Ps, scr, tid);       // P = x Q
        mgs_cols<R>(Ps, tid);
        coldot<R>(M, Ps, Qs, scr, tid);       // Q = x^T P
        mgs_cols<R>(Qs, tid);
    }
    rowdot<R>(M, Qs, Ps, scr, tid);           // U = x Q
    float* Ub = U + int64_t(blockIdx.x) * KD * R;
    float* Qb = Q + int64_t(blockIdx.x) * VD * R;
    for (int i = tid; i < 128 * R; i += NT_LA) {
        Ub[i] = Ps[i];
        Qb[i] = Qs[i];
    }
}

}  // namespace lq

using namespace lq;

extern "C" int lq_quantize(const lq_dims* d, void* ssm, float* Wbuf, float* Pbuf, void* Gbuf, int32_t* hcnt,
                           const float* Q0, const int32_t* idx, int32_t N, int32_t kda, int32_t iters, void* stream) {
    int rc = check_dims(d);
    if (rc) return rc;
    if (!ssm || !Wbuf || !Pbuf || !hcnt || !Q0 || (N > 0 && !idx) || (kda && !Gbuf)) return LQ_ERR_NULL;
    if (N < 0 || iters < 0) return LQ_ERR_RANGE;
    if (misaligned16({ssm}) || (kda && misaligned16({Gbuf}))) return LQ_ERR_ALIGN;
    if (N == 0) return LQ_OK;
    const size_t smem = sizeof(float) * (128 * LDB + 3 * 128 * d->R + 128 + 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(unsigned(N) * d->HV), block(NT_LA);
    if (d->R == 4) {
        if ((rc = ensure_smem((const void*)quantize_kernel<4>, smem))) return rc;
        quantize_kernel<4><<<grid, block, smem, st>>>(*d, (char*)ssm, Wbuf, Pbuf, (uint16_t*)Gbuf, hcnt, Q0, idx, kda, iters);
    } else {
        if ((rc = ensure_smem((const void*)quantize_kernel<8>, smem))) return rc;
        quantize_kernel<8><<<grid, block, smem, st>>>(*d, (char*)ssm, Wbuf, Pbuf, (uint16_t*)Gbuf, hcnt, Q0, idx, kda, iters);
    }
    return finish_launch();
}

extern "C" int lq_dequant(const lq_dims* d, void* ssm, const void* Kbuf, const void* Ubuf, float* Wbuf, float* Pbuf,
                          const void* Gbuf, int32_t* hcnt, const int32_t* idx, int32_t N, int32_t kda, void* stream) {
    int rc = check_dims(d);
    if (rc) return rc;
    if (!ssm || !Kbuf || !Ubuf || !Wbuf || !Pbuf || !hcnt || (N > 0 && !idx) || (kda && !Gbuf)) return LQ_ERR_NULL;
    if (N < 0) return LQ_ERR_RANGE;
    if (misaligned16({ssm, Kbuf, Ubuf})) return LQ_ERR_ALIGN;
    if (N == 0) return LQ_OK;
    const size_t smem = sizeof(float) * (4096 + 3 * 128 + 2 * d->R * 128 + 2 * d->L * 128 + 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid(unsigned(N) * d->HV), block(NT_LA);
    if (d->R == 4) {
        if ((rc = ensure_smem((const void*)dequant_kernel<4>, smem))) return rc;
        dequant_kernel<4><<<grid, block, smem, st>>>(*d, (char*)ssm, (const uint16_t*)Kbuf, (const uint16_t*)Ubuf, Wbuf, Pbuf,
                                                     (const uint16_t*)Gbuf, hcnt, idx, kda);
    } else {
        if ((rc = ensure_smem((const void*)dequant_kernel<8>, smem))) return rc;
        dequant_kernel<8><<<grid, block, smem, st>>>(*d, (char*)ssm, (const uint16_t*)Kbuf, (const uint16_t*)Ubuf, Wbuf, Pbuf,
                                                     (const uint16_t*)Gbuf, hcnt, idx, kda);
    }
    return finish_launch();
}

extern "C" int lq_lowrank(const float* x, const float* Q0, float* U, float* Q, int32_t n, int32_t K, int32_t V, int32_t r,
                          int32_t iters, void* stream) {
    if (!x || !Q0 || !U || !Q) return LQ_ERR_NULL;
    if (K != KD || V != VD || (r != 4 && r != 8)) return LQ_ERR_UNSUPPORTED;
    if (n < 0 || iters < 0) return LQ_ERR_RANGE;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return LQ_ERR_ALIGN;
    if (n == 0) return LQ_OK;
    const size_t smem = sizeof(float) * (128 * LDB + 3 * 128 * r);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if (r == 4) {
        if ((rc = ensure_smem((const void*)lowrank_kernel<4>, smem))) return rc;
        lowrank_kernel<4><<<n, NT_LA, smem, st>>>(x, Q0, U, Q, iters);
    } else {
        if ((rc = ensure_smem((const void*)lowrank_kernel<8>, smem))) return rc;
        lowrank_kernel<8><<<n, NT_LA, smem, st>>>(x, Q0, U, Q, iters);
    }
    return finish_launch();
}
