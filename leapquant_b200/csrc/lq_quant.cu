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
// Row-wise INT8 stage.  The results are those of the reference's true divisions (leapquant/kernels.py:2218-2229):
//   Sv[v] = max(max_c |E / Sk|, EPS),  code = clamp(rint(E / (Sk Sv) * 127)),
// but a division is only executed where it can matter.  Row maximum: the candidates are found with |E| * (1 / Sk) (within
// two ulp of the quotient), and only elements within 1e-6 of the best candidate are divided -- the true maximum is always
// among them.  Codes: y = E * (1 / Sk) * (127 / Sv) is within 5e-5 code units of the exact value, so rint(y) is the exact
// code unless y lies within 1e-3 of a half-integer, and only then is the reference's expression evaluated.
// Warp w takes rows 16 w .. 16 w + 15, four rows per pass; eight lanes share a row, each lane owns columns
// {32 i + 4 l8 .. + 3 | i = 0..3} so that the eight float4 reads of a row are one contiguous 128-B line.
__device__ __forceinline__ void quant_rows_div(const float* __restrict__ E, const float* __restrict__ sk, const float* __restrict__ rsk,
                                               char* base, int tid) {
    const int warp = tid >> 5, lane = tid & 31, l8 = lane & 7, g = lane >> 3;
    uint32_t* codes = reinterpret_cast<uint32_t*>(base + CK_CODES);
    float* svg = reinterpret_cast<float*>(base + CK_SV);
#pragma unroll 1
    for (int it = 0; it < 4; ++it) {
        const int row = warp * 16 + it * 4 + g;
        float e[16], a[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 ev = *reinterpret_cast<const float4*>(E + row * LDB + i * 32 + l8 * 4);
            const float4 rv = *reinterpret_cast<const float4*>(rsk + i * 32 + l8 * 4);
            e[4 * i + 0] = ev.x; e[4 * i + 1] = ev.y; e[4 * i + 2] = ev.z; e[4 * i + 3] = ev.w;
            a[4 * i + 0] = ev.x * rv.x; a[4 * i + 1] = ev.y * rv.y; a[4 * i + 2] = ev.z * rv.z; a[4 * i + 3] = ev.w * rv.w;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(a[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float thr = amax * (1.0f - 1e-6f);
        float rmax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (fabsf(a[i]) >= thr) rmax = fmaxf(rmax, fabsf(e[i] / sk[(i >> 2) * 32 + l8 * 4 + (i & 3)]));
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
        rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 4));
        const float svv = fmaxf(rmax, EPS);
        if (l8 == 0) svg[row] = svv;
        const float rv127 = QMAX / svv;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t b[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float y = a[4 * i + k] * rv127;
                float c = rintf(y);
                if (fabsf(fabsf(y - c) - 0.5f) < 1e-3f)                        // on a rounding boundary: the exact expression decides
                    c = rintf(e[4 * i + k] / (sk[i * 32 + l8 * 4 + k] * svv) * QMAX);
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
__global__ void __launch_bounds__(NT_LA, 3)
quantize_kernel(lq_dims d, char* __restrict__ ssm, float* __restrict__ Wbuf, float* __restrict__ Pbuf,
                uint16_t* __restrict__ Gbuf, int32_t* __restrict__ hcnt, const float* __restrict__ Q0,
                const int32_t* __restrict__ idx, int kda, int iters) {
    extern __shared__ __align__(16) float smem[];
    float* S = smem;                      // [128][LDB]
    float* Qs = S + 128 * LDB;            // [128][R]
    float* Ps = Qs + 128 * R;             // [128][R]
    float* scr = Ps + 128 * R;            // [128][R]
    float* sk = scr + 128 * R;            // [128]
    float* part = sk + 128;               // [2][128]; afterwards [0 .. 127] holds 1 / Sk
    const int tid = threadIdx.x;
    const int n = blockIdx.x / d.HV, hv = blockIdx.x % d.HV;
    const int slot = idx[n];
    if (slot <= 0 || slot >= d.NS) return;
    char* base = head_base(ssm, d.SS, slot, hv);

    // the head's 64 KB arrive as 128 bulk asynchronous copies (one row of 512 bytes each, issued by 128 threads at once) that
    // complete on one mbarrier: the whole tile is in flight from the first instruction on and costs no registers
    __shared__ __align__(8) uint64_t load_bar;
    if (tid == 0) {
        mbar_init(&load_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) mbar_arrive_expect_tx(&load_bar, 128u * 512u);
    __syncthreads();
    if (tid < 128) bulk_g2s(S + tid * LDB, base + tid * 512, 512u, &load_bar);
    for (int i = tid; i < 128 * R; i += NT_LA) Qs[i] = Q0[i];
    {
        bool ok = false;
        for (uint32_t it = 0; it < WAIT_LIMIT && !ok; ++it) ok = mbar_try_wait(&load_bar, 0u);
        if (!ok) atomicOr(&g_status, ST_FLUSH_TIMEOUT);
    }
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
        part[tid] = 1.0f / skv;               // (its own partial sums were read just above)
    }
    __syncthreads();
    quant_rows_div(S, sk, part, base, tid);

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
// S[v][c] = (q8 / 127 Sk[c] Sv[v] + sum_r Q_r[v] U_r[c]) p pc[c] + sum_{j<h} (w_j u_j[v]) (k_j[c] D_j[c])   (leapquant/kernels.py:2105-2117;
// KDA: leapquant/state.py:118-128).  The per-element work is kept to one conversion, one multiply and 1 + R + h fused
// multiply-adds by folding the constants into the vectors first: skq[c] = Sk[c] / 127 (* pc[c]), svp[v] = Sv[v] p,
// Qp_r[v] = Q_r[v] p, Uc_r[c] = U_r[c] (* pc[c]).  The values differ from the reference's evaluation order in the last place of fp32.
// The window rows stay bf16 in shared memory (KDA keys: decayed, fp32), so that three CTAs fit on an SM.
template <int R>
__global__ void __launch_bounds__(NT_LA, 3)
dequant_kernel(lq_dims d, char* __restrict__ ssm, const uint16_t* __restrict__ Kbuf, const uint16_t* __restrict__ Ubuf,
               float* __restrict__ Wbuf, float* __restrict__ Pbuf, const uint16_t* __restrict__ Gbuf,
               int32_t* __restrict__ hcnt, const int32_t* __restrict__ idx, int kda) {
    extern __shared__ __align__(16) float smem[];
    uint32_t* cw = reinterpret_cast<uint32_t*>(smem);     // [128][32] code words
    float* skq = smem + 4096;                             // [128] Sk / 127 (KDA: times pc)
    float* svp = skq + 128;                               // [128] Sv p
    float* Uc = svp + 128;                                // [R][128] U_r (KDA: times pc)
    float* Qp = Uc + R * 128;                             // [R][128] Q_r p
    float* ws = Qp + R * 128;                             // [64] window weights
    float* Kf = ws + 64;                                  // KDA: [L][128] decayed keys (fp32); GDN: [L][64] bf16 pairs
    const int tid = threadIdx.x;
    const int n = blockIdx.x / d.HV, hv = blockIdx.x % d.HV;
    const int slot = idx[n];
    if (slot <= 0 || slot >= d.NS) return;
    char* base = head_base(ssm, d.SS, slot, hv);
    const int64_t sh = int64_t(slot) * d.HV + hv;
    const int h = min(max(hcnt[sh], 0), d.L);
    const float p = kda ? 1.f : Pbuf[sh];
    uint32_t* Kb2 = reinterpret_cast<uint32_t*>(Kf);                              // GDN keys as stored
    uint32_t* Ub2 = reinterpret_cast<uint32_t*>(Kf + (kda ? d.L * 128 : d.L * 64));  // values as stored (bf16 pairs) [L][64]

    for (int i = tid; i < 4096 / 4; i += NT_LA)
        reinterpret_cast<uint4*>(cw)[i] = reinterpret_cast<const uint4*>(base + CK_CODES)[i];
    if (tid < 128) {
        const float pc = kda ? expf(Pbuf[sh * KD + tid]) : 1.f;
        skq[tid] = reinterpret_cast<const float*>(base + CK_SK)[tid] / QMAX * pc;
        svp[tid] = reinterpret_cast<const float*>(base + CK_SV)[tid] * p;
        const uint16_t* uq = reinterpret_cast<const uint16_t*>(base + CK_UQ);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            Uc[r * 128 + tid] = f16_to_f(uq[r * (KD + VD) + tid]) * pc;
            Qp[r * 128 + tid] = f16_to_f(uq[r * (KD + VD) + KD + tid]) * p;
        }
    }
    if (tid < d.L) ws[tid] = tid < h ? Wbuf[sh * d.L + tid] : 0.f;
    {
        const uint4* kb = reinterpret_cast<const uint4*>(Kbuf + sh * d.L * KD);
        const uint4* ub = reinterpret_cast<const uint4*>(Ubuf + sh * d.L * VD);
        for (int i = tid; i < h * 16; i += NT_LA) {
            reinterpret_cast<uint4*>(Ub2)[i] = ub[i];
            const uint4 kv = kb[i];
            if (kda) {
                float4* kp = reinterpret_cast<float4*>(Kf + i * 8);
                const float2 a0 = bf16x2_to_f2(kv.x), a1 = bf16x2_to_f2(kv.y), a2 = bf16x2_to_f2(kv.z), a3 = bf16x2_to_f2(kv.w);
                kp[0] = make_float4(a0.x, a0.y, a1.x, a1.y);
                kp[1] = make_float4(a2.x, a2.y, a3.x, a3.y);
            } else {
                reinterpret_cast<uint4*>(Kb2)[i] = kv;
            }
        }
    }
    __syncthreads();
    if (kda && tid < 128) {                    // D_j = prod_{j < i < h} e_i, backward running product per column
        float dcur = 1.f;
        for (int j = h - 1; j >= 0; --j) {
            Kf[j * 128 + tid] *= dcur;
            dcur *= f16_to_f(Gbuf[(sh * d.L + j) * KD + tid]);
        }
    }
    if (kda) __syncthreads();

    // thread (ty, tx) owns rows v0 .. v0 + 7 and the eight columns 4 tx .. + 3, 64 + 4 tx .. + 3
    const int ty = tid >> 4, tx = tid & 15, v0 = ty * 8;
    float acc[8][8];
    {
        float uu[R][8], skl[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            skl[k] = skq[4 * tx + k];
            skl[4 + k] = skq[64 + 4 * tx + k];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                uu[r][k] = Uc[r * 128 + 4 * tx + k];
                uu[r][4 + k] = Uc[r * 128 + 64 + 4 * tx + k];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float f[8];
            s8x4_to_f4(cw[(v0 + i) * 32 + tx], f[0], f[1], f[2], f[3]);
            s8x4_to_f4(cw[(v0 + i) * 32 + 16 + tx], f[4], f[5], f[6], f[7]);
            const float svv = svp[v0 + i];
            float qv[R];
#pragma unroll
            for (int r = 0; r < R; ++r) qv[r] = Qp[r * 128 + v0 + i];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float a2 = (f[k] * skl[k]) * svv;
#pragma unroll
                for (int r = 0; r < R; ++r) a2 = fmaf(qv[r], uu[r][k], a2);
                acc[i][k] = a2;
            }
        }
    }
    // live window entries
    for (int j = 0; j < h; ++j) {
        const float wj = ws[j];
        const uint4 uw = *reinterpret_cast<const uint4*>(Ub2 + j * 64 + ty * 4);       // values v0 .. v0 + 7
        const float2 u01 = bf16x2_to_f2(uw.x), u23 = bf16x2_to_f2(uw.y), u45 = bf16x2_to_f2(uw.z), u67 = bf16x2_to_f2(uw.w);
        const float uu[8] = {u01.x * wj, u01.y * wj, u23.x * wj, u23.y * wj, u45.x * wj, u45.y * wj, u67.x * wj, u67.y * wj};
        float kk[8];
        if (kda) {
            const float4 ka = *reinterpret_cast<const float4*>(Kf + j * 128 + 4 * tx);
            const float4 kb4 = *reinterpret_cast<const float4*>(Kf + j * 128 + 64 + 4 * tx);
            kk[0] = ka.x; kk[1] = ka.y; kk[2] = ka.z; kk[3] = ka.w; kk[4] = kb4.x; kk[5] = kb4.y; kk[6] = kb4.z; kk[7] = kb4.w;
        } else {
            const uint2 ka = *reinterpret_cast<const uint2*>(Kb2 + j * 64 + 2 * tx), kb2 = *reinterpret_cast<const uint2*>(Kb2 + j * 64 + 32 + 2 * tx);
            const float2 k01 = bf16x2_to_f2(ka.x), k23 = bf16x2_to_f2(ka.y), k45 = bf16x2_to_f2(kb2.x), k67 = bf16x2_to_f2(kb2.y);
            kk[0] = k01.x; kk[1] = k01.y; kk[2] = k23.x; kk[3] = k23.y; kk[4] = k45.x; kk[5] = k45.y; kk[6] = k67.x; kk[7] = k67.y;
        }
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
    // codes, folded scales, factors, weights, window rows (bf16; KDA keys fp32 because they carry the decay)
    const size_t smem = sizeof(float) * (4096 + 2 * 128 + 2 * d->R * 128 + 64 + (kda ? d->L * 128 : d->L * 64) + d->L * 64);
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
