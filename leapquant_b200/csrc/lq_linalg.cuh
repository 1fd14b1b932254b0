// Block-level tall-skinny linear algebra on a 128 x 128 fp32 tile held in shared memory (256-thread CTAs).
// Used by the flush, the standalone quantize and the low-rank kernel.
#pragma once
#include "lq_common.cuh"

namespace lq {

constexpr int LDB = 132;          // row stride of the fp32 tile: 16-B aligned rows, conflict-free float4 reads down a column of rows
constexpr int NT_LA = 256;        // threads of the CTAs that use these helpers

// Y[c][r] = sum_row M[row][c] * X[row][r]      (M: [128][LDB]; X, Y, scratch: [128][R]; all in shared memory)
// The 128 rows are split in two halves of 64 summed in row order each; the halves are then added.
template <int R>
__device__ __forceinline__ void coldot(const float* __restrict__ M, const float* __restrict__ X, float* __restrict__ Y,
                                       float* __restrict__ scratch, int tid) {
    const int c = tid & 127, half = tid >> 7;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    const float* m = M + (half * 64) * LDB + c;
    const float* x = X + (half * 64) * R;
#pragma unroll 4
    for (int row = 0; row < 64; ++row) {
        const float mv = m[row * LDB];
#pragma unroll
        for (int r4 = 0; r4 < R; r4 += 4) {
            const float4 xv = *reinterpret_cast<const float4*>(x + row * R + r4);
            acc[r4 + 0] = fmaf(mv, xv.x, acc[r4 + 0]);
            acc[r4 + 1] = fmaf(mv, xv.y, acc[r4 + 1]);
            acc[r4 + 2] = fmaf(mv, xv.z, acc[r4 + 2]);
            acc[r4 + 3] = fmaf(mv, xv.w, acc[r4 + 3]);
        }
    }
    if (half == 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) scratch[c * R + r] = acc[r];
    }
    __syncthreads();
    if (half == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) Y[c * R + r] = acc[r] + scratch[c * R + r];
    }
    __syncthreads();
}

// Y[row][r] = sum_c M[row][c] * X[c][r]
template <int R>
__device__ __forceinline__ void rowdot(const float* __restrict__ M, const float* __restrict__ X, float* __restrict__ Y,
                                       float* __restrict__ scratch, int tid) {
    const int row = tid & 127, half = tid >> 7;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    const float* m = M + row * LDB + half * 64;
    const float* x = X + (half * 64) * R;
#pragma unroll 2
    for (int c = 0; c < 64; c += 4) {
        const float4 mv = *reinterpret_cast<const float4*>(m + c);
        const float mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int r4 = 0; r4 < R; r4 += 4) {
                const float4 xv = *reinterpret_cast<const float4*>(x + (c + i) * R + r4);
                acc[r4 + 0] = fmaf(mm[i], xv.x, acc[r4 + 0]);
                acc[r4 + 1] = fmaf(mm[i], xv.y, acc[r4 + 1]);
                acc[r4 + 2] = fmaf(mm[i], xv.z, acc[r4 + 2]);
                acc[r4 + 3] = fmaf(mm[i], xv.w, acc[r4 + 3]);
            }
        }
    }
    if (half == 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) scratch[row * R + r] = acc[r];
    }
    __syncthreads();
    if (half == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) Y[row * R + r] = acc[r] + scratch[row * R + r];
    }
    __syncthreads();
}

// Small product  Msm[r][s] = sum_i A[r][i] * X[i][s]  with A: [R][128] (factor-major), X: [128][R]; one warp per output.
template <int R>
__device__ __forceinline__ void factor_gram(const float* __restrict__ A, const float* __restrict__ X, float* __restrict__ Msm,
                                            int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    for (int o = warp; o < R * R; o += NT_LA / 32) {
        const int r = o / R, s = o % R;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc = fmaf(A[r * 128 + lane + 32 * i], X[(lane + 32 * i) * R + s], acc);
        acc = warp_sum(acc);
        if (lane == 0) Msm[o] = acc;
    }
    __syncthreads();
}

// Y[i][s] += p * sum_r A[r][i] * Msm[r][s]   (thread per i < 128), optional fp16 rounding of the result
template <int R, bool ROUND16>
__device__ __forceinline__ void factor_apply(const float* __restrict__ A, const float* __restrict__ Msm, float* __restrict__ Y,
                                             float p, int tid) {
    if (tid < 128) {
        float a[R];
#pragma unroll
        for (int r = 0; r < R; ++r) a[r] = A[r * 128 + tid];
#pragma unroll
        for (int s = 0; s < R; ++s) {
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) acc = fmaf(a[r], Msm[r * R + s], acc);
            float y = fmaf(p, acc, Y[tid * R + s]);
            Y[tid * R + s] = ROUND16 ? round_f16(y) : y;
        }
    }
    __syncthreads();
}

// Modified Gram-Schmidt on the R columns of X [128][R] (shared memory), run by warp 0; the other warps wait at the barrier.
template <int R>
__device__ __forceinline__ void mgs_cols(float* __restrict__ X, int tid) {
    if (tid < 32) {
        float x[4][R];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int r = 0; r < R; ++r) x[i][r] = X[(tid + 32 * i) * R + r];
#pragma unroll
        for (int j = 0; j < R; ++j) {
#pragma unroll
            for (int c = 0; c < j; ++c) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) s = fmaf(x[i][c], x[i][j], s);
                s = warp_sum(s);
#pragma unroll
                for (int i = 0; i < 4; ++i) x[i][j] = fmaf(-s, x[i][c], x[i][j]);
            }
            float n = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) n = fmaf(x[i][j], x[i][j], n);
            n = rsqrtf(fmaxf(warp_sum(n), 1e-30f));
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i][j] *= n;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int r = 0; r < R; ++r) X[(tid + 32 * i) * R + r] = x[i][r];
    }
    __syncthreads();
}

// One CholeskyQR pass on the rows a lane of warp 0 holds (rows lane + 32 i).  DROP = false floors a dependent
// column's pivot at 1e-6 * g_jj, DROP = true zeroes the column.
template <int R, bool DROP>
__device__ __forceinline__ void cholqr_pass_regs(float (&x)[4][R]) {
    float g[R][R];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c <= r; ++c) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) s = fmaf(x[i][r], x[i][c], s);
            g[r][c] = warp_sum(s);
        }
    float l[R][R];
    float inv[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
#pragma unroll
        for (int k = 0; k < j; ++k) {
            float acc = g[j][k];
#pragma unroll
            for (int m = 0; m < k; ++m) acc -= l[j][m] * l[k][m];
            l[j][k] = acc * inv[k];
        }
        float d = g[j][j];
#pragma unroll
        for (int m = 0; m < j; ++m) d -= l[j][m] * l[j][m];
        if (DROP)
            inv[j] = (d > 1e-6f * g[j][j] + 1e-30f) ? rsqrtf(fmaxf(d, 1e-30f)) : 0.f;
        else
            inv[j] = rsqrtf(fmaxf(fmaxf(d, 1e-6f * g[j][j]), 1e-30f));
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < R; ++j) {
            float acc = x[i][j];
#pragma unroll
            for (int m = 0; m < j; ++m) acc -= x[i][m] * l[j][m];
            x[i][j] = acc * inv[j];
        }
    }
}

// CholeskyQR2 on X [128][R] by warp 0; the result is rounded to fp16 values (it becomes the stored Q factor).
template <int R, typename Sync>
__device__ __forceinline__ void cholqr2_f16(float* __restrict__ X, int tid, Sync sync) {
    if (tid < 32) {
        float x[4][R];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int r = 0; r < R; ++r) x[i][r] = X[(tid + 32 * i) * R + r];
        cholqr_pass_regs<R, (R > 4)>(x);
        cholqr_pass_regs<R, (R > 4)>(x);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int r = 0; r < R; ++r) X[(tid + 32 * i) * R + r] = round_f16(x[i][r]);
    }
    sync();
}
template <int R>
__device__ __forceinline__ void cholqr2_f16(float* __restrict__ X, int tid) {
    cholqr2_f16<R>(X, tid, [] { __syncthreads(); });
}

}  // namespace lq
