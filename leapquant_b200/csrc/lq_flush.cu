// Window-flush kernel (sm_100a): rebuild -> rank-R subspace iteration -> residual -> smoothing scales -> INT8.
//
// A head is flushed by a TEAM of NW warps (8 or 16) that share one shared-memory work area and 128 columns of tensor
// memory.  The heavy product of a flush -- the rebuild B[v][c] = sum_j (w_j u_j[v]) k_j[c] of the state from the window,
// 128 x 128 x L -- runs on the fifth-generation tensor cores: the team writes the window tiles into shared memory in
// the canonical 128-byte-swizzled layout, one thread issues tcgen05.mma instructions that accumulate in tensor memory
// (fp32), and every thread then reads ONE ROW of the accumulator back (tcgen05.ld), adds the dequantised checkpoint and
// stores the row of B as f16.  The operand that carries an fp32 scale is split into a bf16 head and a bf16 remainder like
// the reference's (leapquant/kernels.py:1508-1511), which makes two accumulation passes over the same accumulator.
// The tall-skinny products of the subspace iteration and the residual stay on mma.sync (N = R is far below a tcgen05
// tile); B lives in shared memory as an f16 tile like the reference's (leapquant/kernels.py:1156,1483); the residual E
// stays in registers in fp32 until it has become codes.
//
// Two drivers use flush_head(): the standalone flush_kernel below (persistent CTAs of 256 threads = one team of 8 warps,
// two per SM; program p = row * HV + head belongs to CTA p % grid, which tests the window counters of its own programs),
// and the tail of the fused decode kernel (lq_step.cu), whose 512 threads form two teams of 8 warps while at least two
// heads are left and ONE team of 16 warps for a last single head -- the common case of a serving batch whose sequences
// fill their windows at different steps, where the latency of one flush is what the step pays.
#include "lq_linalg.cuh"

namespace lq {

constexpr int TS = 136;          // row stride (16-bit elements) of the f16 state tile: 272 B moves every row one 16-byte bank
                                 // group on, so ldmatrix and fragment loads are conflict-free
constexpr int HS = TS;           // row stride of the factor rows [r][128]
constexpr uint32_t TMEM_COLS = 128;     // tensor-memory columns of one team: the 128 x 128 fp32 accumulator of the rebuild

template <int R> struct FlushK { static constexpr int KC = (R == 4) ? 16 : 32, KS = KC + 8; };  // residual operand rows

struct FlushSmem {
    // region 1, start aligned to 1 KB.  During the rebuild it holds the operand tiles (and the KDA key scales); afterwards the
    // f16 state tile and everything the later stages need.
    char* tile[3];     // [2][Lp][64] bf16 each, 128-byte swizzle: GDN  A head | A remainder | B;  KDA  A | B head | B remainder
    float* tab;        // KDA: [L][128] scale of key (j, c): w_j D_j[c]
    uint16_t* Bh;      // [128][TS] f16 state tile B[v][c]; at the end a warp's rows hold its int8 codes for the coalesced store
    uint16_t* Ac;      // [128][KS] f16 residual operand, row v:  Q | p Q_old head | p Q_old remainder | 0
    uint16_t* Bc;      // [128][KS] f16 residual operand, row c: -U |   U_old      |   U_old           | 0
    float* colpart;    // [8][128] per-row-block column sums of |E|
    float* Qn;         // [128][R] fp32 Q for CholeskyQR
    float* gpart;      // [4][64] per-warp partial Gram matrices of CholeskyQR
    float* rowmax;     // [2][128] per-column-half row maxima (teams of 16 warps)
    // region 2: lives for the whole head
    float* segprod;    // KDA: [4][128] per-segment products of the step factors (written while region 1 holds the key scales)
    uint16_t* Q0h;     // [R][HS] f16 Q0^T, the fixed start of the iteration (written once per team)
    uint16_t* Qh;      // [R][HS] f16 Q^T  (current iterate)
    uint16_t* Ph;      // [R][HS] f16 P^T = new U^T
    uint16_t* Qoh;     // [R][HS] f16 old Q^T
    uint16_t* Uoh;     // [R][HS] f16 old U^T (KDA: times pc, rounded to f16 like the reference, leapquant/kernels.py:1448-1466)
    uint16_t* QoT;     // [128][8] f16 old Q, zero-padded columns R..7
    uint16_t* UoT;     // [128][8] f16 old U
    float* sk;         // [128] column scale operand of the dequant (KDA: Sk pc); later 1 / Sk_new
    float* sv;         // [128]
    float* pc;         // [128]
    float* w;          // [64]
    uint64_t* mbar;    // completion of the rebuild's tensor-core instructions
    int* flags;        // [0] parity of the next completion, [1] outcome of the last wait, [2] due count (standalone kernel)
    int* dlist;        // [maxd]
};

__host__ __device__ inline int flush_lp(int L) { return (L + 15) & ~15; }
template <int R>
__host__ __device__ inline int flush_region1_bytes(int L, bool kda) {
    const int tiles = 3 * flush_lp(L) * 256 + (kda ? L * 512 : 0);
    const int later = 128 * TS * 2 + 2 * 128 * FlushK<R>::KS * 2 + 8 * 128 * 4 + 128 * R * 4 + 4 * 64 * 4 + 2 * 128 * 4;
    return ((tiles > later ? tiles : later) + 127) & ~127;
}
// shared memory of one team, including the slack that lets region 1 start on a 1 KB boundary
template <int R>
__host__ __device__ inline size_t flush_smem_bytes(int L, int maxd, bool kda) {
    return 1024 + size_t(flush_region1_bytes<R>(L, kda)) + 4 * 128 * 4 + 5 * R * HS * 2 + 2 * 128 * 8 * 2 + 3 * 128 * 4 + 64 * 4 + 8 +
           4 * 4 + size_t(maxd) * 4 + 16;
}

// ---- warp-level tensor-core helpers (mma.sync path) ----
__device__ __forceinline__ void mma_h_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// (ldmatrix_x4_trans: lq_quant.cu, compiled ahead of this file in the same translation unit)
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = uint32_t(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t x) { return __half22float2(*reinterpret_cast<const __half2*>(&x)); }

// ---- fifth-generation tensor cores: tensor memory, instruction and operand descriptors ----
// Tensor memory is allocated by one whole warp (a power of two >= 32 of columns; the address lands in shared memory) and
// must be freed by a whole warp before the CTA exits.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] B[smem]: one instruction of M = 128, N = 128, K = 16, issued by ONE thread
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// arrives on the mbarrier once every tensor-core instruction this thread has issued so far is complete
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive fp32 columns of this thread's lane of tensor memory (lane = 32 (warp % 4) + lane id)
__device__ __forceinline__ void tmem_ld_32cols(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Instruction descriptor: fp32 accumulator, bf16 A and B, both operands "MN-major" (the M / N index is the contiguous one in
// shared memory, because the window rows are stored [j][128]), N = 128, M = 128.
constexpr uint32_t UMMA_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
// Operand tile [Lp rows j][128 elements x] of bf16 in the canonical MN-major layout with the 128-byte swizzle: the 128
// elements are two blocks of 64 (128 bytes); block b, row j occupies bytes b * (Lp * 128) + j * 128 .. + 127, and the eight
// 16-byte chunks of such a row are stored at chunk index ^ (j % 8).  Eight rows are one swizzle atom (1 KB): the "stride
// byte offset" between atoms along K is 1 024, the "leading byte offset" between the two blocks along M / N is Lp * 128.
__device__ __forceinline__ uint32_t tile_chunk_offset(int Lp, int j, int c16) {
    return uint32_t(c16 >> 3) * uint32_t(Lp * 128) + uint32_t(j) * 128u + (uint32_t((c16 & 7) ^ (j & 7)) << 4);
}
__device__ __forceinline__ uint64_t umma_desc(const void* tile, int Lp) {
    const uint64_t addr = uint64_t(smem_u32(tile) >> 4) & 0x3FFFull;
    const uint64_t lbo = uint64_t((Lp * 128) >> 4) & 0x3FFFull, sbo = uint64_t(1024 >> 4);
    return addr | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);       // version 1, 128-byte swizzle
}

// x (fp32) ~ hi + lo as two bf16 pieces (16 mantissa bits, relative error 2^-17): the split the reference uses for the
// same operand (reference leapquant/kernels.py:1508-1511).
__device__ __forceinline__ void split2(float x, float& hi, float& lo) {
    hi = round_bf16(x);
    lo = round_bf16(x - hi);
}
// eight bf16 values (a 16-byte chunk) times eight fp32 scales -> head chunk and remainder chunk
__device__ __forceinline__ void scale_split_chunk(const uint4& raw, const float (&sc)[8], uint4& hi, uint4& lo) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float h0, l0, h1, l1;
        split2(bf16lo(w[i]) * sc[2 * i], h0, l0);
        split2(bf16hi(w[i]) * sc[2 * i + 1], h1, l1);
        h[i] = f2_to_bf16x2(h0, h1);
        l[i] = f2_to_bf16x2(l0, l1);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// One tall-skinny product of the subspace iteration with its rank-R correction, warps 0..7, all in registers:
//   TRANS:  Y[c][r] = sum_v B[v][c] X[v][r] + p sum_r' Z[r'][c] (sum_v W[r'][v] X[v][r])     (P = T^T Q:  X = Q, W = Q_old, Z = U_old)
//   !TRANS: Y[v][r] = sum_c B[v][c] X[c][r] + p sum_r' Z[r'][v] (sum_c W[r'][c] X[c][r])     (Q = T P:    X = P, W = U_old, Z = Q_old)
// Xh, Wh: f16 rows [r][128] (stride HS); ZT: f16 [128][8] (Z transposed, columns R..7 zero).  All operands are f16 values by
// definition of the algorithm (B tile, rounded iterates, stored factors), so one mma per tile is exact up to the fp32
// accumulation; the small Gram matrix M^T = X^T W^T comes out of a second mma in exactly the fragment a third mma needs
// as its B operand (times p, as head + remainder).  Warp w owns the output rows 16 w .. 16 w + 15; lane (gid, tig) returns
// d = { Y[16w+gid][2tig], Y[16w+gid][2tig+1], Y[16w+gid+8][2tig], Y[16w+gid+8][2tig+1] }, meaningful for 2 tig < R.
template <int R, bool TRANS>
__device__ __forceinline__ void tall_product(const uint16_t* __restrict__ Bh, const uint16_t* __restrict__ Xh,
                                             const uint16_t* __restrict__ Wh, const uint16_t* __restrict__ ZT, float p,
                                             int warp, int lane, float (&d)[4]) {
    const int gid = lane >> 2, tig = lane & 3, m0 = warp * 16;
    const bool on = gid < R;
    float g[4] = {0.f, 0.f, 0.f, 0.f};
    d[0] = d[1] = d[2] = d[3] = 0.f;
    const uint16_t* xr = Xh + (on ? gid : 0) * HS + 2 * tig;
    const uint16_t* wr = Wh + (on ? gid : 0) * HS + 2 * tig;
    const uint16_t* arow = TRANS ? Bh + ((lane & 7) + 8 * (lane >> 4)) * TS + m0 + 8 * ((lane >> 3) & 1)
                                 : Bh + (m0 + (lane & 7) + 8 * ((lane >> 3) & 1)) * TS + 8 * (lane >> 4);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[4];
        if (TRANS) ldmatrix_x4_trans(a, arow + ks * 16 * TS);
        else ldmatrix_x4(a, arow + ks * 16);
        const uint32_t x0 = on ? *reinterpret_cast<const uint32_t*>(xr + ks * 16) : 0u;
        const uint32_t x1 = on ? *reinterpret_cast<const uint32_t*>(xr + ks * 16 + 8) : 0u;
        const uint32_t w0 = on ? *reinterpret_cast<const uint32_t*>(wr + ks * 16) : 0u;
        const uint32_t w1 = on ? *reinterpret_cast<const uint32_t*>(wr + ks * 16 + 8) : 0u;
        mma_h_16816(d, a[0], a[1], a[2], a[3], x0, x1);
        mma_h_16816(g, x0, 0u, x1, 0u, w0, w1);              // rows 0..7 of the tile: (M^T)[r = gid][r' = 2 tig, 2 tig + 1]
    }
    const float c0 = p * g[0], c1 = p * g[1];
    const __half2 hh = __floats2half2_rn(c0, c1);
    const float2 hf = __half22float2(hh);
    const uint32_t bh = *reinterpret_cast<const uint32_t*>(&hh), bl = pack_h2(c0 - hf.x, c1 - hf.y);
    const uint32_t z0 = *reinterpret_cast<const uint32_t*>(ZT + (m0 + gid) * 8 + 2 * tig);
    const uint32_t z1 = *reinterpret_cast<const uint32_t*>(ZT + (m0 + gid + 8) * 8 + 2 * tig);
    mma_h_16816(d, z0, z1, 0u, 0u, bh, 0u);
    mma_h_16816(d, z0, z1, 0u, 0u, bl, 0u);
}

// G = X^T X for X [128][R] fp32 in shared memory on the tensor cores: mma.sync m16n8k8 with every fp32 value split into a
// tf32 head and a tf32 remainder (head x head + head x remainder + remainder x head: 21 mantissa bits, fp32 range).  The A
// fragment (X^T, rows r) and the B fragment (X, columns c) of a k-step are the same values.  Warp w (of four) sums the 32
// rows 32 w .. 32 w + 31 and writes its partial G[w * 64 + r * 8 + c] for r, c < 8 (rows and columns >= R are zero).
__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32_1688(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
template <int R>
__device__ __forceinline__ void gram_tf32(const float* __restrict__ Xs, float* __restrict__ G, int warp, int lane) {
    const int gid = lane >> 2, tig = lane & 3;
    Xs += warp * 32 * R;
    G += warp * 64;
    const bool on = gid < R;
    float hh[4] = {0.f, 0.f, 0.f, 0.f}, hl[4] = {0.f, 0.f, 0.f, 0.f}, lh[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        const float x0 = on ? Xs[(8 * ks + tig) * R + gid] : 0.f, x1 = on ? Xs[(8 * ks + tig + 4) * R + gid] : 0.f;
        const uint32_t h0 = to_tf32(x0), h1 = to_tf32(x1);
        const uint32_t l0 = to_tf32(x0 - __uint_as_float(h0)), l1 = to_tf32(x1 - __uint_as_float(h1));
        mma_tf32_1688(hh, h0, h1, h0, h1);
        mma_tf32_1688(hl, h0, h1, l0, l1);
        mma_tf32_1688(lh, l0, l1, h0, h1);
    }
    *reinterpret_cast<float2*>(G + gid * 8 + 2 * tig) = make_float2(hh[0] + (hl[0] + lh[0]), hh[1] + (hl[1] + lh[1]));
}

// ---- CholeskyQR on X [128][R] by the first four warps (thread = row) ----
// Sum over the 32 lanes of N values per lane with N + 4 shuffles instead of 5 N: every exchange level halves the number of
// values a lane keeps.  On return the lane holds the totals of indices base .. base + max(N / 32, 1) - 1 in v[0 ..].
template <int N>
__device__ __forceinline__ int fold_over_lanes(float (&v)[N], int lane) {
    int base = 0;
    int n = N;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        if (n > 1) {
            const int half = n >> 1;
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < N / 2; ++i) {
                if (i < half) {
                    const float keep = up ? v[half + i] : v[i];
                    const float send = up ? v[i] : v[half + i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            if (up) base += half;
            n = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
        }
    }
    return base;
}

// One pass: G = X^T X (partial sums per warp -> shared memory -> every row thread adds the four partials), Cholesky of G in
// registers (every thread redundantly), X <- X L^-T applied to the thread's own row.  DROP = false floors a dependent column's
// pivot at 1e-6 g_jj (R <= 4, leapquant/kernels.py:1816-1829), DROP = true zeroes the column (R = 8, :1760-1774).
template <int R, bool DROP, typename Sync>
__device__ __forceinline__ void cholqr_pass_team(float (&x)[R], float* __restrict__ Xs, bool x_in_smem, float* __restrict__ gpart,
                                                 int tid, Sync sync) {
    constexpr bool MMA_GRAM = R > 4;                        // 36 products per row are too many to fold with shuffles
    constexpr int NPP = 16;                                 // R (R + 1) / 2 = 10 products, padded to a power of two (R = 4)
    const int warp = tid >> 5, lane = tid & 31;
    if constexpr (MMA_GRAM) {
        if (!x_in_smem) {
            if (tid < 128) {
#pragma unroll
                for (int r = 0; r < R; ++r) Xs[tid * R + r] = x[r];
            }
            sync();
        }
        if (tid < 128) gram_tf32<R>(Xs, gpart, warp, lane);
    } else {
        if (tid < 128) {
            float pr[NPP];
#pragma unroll
            for (int i = 0; i < NPP; ++i) pr[i] = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int c = 0; c <= r; ++c) pr[r * (r + 1) / 2 + c] = x[r] * x[c];
            const int base = fold_over_lanes<NPP>(pr, lane);
            if ((lane & ((32 / NPP) - 1)) == 0) gpart[warp * 64 + base] = pr[0];
        }
    }
    sync();
    if (tid < 128) {
        float g[R][R];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c <= r; ++c) {
                const int k = MMA_GRAM ? r * 8 + c : r * (r + 1) / 2 + c;
                g[r][c] = (gpart[k] + gpart[64 + k]) + (gpart[128 + k] + gpart[192 + k]);
            }
        // Cholesky G = L L^T, column by column: once column j is final, its products are subtracted from everything to its
        // right.  Each entry still receives its subtractions in the order m = 0, 1, ..., so the result is the one of the usual
        // row-by-row recurrence, but the operations of a step are independent of one another.
        float gd[R], inv[R];
#pragma unroll
        for (int j = 0; j < R; ++j) gd[j] = g[j][j];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const float d = g[j][j];
            if (DROP) inv[j] = (d > 1e-6f * gd[j] + 1e-30f) ? rsqrtf(fmaxf(d, 1e-30f)) : 0.f;
            else inv[j] = rsqrtf(fmaxf(fmaxf(d, 1e-6f * gd[j]), 1e-30f));
#pragma unroll
            for (int i = j + 1; i < R; ++i) g[i][j] *= inv[j];                   // l[i][j]
#pragma unroll
            for (int i = j + 1; i < R; ++i)
#pragma unroll
                for (int k = j + 1; k <= i; ++k) g[i][k] -= g[i][j] * g[k][j];
        }
        // X <- X L^-T by forward substitution on the thread's own row, likewise column by column
#pragma unroll
        for (int m = 0; m < R; ++m) {
            x[m] *= inv[m];
#pragma unroll
            for (int j = m + 1; j < R; ++j) x[j] -= x[m] * g[j][m];
        }
    }
}

// Arguments of the flush of one head (plain pointers: the fused decode kernel flushes heads whose window rows it -- or, with
// the mailboxes, ANOTHER CTA of the same launch -- wrote a moment before: none of them may be read through the
// non-coherent path, and what the step writes (window rows, weights, decay) is read with ld.global.cg, past the L1 of an SM
// that may hold an older copy of a line it shares with a neighbouring head).
struct FlushArgs {
    lq_dims d;
    char* ssm;
    const uint16_t* Kbuf;
    const uint16_t* Ubuf;
    float* Wbuf;
    float* Pbuf;
    uint16_t* Gbuf;
    int32_t* hcnt;
    const float* Q0;
    int iters;
};

template <int R>
__device__ __forceinline__ FlushSmem flush_carve(char* p0, int L, bool kda) {
    constexpr int KS = FlushK<R>::KS;
    FlushSmem s;
    const int Lp = flush_lp(L);
    char* p = p0 + ((1024u - (smem_u32(p0) & 1023u)) & 1023u);       // region 1 on a 1 KB boundary (swizzle atoms)
    s.tile[0] = p;
    s.tile[1] = p + Lp * 256;
    s.tile[2] = p + 2 * Lp * 256;
    s.tab = reinterpret_cast<float*>(p + 3 * Lp * 256);
    s.Bh = reinterpret_cast<uint16_t*>(p);
    s.Ac = s.Bh + 128 * TS;
    s.Bc = s.Ac + 128 * KS;
    s.colpart = reinterpret_cast<float*>(s.Bc + 128 * KS);
    s.Qn = s.colpart + 8 * 128;
    s.gpart = s.Qn + 128 * R;
    s.rowmax = s.gpart + 4 * 64;
    p += flush_region1_bytes<R>(L, kda);
    s.segprod = reinterpret_cast<float*>(p); p += 4 * 128 * 4;
    s.Q0h = reinterpret_cast<uint16_t*>(p); p += R * HS * 2;
    s.Qh = reinterpret_cast<uint16_t*>(p); p += R * HS * 2;
    s.Ph = reinterpret_cast<uint16_t*>(p); p += R * HS * 2;
    s.Qoh = reinterpret_cast<uint16_t*>(p); p += R * HS * 2;
    s.Uoh = reinterpret_cast<uint16_t*>(p); p += R * HS * 2;
    s.QoT = reinterpret_cast<uint16_t*>(p); p += 128 * 8 * 2;
    s.UoT = reinterpret_cast<uint16_t*>(p); p += 128 * 8 * 2;
    s.sk = reinterpret_cast<float*>(p); p += 128 * 4;
    s.sv = reinterpret_cast<float*>(p); p += 128 * 4;
    s.pc = reinterpret_cast<float*>(p); p += 128 * 4;
    s.w = reinterpret_cast<float*>(p); p += 64 * 4;
    s.mbar = reinterpret_cast<uint64_t*>(p); p += 8;
    s.flags = reinterpret_cast<int*>(p); p += 4 * 4;
    s.dlist = reinterpret_cast<int*>(p);
    return s;
}

// Once per team, before its first head: the zero padding of the transposed old factors, the f16 start Q0 of the iteration
// (leapquant/kernels.py:1573-1577) and the completion barrier of the tensor-core instructions.  The caller synchronises.
template <int R>
__device__ __forceinline__ void flush_init(const FlushSmem& s, const float* Q0, int tid, int nthreads) {
    if constexpr (R < 8) {
        for (int i = tid; i < 128 * (8 - R); i += nthreads) {
            const int c = i / (8 - R), r = R + i % (8 - R);
            s.UoT[c * 8 + r] = 0;
            s.QoT[c * 8 + r] = 0;
        }
    }
    if (tid == 0) {
        mbar_init(s.mbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s.flags[0] = 0;
        s.flags[1] = 1;
    }
}

// The flush of head q = slot * HV + hv by a team of NW warps (tid 0 .. 32 NW - 1); sync() is the team's barrier; `tm` is the
// team's tensor-memory base (128 columns).  Returns false if the wait for the tensor cores ran out (status word set): the
// caller then stops flushing.
template <int R, bool KDA, int NW, typename Sync>
__device__ __forceinline__ bool flush_head(const FlushSmem& s, const FlushArgs& A, int q, int tid, uint32_t tm, Sync sync) {
    constexpr int KC = FlushK<R>::KC, KS = FlushK<R>::KS;
    constexpr int NT = 32 * NW;
    constexpr int NH = NW / 8;                                  // column halves the team splits the tile stages into
    constexpr int NTW = 16 / NH;                                // n-tiles (8 columns) per warp in the residual and INT8 stages
    const lq_dims& d = A.d;
    char* ssm = A.ssm;
    const uint16_t* Kbuf = A.Kbuf;
    const uint16_t* Ubuf = A.Ubuf;
    float* Wbuf = A.Wbuf;
    float* Pbuf = A.Pbuf;
    uint16_t* Gbuf = A.Gbuf;
    int32_t* hcnt = A.hcnt;
    const int iters = A.iters;
    const int L = d.L, HV = d.HV, Lp = flush_lp(d.L);
    const int warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    const int slot = q / HV, hv = q - slot * HV;
    const int64_t sh = q;
    char* base = head_base(ssm, d.SS, slot, hv);
    float p = 1.f;
    if (!KDA) p = fmaxf(__ldcg(Pbuf + sh), PNMIN);

    // ---- stage A: operands to shared memory; every global load of the stage is issued before the first store so that
    //      their latencies overlap.  The window rows go straight into the tensor-core operand tiles. ----
    {
        const uint16_t* uq = reinterpret_cast<const uint16_t*>(base + CK_UQ);
        const uint4* kb = reinterpret_cast<const uint4*>(Kbuf + sh * L * KD);
        const uint4* ub = reinterpret_cast<const uint4*>(Ubuf + sh * L * VD);
        constexpr int NF = (R * 128 + NT - 1) / NT;         // factor elements per thread
        constexpr int NTC = 64 * 16 / NT;                   // window-row chunks (16 bytes) per thread (Lp <= 64)
        float wv = 0.f, pcv = 1.f, skv = 0.f, svv = 0.f, pcf[NF], wrow[NTC];
        uint16_t fu[NF], fq[NF];
        float q0v[NF];                                      // the fixed start Q0 of the iteration: fetched with the head's other operands
        uint4 tk[NTC], tu[NTC], tg[KDA ? NTC : 1];
        const uint4* gbc = reinterpret_cast<const uint4*>(Gbuf + (KDA ? sh * L * KD : 0));
        if (tid < L) wv = __ldcg(Wbuf + sh * L + tid);
        if (tid < 128) {
            if (KDA) pcv = __ldcg(Pbuf + sh * KD + tid);
            skv = reinterpret_cast<const float*>(base + CK_SK)[tid];
            svv = reinterpret_cast<const float*>(base + CK_SV)[tid];
        }
#pragma unroll
        for (int u = 0; u < NF; ++u) {
            const int i = tid + u * NT, r = i >> 7, c = i & 127;
            const bool in = i < R * 128;
            fu[u] = in ? uq[r * (KD + VD) + c] : uint16_t(0);
            fq[u] = in ? uq[r * (KD + VD) + KD + c] : uint16_t(0);
            pcf[u] = (KDA && in) ? __ldcg(Pbuf + sh * KD + c) : 0.f;
            q0v[u] = in ? __ldg(A.Q0 + i) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < NTC; ++u) {
            const int i = tid + u * NT;
            const bool in = i < L * 16;
            tk[u] = in ? __ldcg(kb + i) : make_uint4(0u, 0u, 0u, 0u);
            tu[u] = in ? __ldcg(ub + i) : make_uint4(0u, 0u, 0u, 0u);
            wrow[u] = (!KDA && in) ? __ldcg(Wbuf + sh * L + (i >> 4)) : 0.f;
            if (KDA) tg[u] = in ? __ldcg(gbc + i) : make_uint4(0u, 0u, 0u, 0u);
        }
        if (tid < L) s.w[tid] = wv;
        if (tid < 128) {
            pcv = KDA ? expf(pcv) : 1.f;
            s.pc[tid] = pcv;
            s.sk[tid] = skv * pcv;
            s.sv[tid] = svv;
        }
        // old factors as stored (f16); KDA: U^T times pc, rounded to f16.  Kept as rows [r][128] and transposed [128][8].
#pragma unroll
        for (int u = 0; u < NF; ++u) {
            const int i = tid + u * NT, r = i >> 7, c = i & 127;
            if (i < R * 128) {
                uint16_t uu = fu[u];
                if (KDA) uu = f_to_f16(f16_to_f(uu) * expf(pcf[u]));
                s.Uoh[r * HS + c] = uu;
                s.Qoh[r * HS + c] = fq[u];
                s.UoT[c * 8 + r] = uu;
                s.QoT[c * 8 + r] = fq[u];
                s.Q0h[(i % R) * HS + i / R] = f_to_f16(q0v[u]);      // Q0 is [128][R] row-major; kept transposed as f16
            }
        }
        // window rows -> operand tiles (rows L .. Lp-1 are zero).  GDN: tile 0 / 1 = head / remainder of w_j u_j, tile 2 = keys.
        // KDA: tile 0 = values, tile 1 = keys as stored for now (scaled and split below, once their scales are known).
#pragma unroll
        for (int u = 0; u < NTC; ++u) {
            const int i = tid + u * NT;
            if (i < Lp * 16) {
                const int j = i >> 4, c16 = i & 15;
                const uint32_t off = tile_chunk_offset(Lp, j, c16);
                if (KDA) {
                    *reinterpret_cast<uint4*>(s.tile[0] + off) = tu[u];
                    *reinterpret_cast<uint4*>(s.tile[1] + off) = tk[u];
                    if (j < L) {                            // the row's step factors e_j[c], as fp32, where the key scales will be
                        const float2 e0 = f16x2_to_f2(tg[u].x), e1 = f16x2_to_f2(tg[u].y), e2 = f16x2_to_f2(tg[u].z), e3 = f16x2_to_f2(tg[u].w);
                        float4* tp = reinterpret_cast<float4*>(s.tab + j * 128 + c16 * 8);
                        tp[0] = make_float4(e0.x, e0.y, e1.x, e1.y);
                        tp[1] = make_float4(e2.x, e2.y, e3.x, e3.y);
                    }
                } else {
                    const float sc[8] = {wrow[u], wrow[u], wrow[u], wrow[u], wrow[u], wrow[u], wrow[u], wrow[u]};
                    uint4 hi, lo;
                    scale_split_chunk(tu[u], sc, hi, lo);
                    *reinterpret_cast<uint4*>(s.tile[0] + off) = hi;
                    *reinterpret_cast<uint4*>(s.tile[1] + off) = lo;
                    *reinterpret_cast<uint4*>(s.tile[2] + off) = tk[u];
                }
            }
        }
    }
    if (KDA) {
        // key scale w_j D_j[c] with D_{L-1} = 1, D_j = D_{j+1} e_{j+1}, in place over the step factors: the L rows are cut into
        // four segments (L % 4 == 0), a thread takes one column of one segment (of two, in a team of 8 warps); first the
        // product of each segment's factors, then the running products.  The order of the multiplications does not depend
        // on the size of the team.
        sync();                                             // the step factors are in shared memory
        constexpr int SPT = 4 * 128 / NT;                   // segments per thread
        const int c = tid & 127, slen = L >> 2;
#pragma unroll
        for (int q2 = 0; q2 < SPT; ++q2) {
            const int seg = (tid >> 7) + q2 * (NT / 128);
            float ev[16], prod = 1.f;
#pragma unroll
            for (int k = 0; k < 16; ++k) ev[k] = (k < slen) ? s.tab[((seg + 1) * slen - 1 - k) * 128 + c] : 1.f;
#pragma unroll
            for (int k = 0; k < 16; ++k) prod *= ev[k];
            s.segprod[seg * 128 + c] = prod;
        }
        sync();
#pragma unroll
        for (int q2 = 0; q2 < SPT; ++q2) {
            const int seg = (tid >> 7) + q2 * (NT / 128);
            float dcur = 1.f;
#pragma unroll
            for (int s2 = 3; s2 > 0; --s2)
                if (s2 > seg) dcur *= s.segprod[s2 * 128 + c];
            float ev[16], wv2[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int j = (seg + 1) * slen - 1 - k;
                ev[k] = (k < slen) ? s.tab[j * 128 + c] : 1.f;
                wv2[k] = (k < slen) ? s.w[j] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                if (k < slen) s.tab[((seg + 1) * slen - 1 - k) * 128 + c] = wv2[k] * dcur;
                dcur *= ev[k];
            }
        }
        sync();
        // keys times their scale, as head (tile 1) and remainder (tile 2); a thread rewrites the chunks it wrote above
        constexpr int NTC = 64 * 16 / NT;
#pragma unroll
        for (int u = 0; u < NTC; ++u) {
            const int i = tid + u * NT;
            if (i < Lp * 16) {
                const int j = i >> 4, c16 = i & 15;
                const uint32_t off = tile_chunk_offset(Lp, j, c16);
                uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
                if (j < L) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(s.tile[1] + off);
                    const float4 t0 = *reinterpret_cast<const float4*>(s.tab + j * 128 + c16 * 8);
                    const float4 t1 = *reinterpret_cast<const float4*>(s.tab + j * 128 + c16 * 8 + 4);
                    const float sc[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
                    scale_split_chunk(raw, sc, hi, lo);
                }
                *reinterpret_cast<uint4*>(s.tile[1] + off) = hi;
                *reinterpret_cast<uint4*>(s.tile[2] + off) = lo;
            }
        }
    }
    fence_async_smem();                                    // the tiles were written through the generic proxy; the tensor cores read them through the asynchronous one
    sync();

    // ---- stage B: B = deq(checkpoint) * decay + sum_j (w_j u_j) k_j^T.  One thread issues the tensor-core instructions
    //      (two passes of Lp / 16 instructions of M = N = 128, K = 16: head and remainder of the scaled operand) and waits
    //      for their completion; the others fetch their share of the INT8 codes meanwhile.  Thread (warp, lane) then owns
    //      row v = 32 (warp % 4) + lane of the accumulator and the CPW columns starting at CPW (warp / 4). ----
    constexpr int CPW = 128 / (NW / 4);
    const int vrow = 32 * (warp & 3) + lane, col0 = CPW * (warp >> 2);
    uint4 cpre[CPW / 16];
    {
        const uint4* crow = reinterpret_cast<const uint4*>(base + CK_CODES + vrow * KD + col0);
#pragma unroll
        for (int i = 0; i < CPW / 16; ++i) cpre[i] = crow[i];
    }
    if (tid == 0) {
        tc_fence_after_sync();
        const uint64_t da0 = umma_desc(s.tile[0], Lp), da1 = umma_desc(KDA ? s.tile[0] : s.tile[1], Lp);
        const uint64_t db0 = umma_desc(KDA ? s.tile[1] : s.tile[2], Lp), db1 = umma_desc(s.tile[2], Lp);
        const int nk = Lp >> 4;
        // one K step = 16 rows j = two swizzle atoms of eight rows = 2 048 bytes = 128 units of the descriptor's address field
        for (int ks = 0; ks < nk; ++ks) umma_bf16_ss(tm, da0 + uint64_t(ks) * 128u, db0 + uint64_t(ks) * 128u, UMMA_IDESC, ks > 0);
        for (int ks = 0; ks < nk; ++ks) umma_bf16_ss(tm, da1 + uint64_t(ks) * 128u, db1 + uint64_t(ks) * 128u, UMMA_IDESC, 1u);
        umma_commit(s.mbar);
        const uint32_t ph = uint32_t(s.flags[0]);
        bool ok = false;
        for (uint32_t it = 0; it < WAIT_LIMIT && !ok; ++it) ok = mbar_try_wait(s.mbar, ph);
        s.flags[0] = int(ph ^ 1u);
        s.flags[1] = ok ? 1 : 0;
        if (!ok) atomicOr(&g_status, ST_FLUSH_TIMEOUT);
    }
    sync();
    if (s.flags[1] == 0) return false;                     // uniform: the whole team leaves
    tc_fence_after_sync();
    {
        const float pq = KDA ? (1.0f / QMAX) : (p / QMAX);
        const float svr = s.sv[vrow] * pq;
#pragma unroll
        for (int ch = 0; ch < CPW / 32; ++ch) {
            uint32_t acc[32];
            tmem_ld_32cols(tm + (uint32_t(32 * (warp & 3)) << 16) + uint32_t(col0 + 32 * ch), acc);
            tmem_ld_wait();
            uint32_t outw[16];
#pragma unroll
            for (int g4 = 0; g4 < 8; ++g4) {                // four codes = four columns at a time
                const uint4 cw4 = cpre[2 * ch + (g4 >> 2)];
                const uint32_t cw = (g4 & 3) == 0 ? cw4.x : (g4 & 3) == 1 ? cw4.y : (g4 & 3) == 2 ? cw4.z : cw4.w;
                float f0, f1, f2, f3;
                s8x4_to_f4(cw, f0, f1, f2, f3);
                const float4 sk4 = *reinterpret_cast<const float4*>(s.sk + col0 + 32 * ch + 4 * g4);
                const float o0 = (f0 * svr) * sk4.x + __uint_as_float(acc[4 * g4]);
                const float o1 = (f1 * svr) * sk4.y + __uint_as_float(acc[4 * g4 + 1]);
                const float o2 = (f2 * svr) * sk4.z + __uint_as_float(acc[4 * g4 + 2]);
                const float o3 = (f3 * svr) * sk4.w + __uint_as_float(acc[4 * g4 + 3]);
                outw[2 * g4] = pack_h2(o0, o1);
                outw[2 * g4 + 1] = pack_h2(o2, o3);
            }
            uint4* dst = reinterpret_cast<uint4*>(s.Bh + vrow * TS + col0 + 32 * ch);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(outw[4 * i], outw[4 * i + 1], outw[4 * i + 2], outw[4 * i + 3]);
        }
    }
    tc_fence_before_sync();                                // the accumulator has been read: the next head may overwrite it
    sync();                                                // the operand tiles are dead: region 1 now holds B and the later operands

    // ---- stage C: subspace iteration on T = B + p Q_old U_old^T (warps 0..7 compute the products) ----
    const int m0w = (warp & 7) * 16;
    float dd[4] = {0.f, 0.f, 0.f, 0.f};
    auto store_p = [&] {                                    // P (rounded to f16) as rows [r][c]
        if (2 * tig < R) {
            s.Ph[(2 * tig) * HS + m0w + gid] = f_to_f16(dd[0]);
            s.Ph[(2 * tig + 1) * HS + m0w + gid] = f_to_f16(dd[1]);
            s.Ph[(2 * tig) * HS + m0w + gid + 8] = f_to_f16(dd[2]);
            s.Ph[(2 * tig + 1) * HS + m0w + gid + 8] = f_to_f16(dd[3]);
        }
    };
    if (warp < 8) {
        tall_product<R, true>(s.Bh, s.Q0h, s.Qoh, s.UoT, p, warp, lane, dd);        // P = T^T Q0
        store_p();
    }
    sync();
    if (iters == 0) {                                       // no round: the stored Q is the start itself
        for (int i = tid; i < R * HS; i += NT) s.Qh[i] = s.Q0h[i];
        sync();
    }
    for (int it = 0; it < iters; ++it) {
        if (warp < 8) {
            tall_product<R, false>(s.Bh, s.Ph, s.Uoh, s.QoT, p, warp, lane, dd);    // Q = T P
            if (2 * tig < R) {
                *reinterpret_cast<float2*>(s.Qn + (m0w + gid) * R + 2 * tig) = make_float2(dd[0], dd[1]);
                *reinterpret_cast<float2*>(s.Qn + (m0w + gid + 8) * R + 2 * tig) = make_float2(dd[2], dd[3]);
            }
        }
        sync();
        {   // CholeskyQR twice in fp32 (leapquant/kernels.py:1741-1835), thread = row; the result rounded to f16 is the new Q
            float x[R];
#pragma unroll
            for (int r = 0; r < R; ++r) x[r] = (tid < 128) ? s.Qn[tid * R + r] : 0.f;
            cholqr_pass_team<R, (R > 4)>(x, s.Qn, true, s.gpart, tid, sync);
            sync();                                         // the Gram matrix is read: the second pass may overwrite it
            cholqr_pass_team<R, (R > 4)>(x, s.Qn, false, s.gpart, tid, sync);
            if (tid < 128) {
#pragma unroll
                for (int r = 0; r < R; ++r) s.Qh[r * HS + tid] = f_to_f16(x[r]);
            }
        }
        sync();
        if (warp < 8) {
            tall_product<R, true>(s.Bh, s.Qh, s.Qoh, s.UoT, p, warp, lane, dd);     // P = T^T Q
            store_p();
        }
        sync();
    }

    // ---- stage D: new factors to the checkpoint (16-byte copies of the f16 rows); operands of the residual ----
    if (tid < R * 32) {
        const int r = tid >> 5, j = tid & 31;
        const uint16_t* src = (j < 16) ? s.Ph + r * HS + j * 8 : s.Qh + r * HS + (j - 16) * 8;
        reinterpret_cast<uint4*>(base + CK_UQ)[r * 32 + j] = *reinterpret_cast<const uint4*>(src);
    }
    if (tid < 128) {
        uint16_t* row = s.Ac + tid * KS;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            row[r] = s.Qh[r * HS + tid];
            const float x = p * f16_to_f(s.Qoh[r * HS + tid]);
            const uint16_t hi = f_to_f16(x);
            row[R + r] = hi;
            row[2 * R + r] = f_to_f16(x - f16_to_f(hi));
        }
#pragma unroll
        for (int c = 3 * R; c < KC; ++c) row[c] = 0;
    } else if (tid < 256) {
        const int c = tid - 128;
        uint16_t* row = s.Bc + c * KS;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            row[r] = s.Ph[r * HS + c] ^ 0x8000u;
            row[R + r] = row[2 * R + r] = s.Uoh[r * HS + c];
        }
#pragma unroll
        for (int c2 = 3 * R; c2 < KC; ++c2) row[c2] = 0;
    }
    sync();

    // ---- stage E: residual E = B + p Q_old U_old^T - Q U^T on the tensor cores (mma.sync), fp32 in registers: a warp owns
    //      rows m0w .. m0w + 15 and the NTW n-tiles from nt0 on; lane (gid, tig) holds rows gid, gid + 8 at columns
    //      8 nt + 2 tig, + 1 ----
    const int nt0 = (warp >> 3) * NTW;
    float e[NTW][4];
    {
        const uint16_t* b0p = s.Bh + (m0w + gid) * TS + 8 * nt0 + 2 * tig;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const float2 lo = unpack_h2(*reinterpret_cast<const uint32_t*>(b0p + 8 * nt));
            const float2 hi = unpack_h2(*reinterpret_cast<const uint32_t*>(b0p + 8 * TS + 8 * nt));
            e[nt][0] = lo.x; e[nt][1] = lo.y; e[nt][2] = hi.x; e[nt][3] = hi.y;
        }
#pragma unroll
        for (int ks = 0; ks < KC; ks += 16) {
            const uint16_t* ap = s.Ac + (m0w + gid) * KS + ks + 2 * tig;
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(ap), a1 = *reinterpret_cast<const uint32_t*>(ap + 8 * KS);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(ap + 8), a3 = *reinterpret_cast<const uint32_t*>(ap + 8 * KS + 8);
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) {
                const uint16_t* bp = s.Bc + (8 * (nt0 + nt) + gid) * KS + ks + 2 * tig;
                mma_h_16816(e[nt], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(bp), *reinterpret_cast<const uint32_t*>(bp + 8));
            }
        }
    }
    // column sums of |E|: 2 NTW partial sums per lane (two rows each), folded over the eight row groups of the warp by
    // three exchange levels that halve the number of values a lane keeps
    {
        float cs[2 * NTW];
#pragma unroll
        for (int i = 0; i < 2 * NTW; ++i) cs[i] = fabsf(e[i >> 1][i & 1]) + fabsf(e[i >> 1][2 + (i & 1)]);
        int ntb = 0;
        int n = 2 * NTW;
#pragma unroll
        for (int off = 16; off >= 4; off >>= 1) {
            const int half = n >> 1;
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < NTW; ++i) {
                if (i < half) {
                    const float keep = up ? cs[half + i] : cs[i];
                    const float send = up ? cs[i] : cs[half + i];
                    cs[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            if (up) ntb += half >> 1;
            n = half;
        }
        // n = NTW / 4 values: NTW / 8 n-tiles from ntb on, two columns each
#pragma unroll
        for (int t2 = 0; t2 < NTW / 8; ++t2)
            *reinterpret_cast<float2*>(s.colpart + (warp & 7) * 128 + 8 * (nt0 + ntb + t2) + 2 * tig) = make_float2(cs[2 * t2], cs[2 * t2 + 1]);
    }
    sync();
    if (tid < 128) {
        float m = 0.f;
#pragma unroll
        for (int t2 = 0; t2 < 8; ++t2) m += s.colpart[t2 * 128 + tid];
        m *= (1.0f / float(VD));
        const float skn = fmaxf(sqrtf(m), EPS);
        reinterpret_cast<float*>(base + CK_SK)[tid] = skn;
        s.sk[tid] = 1.0f / skn;                           // reciprocal of the STORED scale
    }
    sync();

    // ---- stage F: row scales and INT8 codes, staged in the warp's own part of the (dead) state tile ----
    {
        float r0 = 0.f, r1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const float2 rk = *reinterpret_cast<const float2*>(s.sk + 8 * (nt0 + nt) + 2 * tig);
            e[nt][0] *= rk.x; e[nt][1] *= rk.y; e[nt][2] *= rk.x; e[nt][3] *= rk.y;
            r0 = fmaxf(r0, fmaxf(fabsf(e[nt][0]), fabsf(e[nt][1])));
            r1 = fmaxf(r1, fmaxf(fabsf(e[nt][2]), fabsf(e[nt][3])));
        }
        r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 1)); r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 1));
        r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 2)); r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 2));
        if constexpr (NH > 1) {                             // the row's other columns belong to another warp
            if (tig == 0) {
                s.rowmax[(warp >> 3) * 128 + m0w + gid] = r0;
                s.rowmax[(warp >> 3) * 128 + m0w + gid + 8] = r1;
            }
            sync();
            r0 = fmaxf(s.rowmax[m0w + gid], s.rowmax[128 + m0w + gid]);
            r1 = fmaxf(s.rowmax[m0w + gid + 8], s.rowmax[128 + m0w + gid + 8]);
        }
        const float sv0 = fmaxf(r0, EPS), sv1 = fmaxf(r1, EPS);
        const float rm0 = QMAX * __frcp_rn(sv0), rm1 = QMAX * __frcp_rn(sv1);
        if (tig == 0 && warp < 8) {
            float* svg = reinterpret_cast<float*>(base + CK_SV);
            svg[m0w + gid] = sv0;
            svg[m0w + gid + 8] = sv1;
        }
        char* cw = reinterpret_cast<char*>(s.Bh) + (m0w + gid) * (TS * 2) + 8 * nt0 + 2 * tig;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            const uint32_t lo = __byte_perm(rne_code(e[nt][0], rm0), rne_code(e[nt][1], rm0), 0x0040);
            const uint32_t hi = __byte_perm(rne_code(e[nt][2], rm1), rne_code(e[nt][3], rm1), 0x0040);
            *reinterpret_cast<uint16_t*>(cw + 8 * nt) = uint16_t(lo);
            *reinterpret_cast<uint16_t*>(cw + 8 * (TS * 2) + 8 * nt) = uint16_t(hi);
        }
        __syncwarp();
        // the warp's 16 rows x 8 NTW bytes, two lanes per row
        const int row = m0w + (lane >> 1), part = lane & 1;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(s.Bh) + row * (TS * 2) + 8 * nt0 + part * (4 * NTW));
        uint4* dst = reinterpret_cast<uint4*>(base + CK_CODES + row * KD + 8 * nt0 + part * (4 * NTW));
#pragma unroll
        for (int i = 0; i < NTW / 4; ++i) dst[i] = src[i];
    }
    // ---- stage G: window reset ----
    if (tid < L) Wbuf[sh * L + tid] = 0.f;
    if (KDA) {
        if (tid < 128) Pbuf[sh * KD + tid] = 0.f;
        uint32_t* g32 = reinterpret_cast<uint32_t*>(Gbuf + sh * L * KD);
        for (int i = tid; i < L * KD / 2; i += NT) g32[i] = 0x3C003C00u;
    } else if (tid == 0) {
        Pbuf[sh] = 1.f;
    }
    if (tid == 0) hcnt[sh] = 0;
    sync();
    return true;
}

template <int R, bool KDA>
__global__ void __launch_bounds__(NT_LA, 2)
flush_kernel(lq_dims d, char* ssm, const uint16_t* Kbuf, const uint16_t* Ubuf, float* Wbuf, float* Pbuf, uint16_t* Gbuf,
             int32_t* hcnt, const float* __restrict__ Q0, const int32_t* __restrict__ idx, int N, int iters, int maxd) {
    extern __shared__ __align__(128) char flush_smem[];
    __shared__ uint32_t tm_slot;
    const FlushSmem s = flush_carve<R>(flush_smem, d.L, KDA);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, bid = blockIdx.x;
    const int L = d.L, HV = d.HV;
    pdl_trigger();
    pdl_wait();                                                  // the scan reads the counters the step kernel just wrote

    // ---------------- the due programs of this CTA ----------------
    // Program p = n * HV + hv belongs to CTA p % G, whatever the state of the windows: a CTA tests only its own programs and
    // reads each counter once, so the assignment does not depend on counters that other CTAs reset while they work, nor
    // on all CTAs being resident at the same time.  Warp 0 compacts the due ones in program order.
    const int total = N * HV;
    const int nmine = (total > bid) ? (total - bid + G - 1) / G : 0;
    if (warp == 0) {
        int nb = 0;
        const uint32_t lt = (1u << lane) - 1u;
        for (int b0 = 0; b0 < nmine; b0 += 32) {
            const int i = b0 + lane;
            int q = 0;
            bool f = false;
            if (i < nmine) {
                const int pgm = bid + i * G;
                const int n = pgm / HV, hv = pgm - n * HV;
                const int slot = idx[n];
                if (slot > 0 && slot < d.NS) {
                    q = slot * HV + hv;
                    f = hcnt[q] == L;
                }
            }
            const uint32_t m = __ballot_sync(0xffffffffu, f);
            if (f) s.dlist[nb + __popc(m & lt)] = q;
            nb += __popc(m);
        }
        if (lane == 0) s.flags[2] = nb;
    }
    __syncthreads();
    const int mine = min(s.flags[2], maxd);
    if (mine == 0) return;                                       // (before any tensor memory is held)

    if (warp == 0) tmem_alloc(&tm_slot, TMEM_COLS);
    flush_init<R>(s, Q0, tid, NT_LA);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tm = tm_slot;
    FlushArgs A;
    A.d = d; A.ssm = ssm; A.Kbuf = Kbuf; A.Ubuf = Ubuf; A.Wbuf = Wbuf; A.Pbuf = Pbuf; A.Gbuf = Gbuf; A.hcnt = hcnt; A.Q0 = Q0;
    A.iters = iters;
    for (int k = 0; k < mine; ++k)
        if (!flush_head<R, KDA, 8>(s, A, s.dlist[k], tid, tm, [] { __syncthreads(); })) break;
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tm, TMEM_COLS);
}

template <int R, bool KDA>
static int launch_flush(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                        int32_t* hcnt, const float* Q0, const int32_t* idx, int N, int iters, cudaStream_t st) {
    const int total = N * d->HV;
    // two CTAs per SM when the shared memory of one allows it: a flush is a chain of short phases, and a second head in
    // flight on the SM hides most of their latency
    int per_sm = 1;
    {
        const int g2 = min(2 * device_sm_count(), total);
        const size_t s2 = flush_smem_bytes<R>(d->L, (total + g2 - 1) / g2 + 1, KDA);
        if (s2 <= 113 * 1024) per_sm = 2;
    }
    const int G = min(per_sm * device_sm_count(), total);
    const int maxd = (total + G - 1) / G + 1;
    const size_t smem = flush_smem_bytes<R>(d->L, maxd, KDA);
    if (smem > 227 * 1024) return LQ_ERR_UNSUPPORTED;
    int rc = ensure_smem((const void*)flush_kernel<R, KDA>, smem);
    if (rc) return rc;
    cudaError_t le = launch_dependent(flush_kernel<R, KDA>, unsigned(G), unsigned(NT_LA), smem, st, *d, (char*)ssm, (const uint16_t*)Kbuf,
                                      (const uint16_t*)Ubuf, Wbuf, Pbuf, (uint16_t*)Gbuf, hcnt, Q0, idx, N, iters, maxd);
    if (le != cudaSuccess) { set_last_cuda_error(le); return LQ_ERR_LAUNCH; }
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
    if (misaligned16({ssm, Kbuf, Ubuf, Wbuf}) || (kda && misaligned16({Gbuf, Pbuf}))) return LQ_ERR_ALIGN;
    if (N == 0) return LQ_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->R == 4)
        return kda ? launch_flush<4, true>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st)
                   : launch_flush<4, false>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st);
    return kda ? launch_flush<8, true>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st)
               : launch_flush<8, false>(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, iters, st);
}
