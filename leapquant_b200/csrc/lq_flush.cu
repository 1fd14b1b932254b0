// Window-flush kernel (sm_100a): rebuild -> rank-R subspace iteration -> residual -> smoothing scales -> INT8.
//
// Persistent CTAs of 256 threads, two per SM.  Program p = row * HV + head belongs to CTA p % grid; a CTA tests the window
// counters of its own programs and flushes the due ones, so the launch shape never depends on device data and no CTA
// relies on what another one reads or resets.
//
// All matrix products of a head run on the tensor cores (mma.sync m16n8k16, fp32 accumulate): the window product that
// rebuilds the state B (bf16 operands, the scaled one as head + remainder), the tall-skinny products of the subspace
// iteration with their rank-R corrections, and the residual.  B lives in shared memory as an f16 tile like the
// reference's (leapquant/kernels.py:1156,1483); the residual E stays in registers in fp32 until it has become codes.
#include "lq_linalg.cuh"

namespace lq {

constexpr int TS = 136;          // row stride (16-bit elements) of the window tiles and of the f16 state tile: 272 B moves
                                 // every row one 16-byte bank group on, so ldmatrix and fragment loads are conflict-free
constexpr int HS = TS;           // row stride of the factor rows [r][128]

template <int R> struct FlushK { static constexpr int KC = (R == 4) ? 16 : 32, KS = KC + 8; };  // residual operand rows

struct FlushSmem {
    uint16_t* Bh;      // [128][TS] f16 state tile B[v][c]; at the end a warp's 16 rows hold its int8 codes for the coalesced store
    uint16_t* Kt;      // [Lp][TS] window keys, bf16 as stored (rows L.. zero)
    uint16_t* Ut;      // [Lp][TS] window values, bf16 as stored (rows L.. zero)
    // the window tiles are dead after the rebuild; the region then holds:
    uint16_t* Ac;      // [128][KS] f16 residual operand, row v:  Q | p Q_old head | p Q_old remainder | 0
    uint16_t* Bc;      // [128][KS] f16 residual operand, row c: -U |   U_old      |   U_old           | 0
    float* colpart;    // [8][128] per-warp column sums of |E|
    float* Qn;         // [128][R] fp32 Q for CholeskyQR
    float* tab;        // KDA: [L][128] scale of key (j, c): w_j D_j[c]
    uint16_t* Q0h;     // [R][HS] f16 Q0^T, the fixed start of the iteration (written once per CTA)
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
    int* wcnt;         // [8]
    int* dlist;        // [maxd]
};

__host__ __device__ inline int flush_lp(int L) { return (L + 15) & ~15; }
// bytes of the region shared by the window tiles (rebuild) and Ac + Bc + colpart + Qn (afterwards)
template <int R>
__host__ __device__ inline int flush_region_bytes(int L) {
    const int tiles = 2 * flush_lp(L) * TS * 2;
    const int later = 2 * 128 * FlushK<R>::KS * 2 + 8 * 128 * 4 + 128 * R * 4;
    return tiles > later ? tiles : later;
}
template <int R>
__host__ __device__ inline size_t flush_smem_bytes(int L, int maxd, bool kda) {
    return size_t(128) * TS * 2 + flush_region_bytes<R>(L) + (kda ? size_t(L) * 128 * 4 : 0) + 5 * R * HS * 2 + 2 * 128 * 8 * 2 +
           3 * 128 * 4 + 64 * 4 + 8 * 4 + size_t(maxd) * 4 + 16;
}

// ---- warp-level tensor-core helpers (mma.sync path) ----
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_h_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = uint32_t(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
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
// x (fp32) ~ hi + lo as two bf16 pieces (16 mantissa bits, relative error 2^-17): the split the reference uses for the
// same operand (reference leapquant/kernels.py:1508-1511).  The tensor pipe bounds the rebuild, so a third piece
// would cost 50 % more time for accuracy far below the INT8 step.
__device__ __forceinline__ void split2(float x, float& hi, float& lo) {
    hi = round_bf16(x);
    lo = round_bf16(x - hi);
}

// One tall-skinny product of the subspace iteration with its rank-R correction, all eight warps, all in registers:
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

// Arguments of the flush of one head (plain pointers: the fused decode kernel flushes heads whose window rows it wrote
// itself a moment before, so none of them may be read through the non-coherent path).
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
__device__ __forceinline__ FlushSmem flush_carve(char* p, int L, bool kda) {
    constexpr int KS = FlushK<R>::KS;
    FlushSmem s;
    const int Lp = flush_lp(L);
    s.Bh = reinterpret_cast<uint16_t*>(p); p += 128 * TS * 2;
    s.Kt = reinterpret_cast<uint16_t*>(p);
    s.Ut = s.Kt + Lp * TS;
    s.Ac = reinterpret_cast<uint16_t*>(p);
    s.Bc = s.Ac + 128 * KS;
    s.colpart = reinterpret_cast<float*>(s.Bc + 128 * KS);
    s.Qn = s.colpart + 8 * 128;
    p += flush_region_bytes<R>(L);
    s.tab = reinterpret_cast<float*>(p); p += kda ? L * 128 * 4 : 0;
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
    s.wcnt = reinterpret_cast<int*>(p); p += 8 * 4;
    s.dlist = reinterpret_cast<int*>(p);
    return s;
}

// Once per team of 256 threads, before its first head: the zero padding of the transposed old factors and the f16 start
// Q0 of the iteration (leapquant/kernels.py:1573-1577).  The first sync() of flush_head orders these writes.
template <int R>
__device__ __forceinline__ void flush_init(const FlushSmem& s, const float* Q0, int tid) {
    if constexpr (R < 8) {
        for (int i = tid; i < 128 * (8 - R); i += NT_LA) {
            const int c = i / (8 - R), r = R + i % (8 - R);
            s.UoT[c * 8 + r] = 0;
            s.QoT[c * 8 + r] = 0;
        }
    }
    for (int i = tid; i < 128 * R; i += NT_LA) s.Q0h[(i % R) * HS + i / R] = f_to_f16(Q0[i]);
}

// The flush of head q = slot * HV + hv by a team of 256 threads (tid 0 .. 255); sync() is the team's barrier.
template <int R, bool KDA, typename Sync>
__device__ __forceinline__ void flush_head(const FlushSmem& s, const FlushArgs& A, int q, int tid, Sync sync) {
    constexpr int KC = FlushK<R>::KC, KS = FlushK<R>::KS;
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
    if (!KDA) p = fmaxf(Pbuf[sh], PNMIN);

    // ---- stage A: operands to shared memory; every global load of the stage is issued before the first store so that
    //      their latencies overlap (the stores would otherwise fence the loads behind them) ----
    {
        const uint16_t* uq = reinterpret_cast<const uint16_t*>(base + CK_UQ);
        const uint4* kb = reinterpret_cast<const uint4*>(Kbuf + sh * L * KD);
        const uint4* ub = reinterpret_cast<const uint4*>(Ubuf + sh * L * VD);
        constexpr int NF = R * 128 / NT_LA;                 // factor elements per thread
        constexpr int NTC = 4;                              // window-tile chunks per thread and pass (Lp <= 64)
        float wv = 0.f, pcv = 1.f, skv = 0.f, svv = 0.f, pcf[NF];
        uint16_t fu[NF], fq[NF];
        uint4 tk[NTC], tu[NTC];
        if (tid < L) wv = Wbuf[sh * L + tid];
        if (tid < 128) {
            if (KDA) pcv = Pbuf[sh * KD + tid];
            skv = reinterpret_cast<const float*>(base + CK_SK)[tid];
            svv = reinterpret_cast<const float*>(base + CK_SV)[tid];
        }
#pragma unroll
        for (int u = 0; u < NF; ++u) {
            const int i = tid + u * NT_LA, r = i >> 7, c = i & 127;
            fu[u] = uq[r * (KD + VD) + c];
            fq[u] = uq[r * (KD + VD) + KD + c];
            pcf[u] = KDA ? Pbuf[sh * KD + c] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < NTC; ++u) {
            const int i = tid + u * NT_LA;
            const bool in = i < L * 16;
            tk[u] = in ? kb[i] : make_uint4(0u, 0u, 0u, 0u);
            tu[u] = in ? ub[i] : make_uint4(0u, 0u, 0u, 0u);
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
            const int i = tid + u * NT_LA, r = i >> 7, c = i & 127;
            uint16_t uu = fu[u];
            if (KDA) uu = f_to_f16(f16_to_f(uu) * expf(pcf[u]));
            s.Uoh[r * HS + c] = uu;
            s.Qoh[r * HS + c] = fq[u];
            s.UoT[c * 8 + r] = uu;
            s.QoT[c * 8 + r] = fq[u];
        }
        // window rows as stored (bf16), 16 bytes at a time into the padded tiles; rows L .. Lp-1 are zero
#pragma unroll
        for (int u = 0; u < NTC; ++u) {
            const int i = tid + u * NT_LA;
            if (i < Lp * 16) {
                const int j = i >> 4, c8 = i & 15;
                *reinterpret_cast<uint4*>(s.Kt + j * TS + c8 * 8) = tk[u];
                *reinterpret_cast<uint4*>(s.Ut + j * TS + c8 * 8) = tu[u];
            }
        }
    }
    sync();
    if (KDA && tid < 128) {
        // key scale w_j D_j[c] with D_{L-1} = 1, D_j = D_{j+1} e_{j+1}
        float dcur = 1.f;
        const uint16_t* gb = Gbuf + sh * L * KD + tid;
        for (int j = L - 1; j >= 0; --j) {
            s.tab[j * 128 + tid] = s.w[j] * dcur;
            dcur *= f16_to_f(gb[j * KD]);
        }
    }
    if (KDA) sync();

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
        // add the dequantised checkpoint and store B[v][c] as f16; accumulator (e, nt): row m0 + r + 8 (e >> 1), col 8 nt + q2 + (e & 1)
        const float pq = KDA ? (1.0f / QMAX) : (p / QMAX);
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int mm = m0 + r + 8 * hrow, nn = 8 * nt + q2;
                const uint32_t cw = (cpre[nt] >> (16 * hrow)) & 0xffffu;
                const float f0 = float(int(int8_t(cw & 0xff))), f1 = float(int(int8_t(cw >> 8)));
                if (!KDA) {                                 // (v, c) = (mm, nn), (mm, nn + 1): two adjacent codes
                    const float svr = s.sv[mm] * pq;
                    const float o0 = (f0 * svr) * s.sk[nn] + acc[nt][2 * hrow];
                    const float o1 = (f1 * svr) * s.sk[nn + 1] + acc[nt][2 * hrow + 1];
                    *reinterpret_cast<uint32_t*>(s.Bh + mm * TS + nn) = pack_h2(o0, o1);
                } else {                                    // (c, v) = (mm, nn), (mm, nn + 1): codes of rows nn, nn + 1
                    const float skc = s.sk[mm];
                    s.Bh[nn * TS + mm] = f_to_f16((f0 * (s.sv[nn] * pq)) * skc + acc[nt][2 * hrow]);
                    s.Bh[(nn + 1) * TS + mm] = f_to_f16((f1 * (s.sv[nn + 1] * pq)) * skc + acc[nt][2 * hrow + 1]);
                }
            }
        }
    }
    sync();                                        // the window tiles are dead: the region may be reused
    // ---- stage C: subspace iteration on T = B + p Q_old U_old^T ----
    const int m0w = warp * 16;
    float dd[4] = {0.f, 0.f, 0.f, 0.f};
    auto store_p = [&] {                                    // P (rounded to f16) as rows [r][c]
        if (2 * tig < R) {
            s.Ph[(2 * tig) * HS + m0w + gid] = f_to_f16(dd[0]);
            s.Ph[(2 * tig + 1) * HS + m0w + gid] = f_to_f16(dd[1]);
            s.Ph[(2 * tig) * HS + m0w + gid + 8] = f_to_f16(dd[2]);
            s.Ph[(2 * tig + 1) * HS + m0w + gid + 8] = f_to_f16(dd[3]);
        }
    };
    tall_product<R, true>(s.Bh, s.Q0h, s.Qoh, s.UoT, p, warp, lane, dd);        // P = T^T Q0
    store_p();
    sync();
    if (iters == 0) {                                       // no round: the stored Q is the start itself
        for (int i = tid; i < R * HS; i += NT_LA) s.Qh[i] = s.Q0h[i];
        sync();
    }
    for (int it = 0; it < iters; ++it) {
        tall_product<R, false>(s.Bh, s.Ph, s.Uoh, s.QoT, p, warp, lane, dd);    // Q = T P
        if (2 * tig < R) {
            *reinterpret_cast<float2*>(s.Qn + (m0w + gid) * R + 2 * tig) = make_float2(dd[0], dd[1]);
            *reinterpret_cast<float2*>(s.Qn + (m0w + gid + 8) * R + 2 * tig) = make_float2(dd[2], dd[3]);
        }
        sync();
        cholqr2_f16<R>(s.Qn, tid, sync);
        for (int i = tid; i < 128 * R; i += NT_LA) s.Qh[(i % R) * HS + i / R] = f_to_f16(s.Qn[i]);
        sync();
        tall_product<R, true>(s.Bh, s.Qh, s.Qoh, s.UoT, p, warp, lane, dd);     // P = T^T Q
        store_p();
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
    } else {
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

    // ---- stage E: residual E = B + p Q_old U_old^T - Q U^T on the tensor cores, fp32 in registers: warp w owns rows
    //      16 w .. 16 w + 15, lane (gid, tig) holds rows gid, gid + 8 at columns 8 nt + 2 tig, + 1 ----
    float e[16][4];
    {
        const uint16_t* b0p = s.Bh + (m0w + gid) * TS + 2 * tig;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
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
            for (int nt = 0; nt < 16; ++nt) {
                const uint16_t* bp = s.Bc + (8 * nt + gid) * KS + ks + 2 * tig;
                mma_h_16816(e[nt], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(bp), *reinterpret_cast<const uint32_t*>(bp + 8));
            }
        }
    }
    // column sums of |E|: 32 partial sums per lane (two rows each), folded over the eight row groups of the warp by
    // three exchange levels that halve the number of values a lane keeps
    {
        const bool h4 = (lane & 16) != 0, h3 = (lane & 8) != 0, h2 = (lane & 4) != 0;
        float c16[16], c8[8], c4[4];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float a = fabsf(e[i >> 1][i & 1]) + fabsf(e[i >> 1][2 + (i & 1)]);
            const float b = fabsf(e[8 + (i >> 1)][i & 1]) + fabsf(e[8 + (i >> 1)][2 + (i & 1)]);
            c16[i] = (h4 ? b : a) + __shfl_xor_sync(0xffffffffu, h4 ? a : b, 16);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) c8[i] = (h3 ? c16[8 + i] : c16[i]) + __shfl_xor_sync(0xffffffffu, h3 ? c16[i] : c16[8 + i], 8);
#pragma unroll
        for (int i = 0; i < 4; ++i) c4[i] = (h2 ? c8[4 + i] : c8[i]) + __shfl_xor_sync(0xffffffffu, h2 ? c8[i] : c8[4 + i], 4);
        const int nt0 = (h4 ? 8 : 0) + (h3 ? 4 : 0) + (h2 ? 2 : 0);
        *reinterpret_cast<float2*>(s.colpart + warp * 128 + 8 * nt0 + 2 * tig) = make_float2(c4[0], c4[1]);
        *reinterpret_cast<float2*>(s.colpart + warp * 128 + 8 * (nt0 + 1) + 2 * tig) = make_float2(c4[2], c4[3]);
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

    // ---- stage F: row scales and INT8 codes, staged in the warp's own rows of the (dead) state tile ----
    {
        float r0 = 0.f, r1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            const float2 rk = *reinterpret_cast<const float2*>(s.sk + 8 * nt + 2 * tig);
            e[nt][0] *= rk.x; e[nt][1] *= rk.y; e[nt][2] *= rk.x; e[nt][3] *= rk.y;
            r0 = fmaxf(r0, fmaxf(fabsf(e[nt][0]), fabsf(e[nt][1])));
            r1 = fmaxf(r1, fmaxf(fabsf(e[nt][2]), fabsf(e[nt][3])));
        }
        r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 1)); r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 1));
        r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 2)); r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 2));
        const float sv0 = fmaxf(r0, EPS), sv1 = fmaxf(r1, EPS);
        const float rm0 = QMAX * __frcp_rn(sv0), rm1 = QMAX * __frcp_rn(sv1);
        if (tig == 0) {
            float* svg = reinterpret_cast<float*>(base + CK_SV);
            svg[m0w + gid] = sv0;
            svg[m0w + gid + 8] = sv1;
        }
        char* cw = reinterpret_cast<char*>(s.Bh) + (m0w + gid) * (TS * 2) + 2 * tig;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            const uint32_t lo = __byte_perm(rne_code(e[nt][0], rm0), rne_code(e[nt][1], rm0), 0x0040);
            const uint32_t hi = __byte_perm(rne_code(e[nt][2], rm1), rne_code(e[nt][3], rm1), 0x0040);
            *reinterpret_cast<uint16_t*>(cw + 8 * nt) = uint16_t(lo);
            *reinterpret_cast<uint16_t*>(cw + 8 * (TS * 2) + 8 * nt) = uint16_t(hi);
        }
        __syncwarp();
        const int row = m0w + (lane >> 1), half = lane & 1;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(s.Bh) + row * (TS * 2) + half * 64);
        uint4* dst = reinterpret_cast<uint4*>(base + CK_CODES + row * KD + half * 64);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = src[i];
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
    sync();
}

template <int R, bool KDA>
__global__ void __launch_bounds__(NT_LA, 2)
flush_kernel(lq_dims d, char* ssm, const uint16_t* Kbuf, const uint16_t* Ubuf, float* Wbuf, float* Pbuf, uint16_t* Gbuf,
             int32_t* hcnt, const float* __restrict__ Q0, const int32_t* __restrict__ idx, int N, int iters, int maxd) {
    extern __shared__ __align__(16) float smem[];
    const FlushSmem s = flush_carve<R>(reinterpret_cast<char*>(smem), d.L, KDA);
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
        int base = 0;
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
            if (f) s.dlist[base + __popc(m & lt)] = q;
            base += __popc(m);
        }
        if (lane == 0) s.wcnt[0] = base;
    }
    __syncthreads();
    const int mine = min(s.wcnt[0], maxd);
    if (mine == 0) return;

    flush_init<R>(s, Q0, tid);
    FlushArgs A;
    A.d = d; A.ssm = ssm; A.Kbuf = Kbuf; A.Ubuf = Ubuf; A.Wbuf = Wbuf; A.Pbuf = Pbuf; A.Gbuf = Gbuf; A.hcnt = hcnt; A.Q0 = Q0;
    A.iters = iters;
    for (int k = 0; k < mine; ++k) flush_head<R, KDA>(s, A, s.dlist[k], tid, [] { __syncthreads(); });
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
