// Standalone quantize, in-place dequantize and low-rank factorisation kernels (sm_100a).
//
// Quantize and low-rank: one CTA of 256 threads per (row, value head), the head's 128 x 128 fp32 tile in shared memory for
// the whole kernel.  Dequantize: persistent CTAs that walk the heads, each head's checkpoint staged in shared memory.
// Either way the in-place rewrite of a slot (fp32 state <-> packed 8-bit checkpoint) never reads what it has already
// overwritten.
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
            // rint() by adding 1.5 * 2^23: the sum's low mantissa byte is the code in two's complement.  |y| <= 127 (1 + 3e-7) by
            // construction of Sv, so the reference's clamp to [-127, 127] never acts and is not evaluated.
            uint32_t b[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float y = a[4 * i + k] * rv127;
                float t = y + 12582912.0f;
                const float c = t - 12582912.0f;
                if (fabsf(fabsf(y - c) - 0.5f) < 1e-3f)                        // on a rounding boundary: the exact expression decides
                    t = e[4 * i + k] / (sk[i * 32 + l8 * 4 + k] * svv) * QMAX + 12582912.0f;
                b[k] = __float_as_uint(t);
            }
            codes[row * 32 + i * 8 + l8] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
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

// four 8 x 8 b16 tiles, transposed: lane l supplies the address of row l % 8 of tile l / 8 and receives, of each tile, the
// elements (2 (l % 4), l / 4) and (2 (l % 4) + 1, l / 4)
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

// ------------------------------------------------------------------------------------------------------------------
// dequantize in place
// ------------------------------------------------------------------------------------------------------------------
// S[v][c] = (q8 / 127 Sk[c] Sv[v] + sum_r Q_r[v] U_r[c]) p pc[c] + sum_{j<h} (w_j u_j[v]) (k_j[c] D_j[c])   (leapquant/kernels.py:2105-2117;
// KDA: leapquant/state.py:118-128).  The constants are folded into the vectors first: skq[c] = Sk[c] / 127 (* pc[c]),
// svp[v] = Sv[v] p, Qp_r[v] = Q_r[v] p, Uc_r[c] = U_r[c] (* pc[c]).  The rank-R term runs on the tensor cores: Qp and Uc are
// split into a bf16 head and a bf16 remainder and the three products head x head, remainder x head, head x remainder are laid
// side by side along K of one `mma.sync.m16n8k16` (R = 4: K = 12 of 16; R = 8: two instructions), which keeps 16 bits of each
// factor -- 1e-5 of the term -- and replaces 4 R multiply-adds per element by an eighth of an instruction.  What is left per
// element is one conversion, one multiply, one fused multiply-add and h multiply-adds for the live window entries.  The
// values differ from the reference's evaluation order by a few units in the last place of fp32.
// Warp w owns rows 16 w .. 16 w + 15; lane (gid, tig) owns rows 16 w + gid, + 8 and, in each group of 16 columns, the four
// columns 4 tig .. 4 tig + 3: the two n-tiles of a group are mapped onto the columns so that every lane ends up with four
// contiguous ones (n index g of the first tile is column 4 (g / 2) + g % 2, of the second the same + 2).
// The window rows stay bf16 in shared memory (KDA keys: decayed, fp32).
// The kernel is persistent: two CTAs per SM, each taking the heads blockIdx.x, + gridDim.x, ...  A ninth warp runs ahead of
// the eight that compute: it looks up the slot, the window count and the scale of the heads to come (thirty-two at a time,
// one per lane) and brings each head's checkpoint -- codes, scales, factors: one contiguous piece -- into one of two stages
// with a bulk asynchronous copy, so that the three dependent trips to memory of a head (index -> counters -> checkpoint) are
// spent while the heads before it are evaluated and stored.  The output overwrites the checkpoint it was computed from,
// which is in shared memory by then; different heads never share bytes.
constexpr int DQ_THREADS = NT_LA + 32;
// A stage: the checkpoint, the KDA decay row, and -- for a head with at most DQ_ROWS live window entries, the case right
// after a prefill -- its window weights and its live rows of keys, values and (KDA) per-step decays.
constexpr int DQ_ROWS = 8;
__host__ __device__ constexpr int dq_off_w(int R) { return ck_bytes(R) + 512; }
__host__ __device__ constexpr int dq_off_rows(int R) { return dq_off_w(R) + 256; }
__host__ __device__ constexpr int dq_stage_bytes(int R) { return (dq_off_rows(R) + 3 * DQ_ROWS * 256 + 127) & ~127; }
struct DqInfo { int slot, h; float p; int valid; };
template <int R>
__global__ void __launch_bounds__(DQ_THREADS, 2)
dequant_kernel(lq_dims d, char* __restrict__ ssm, const uint16_t* __restrict__ Kbuf, const uint16_t* __restrict__ Ubuf,
               float* __restrict__ Wbuf, float* __restrict__ Pbuf, const uint16_t* __restrict__ Gbuf,
               int32_t* __restrict__ hcnt, const int32_t* __restrict__ idx, int nheads, int kda) {
    constexpr int KT = (3 * R + 15) / 16 * 16;            // K of the rank-R product: three pieces of R, padded to the instruction
    constexpr int KS = KT + 8;                            // row stride of the operands in bf16 elements (16 bytes of padding)
    constexpr int STAGE = dq_stage_bytes(R);
    extern __shared__ __align__(128) char dq_smem[];
    float* skq = reinterpret_cast<float*>(dq_smem + 2 * STAGE);   // [128] Sk / 127 (KDA: times pc)
    float* svp = skq + 128;                               // [128] Sv p
    uint16_t* Aop = reinterpret_cast<uint16_t*>(svp + 128);   // [128 rows v][KS]: Qp head | Qp remainder | Qp head | 0
    uint16_t* Bop = Aop + 128 * KS;                       // [128 cols c][KS]: Uc head | Uc head | Uc remainder | 0
    float* ws = reinterpret_cast<float*>(Bop + 128 * KS); // [64] window weights
    uint64_t* full = reinterpret_cast<uint64_t*>(ws + 64);    // [2] stage filled; [2] stage read to the end
    uint64_t* empty = full + 2;
    DqInfo* info = reinterpret_cast<DqInfo*>(empty + 2);  // [2]
    volatile int* okflag = reinterpret_cast<volatile int*>(info + 2);
    float* Kf = reinterpret_cast<float*>(info + 2) + 4;   // keys [Lp][WST] bf16 (columns permuted), values [Lp][WST] bf16; KDA: the keys are
                                                          // the head of k_j D_j, followed by its remainder [Lp][WST] and the raw keys [Lp][128]
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    constexpr int WST = 136;                              // GDN window rows in shared memory: 128 bf16 + 16 bytes, so that the
                                                          // eight rows of an ldmatrix tile fall into different bank groups
    const int Lp = (d.L + 15) & ~15;
    uint16_t* Ks = reinterpret_cast<uint16_t*>(Kf);       // keys: within every 16 columns c -> 8 (c % 4 / 2) + 2 (c / 4) + c % 2
    uint16_t* Us = Ks + Lp * WST;                         // values as stored
    uint16_t* Kl = Us + Lp * WST;                         // KDA: remainder of k_j D_j, same layout as Ks
    uint16_t* Kraw = Kl + Lp * WST;                       // KDA: keys as stored [Lp][128], read by the scan below

    if (tid == 0) {
        mbar_init(full + 0, 1); mbar_init(full + 1, 1);
        mbar_init(empty + 0, NT_LA / 32); mbar_init(empty + 1, NT_LA / 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    __syncthreads();
    const int first = blockIdx.x, stride = gridDim.x;

    if (warp == NT_LA / 32) {
        // ================= the warp that runs ahead =================
        int l_slot = 0, l_h = 0, l_valid = 0;
        float l_p = 1.f;
        for (int i = 0; first + i * stride < nheads; ++i) {
            if ((i & 31) == 0) {                          // the scalars of the next 32 heads of this CTA, one head per lane
                const int pg = first + (i + lane) * stride;
                l_slot = 0; l_h = 0; l_valid = 0; l_p = 1.f;
                if (pg < nheads) {
                    const int hvv = pg % d.HV;
                    l_slot = idx[pg / d.HV];
                    l_valid = l_slot > 0 && l_slot < d.NS;
                    if (l_valid) {
                        const int64_t sh = int64_t(l_slot) * d.HV + hvv;
                        l_h = min(max(hcnt[sh], 0), d.L);
                        l_p = kda ? 1.f : Pbuf[sh];
                    }
                }
            }
            const int s = i & 1;
            if (i >= 2 && !warp_wait_bounded(empty + s, uint32_t((i >> 1) - 1) & 1u, lane)) {
                if (lane == 0) atomicOr(&g_status, ST_PRODUCER_TIMEOUT);
                return;
            }
            const int src = i & 31;
            const int slot = __shfl_sync(0xffffffffu, l_slot, src), h = __shfl_sync(0xffffffffu, l_h, src);
            const int valid = __shfl_sync(0xffffffffu, l_valid, src);
            const float pp = __shfl_sync(0xffffffffu, l_p, src);
            if (lane == 0) {
                const int pg = first + i * stride, hv = pg % d.HV;
                info[s].slot = slot; info[s].h = h; info[s].p = pp; info[s].valid = valid;
                if (valid) {
                    fence_async_smem();                   // the stage's last readers used ordinary loads
                    const int64_t sh = int64_t(slot) * d.HV + hv;
                    const bool rows_in = h > 0 && h <= DQ_ROWS && d.L <= 64 && (d.L & 3) == 0;
                    const uint32_t rb = rows_in ? uint32_t(h) * 256u : 0u;
                    mbar_arrive_expect_tx(full + s, uint32_t(ck_bytes(R)) + (kda ? 512u : 0u) + (rows_in ? uint32_t(d.L) * 4u : 0u) + (kda ? 3u : 2u) * rb);
                    char* stg = dq_smem + s * STAGE;
                    bulk_g2s(stg, head_base(ssm, d.SS, slot, hv), uint32_t(ck_bytes(R)), full + s);
                    if (kda) bulk_g2s(stg + ck_bytes(R), Pbuf + sh * KD, 512u, full + s);
                    if (rows_in) {
                        bulk_g2s(stg + dq_off_w(R), Wbuf + sh * d.L, uint32_t(d.L) * 4u, full + s);
                        bulk_g2s(stg + dq_off_rows(R), Kbuf + sh * d.L * KD, rb, full + s);
                        bulk_g2s(stg + dq_off_rows(R) + DQ_ROWS * 256, Ubuf + sh * d.L * VD, rb, full + s);
                        if (kda) bulk_g2s(stg + dq_off_rows(R) + 2 * DQ_ROWS * 256, Gbuf + sh * d.L * KD, rb, full + s);
                    }
                } else {
                    mbar_arrive(full + s);                // padding row or null slot: nothing to fetch
                }
            }
            __syncwarp();
        }
        return;
    }

    // ================= the eight warps that evaluate and store =================
    for (int i = 0; first + i * stride < nheads; ++i) {
    const int s = i & 1;
    if (warp == 0) {
        const bool got = warp_wait_bounded(full + s, uint32_t(i >> 1) & 1u, lane);
        if (lane == 0) *okflag = got ? 1 : 0;
    }
    named_bar(1, NT_LA);                                  // (also: every warp is done with the previous head's operands and window rows)
    if (*okflag == 0) {
        if (tid == 0) atomicOr(&g_status, ST_CONSUMER_TIMEOUT);
        return;
    }
    const DqInfo hi = info[s];
    if (!hi.valid) {
        if (lane == 0) mbar_arrive(empty + s);
        continue;
    }
    const int pg = first + i * stride;
    const int hv = pg % d.HV, slot = hi.slot, h = hi.h;
    const float p = hi.p;
    char* base = head_base(ssm, d.SS, slot, hv);
    const char* stg = dq_smem + s * STAGE;
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(stg + CK_CODES);      // [128][32] code words
    const int64_t sh = int64_t(slot) * d.HV + hv;

    if (tid < 128) {
        const float pc = kda ? expf(reinterpret_cast<const float*>(stg + ck_bytes(R))[tid]) : 1.f;
        skq[tid] = reinterpret_cast<const float*>(stg + CK_SK)[tid] / QMAX * pc;
        svp[tid] = reinterpret_cast<const float*>(stg + CK_SV)[tid] * p;
        const uint16_t* uq = reinterpret_cast<const uint16_t*>(stg + CK_UQ);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float u = f16_to_f(uq[r * (KD + VD) + tid]) * pc, q = f16_to_f(uq[r * (KD + VD) + KD + tid]) * p;
            const uint16_t uh = f_to_bf16(u), qh = f_to_bf16(q);
            const uint16_t ul = f_to_bf16(u - bf16_to_f(uh)), ql = f_to_bf16(q - bf16_to_f(qh));
            Aop[tid * KS + r] = qh; Aop[tid * KS + R + r] = ql; Aop[tid * KS + 2 * R + r] = qh;
            Bop[tid * KS + r] = uh; Bop[tid * KS + R + r] = uh; Bop[tid * KS + 2 * R + r] = ul;
        }
#pragma unroll
        for (int r = 3 * R; r < KT; ++r) { Aop[tid * KS + r] = 0; Bop[tid * KS + r] = 0; }
    }
    // a short window came with the stage; a longer one is read from global memory here, four 16-byte pieces per thread in
    // flight at a time
    const bool rows_in = h > 0 && h <= DQ_ROWS && d.L <= 64 && (d.L & 3) == 0;
    if (tid < 64) {                                           // (all 64: the tensor-core window term reads whole steps of 16)
        float wv = 0.f;
        if (tid < h) wv = rows_in ? reinterpret_cast<const float*>(stg + dq_off_w(R))[tid] : Wbuf[sh * d.L + tid];
        ws[tid] = wv;
    }
    {
        const int hp = (h + 15) & ~15;                       // whole k-steps of 16 rows, the rows past h zero
        auto place = [&](int i2, const uint4& uv, const uint4& kv) {
            const int j = i2 >> 4, c8 = i2 & 15;              // row, 16-byte chunk (8 columns) of the row
            *reinterpret_cast<uint4*>(Us + j * WST + 8 * c8) = uv;
            if (kda) {
                reinterpret_cast<uint4*>(Kraw)[i2] = kv;
            } else {
                // the chunk holds columns 4 t .. 4 t + 7 of a group of 16 (t = 0 or 2): pairs (4t, 4t+1), (4t+4, 4t+5) go to the
                // first n-tile of the group at 2 t, 2 t + 2, pairs (4t+2, 4t+3), (4t+6, 4t+7) to the second at 8 + 2 t, 8 + 2 t + 2
                uint16_t* kd = Ks + j * WST + 16 * (c8 >> 1) + 4 * (c8 & 1);
                *reinterpret_cast<uint2*>(kd) = make_uint2(kv.x, kv.z);
                *reinterpret_cast<uint2*>(kd + 8) = make_uint2(kv.y, kv.w);
            }
        };
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        if (rows_in) {
            const uint4* kb = reinterpret_cast<const uint4*>(stg + dq_off_rows(R));
            const uint4* ub = reinterpret_cast<const uint4*>(stg + dq_off_rows(R) + DQ_ROWS * 256);
            for (int i2 = tid; i2 < hp * 16; i2 += NT_LA) {
                const bool live = (i2 >> 4) < h;
                place(i2, live ? ub[i2] : z, live ? kb[i2] : z);
            }
        } else if (h > 0) {
            const uint4* kb = reinterpret_cast<const uint4*>(Kbuf + sh * d.L * KD);
            const uint4* ub = reinterpret_cast<const uint4*>(Ubuf + sh * d.L * VD);
            for (int i0 = tid; i0 < hp * 16; i0 += 4 * NT_LA) {
                uint4 uv[4], kv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i2 = i0 + u * NT_LA;
                    const bool live = (i2 >> 4) < h;
                    uv[u] = live ? ldg_stream(ub + i2) : z;
                    kv[u] = live ? ldg_stream(kb + i2) : z;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i0 + u * NT_LA < hp * 16) place(i0 + u * NT_LA, uv[u], kv[u]);
            }
        }
    }
    named_bar(1, NT_LA);
    if (kda && h > 0) {
        if (tid < 128) {                       // D_j = prod_{j < i < h} e_i, backward running product per column; k_j D_j as a
            float dcur = 1.f;                  // bf16 head and remainder at the column's place in the permuted rows
            const int hp = (h + 15) & ~15;
            const int cp = (tid & ~15) + 8 * ((tid & 3) >> 1) + 2 * ((tid & 15) >> 2) + (tid & 1);
            for (int j = hp - 1; j >= h; --j) { Ks[j * WST + cp] = 0; Kl[j * WST + cp] = 0; }
            auto scan = [&](int j, float e) {
                const float kd = bf16_to_f(Kraw[j * 128 + tid]) * dcur;
                const uint16_t kh = f_to_bf16(kd);
                Ks[j * WST + cp] = kh;
                Kl[j * WST + cp] = f_to_bf16(kd - bf16_to_f(kh));
                dcur *= e;
            };
            if (rows_in) {
                const uint16_t* gs = reinterpret_cast<const uint16_t*>(stg + dq_off_rows(R) + 2 * DQ_ROWS * 256);
                for (int j = h - 1; j >= 0; --j) scan(j, f16_to_f(gs[j * KD + tid]));
            } else {                           // the per-step decays from global memory, eight in flight
                const uint16_t* gg = Gbuf + sh * d.L * KD + tid;
                for (int j0 = h - 1; j0 >= 0; j0 -= 8) {
                    uint16_t e[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) e[u] = j0 - u >= 0 ? __ldg(gg + (j0 - u) * KD) : uint16_t(0);
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (j0 - u >= 0) scan(j0 - u, f16_to_f(e[u]));
                }
            }
        }
        named_bar(1, NT_LA);
    }

    const int r0 = 16 * warp + gid, r1 = r0 + 8;
    // rank-R term: A fragments of this warp's 16 rows once per K step, B fragments per n-tile
    uint32_t af[KT / 16][4];
#pragma unroll
    for (int ks = 0; ks < KT / 16; ++ks) {
        af[ks][0] = *reinterpret_cast<const uint32_t*>(Aop + r0 * KS + 16 * ks + 2 * tig);
        af[ks][1] = *reinterpret_cast<const uint32_t*>(Aop + r1 * KS + 16 * ks + 2 * tig);
        af[ks][2] = *reinterpret_cast<const uint32_t*>(Aop + r0 * KS + 16 * ks + 8 + 2 * tig);
        af[ks][3] = *reinterpret_cast<const uint32_t*>(Aop + r1 * KS + 16 * ks + 8 + 2 * tig);
    }
    const int cn = 4 * (gid >> 1) + (gid & 1);              // column (within a group of 16) that n index gid of the first n-tile stands for
    const float sv0 = svp[r0], sv1 = svp[r1];
    float* out = reinterpret_cast<float*>(base);            // (everything of the slot that is read was copied to shared memory above)
    // two groups of 16 columns at a time, start to finish: sixteen accumulators per thread instead of sixty-four, and the
    // values of a window entry are fetched four times per entry, not eight
#pragma unroll 1
    for (int qp = 0; qp < 4; ++qp) {
        float a0[2][4], a1[2][4];                           // [group][column]: rows r0 and r1, columns 16 q + 4 tig + k
#pragma unroll
        for (int g2 = 0; g2 < 2; ++g2) {
            const int q = 2 * qp + g2;
            float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < KT / 16; ++ks) {
                const uint16_t* b0p = Bop + (16 * q + cn) * KS + 16 * ks + 2 * tig;
                const uint16_t* b1p = b0p + 2 * KS;
                mma_bf16_16816(c0, af[ks][0], af[ks][1], af[ks][2], af[ks][3], *reinterpret_cast<const uint32_t*>(b0p),
                               *reinterpret_cast<const uint32_t*>(b0p + 8));
                mma_bf16_16816(c1, af[ks][0], af[ks][1], af[ks][2], af[ks][3], *reinterpret_cast<const uint32_t*>(b1p),
                               *reinterpret_cast<const uint32_t*>(b1p + 8));
            }
            // codes: one word = this lane's four columns of a row
            // (packed pairs: the same three roundings per element -- convert, times the column scale, fused with the row
            //  scale into the rank-R term -- in half the instructions)
            const float4 sk4 = *reinterpret_cast<const float4*>(skq + 16 * q + 4 * tig);
            const float2 sk01 = make_float2(sk4.x, sk4.y), sk23 = make_float2(sk4.z, sk4.w);
            const float2 s0 = make_float2(sv0, sv0), s1 = make_float2(sv1, sv1);
            float2 f01, f23, g01, g23;
            s8x4_to_f2x2(cw[r0 * 32 + 4 * q + tig], f01, f23);
            s8x4_to_f2x2(cw[r1 * 32 + 4 * q + tig], g01, g23);
            const float2 x01 = __ffma2_rn(__fmul2_rn(f01, sk01), s0, make_float2(c0[0], c0[1]));
            const float2 x23 = __ffma2_rn(__fmul2_rn(f23, sk23), s0, make_float2(c1[0], c1[1]));
            const float2 y01 = __ffma2_rn(__fmul2_rn(g01, sk01), s1, make_float2(c0[2], c0[3]));
            const float2 y23 = __ffma2_rn(__fmul2_rn(g23, sk23), s1, make_float2(c1[2], c1[3]));
            a0[g2][0] = x01.x; a0[g2][1] = x01.y; a0[g2][2] = x23.x; a0[g2][3] = x23.y;
            a1[g2][0] = y01.x; a1[g2][1] = y01.y; a1[g2][2] = y23.x; a1[g2][3] = y23.y;
        }
        // live window entries: sum_j (w_j u_j[v]) (k_j[c] D_j[c]) on the tensor cores, 16 entries per step.  A = the values, read
        // transposed from their rows ([j][v] -> rows v, K index j), scaled by w_j in registers and split into a bf16 head and
        // remainder; B = the keys, read transposed from their column-permuted rows (GDN: exact in bf16; KDA: head and remainder
        // of the decayed keys, three products).
        for (int j0 = 0; j0 < h; j0 += 16) {
            uint32_t au[4];
            ldmatrix_x4_trans(au, Us + (j0 + (lane & 7) + ((lane >> 4) << 3)) * WST + 16 * warp + (((lane >> 3) & 1) << 3));
            const float2 w01 = *reinterpret_cast<const float2*>(ws + j0 + 2 * tig), w89 = *reinterpret_cast<const float2*>(ws + j0 + 8 + 2 * tig);
            uint32_t ah[4], al[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {                    // au[0], au[1]: entries j0 + 2 tig, + 1; au[2], au[3]: j0 + 8 + 2 tig, + 1
                const float2 wv = i < 2 ? w01 : w89;
                const float2 uv = bf16x2_to_f2(au[i]);
                const float x0 = uv.x * wv.x, x1 = uv.y * wv.y;
                ah[i] = f2_to_bf16x2(x0, x1);
                const float2 hv2 = bf16x2_to_f2(ah[i]);
                al[i] = f2_to_bf16x2(x0 - hv2.x, x1 - hv2.y);
            }
#pragma unroll
            for (int g2 = 0; g2 < 2; ++g2) {
                const int koff = (j0 + (lane & 7) + (((lane >> 3) & 1) << 3)) * WST + 16 * (2 * qp + g2) + ((lane >> 4) << 3);
                uint32_t bk[4];                              // keys of the group's two n-tiles: (tile 0: rows j0.., j0 + 8..), (tile 1: ..)
                ldmatrix_x4_trans(bk, Ks + koff);
                float c0[4] = {a0[g2][0], a0[g2][1], a1[g2][0], a1[g2][1]}, c1[4] = {a0[g2][2], a0[g2][3], a1[g2][2], a1[g2][3]};
                mma_bf16_16816(c0, ah[0], ah[1], ah[2], ah[3], bk[0], bk[1]);
                mma_bf16_16816(c0, al[0], al[1], al[2], al[3], bk[0], bk[1]);
                mma_bf16_16816(c1, ah[0], ah[1], ah[2], ah[3], bk[2], bk[3]);
                mma_bf16_16816(c1, al[0], al[1], al[2], al[3], bk[2], bk[3]);
                if (kda) {
                    uint32_t bl[4];
                    ldmatrix_x4_trans(bl, Kl + koff);
                    mma_bf16_16816(c0, ah[0], ah[1], ah[2], ah[3], bl[0], bl[1]);
                    mma_bf16_16816(c1, ah[0], ah[1], ah[2], ah[3], bl[2], bl[3]);
                }
                a0[g2][0] = c0[0]; a0[g2][1] = c0[1]; a1[g2][0] = c0[2]; a1[g2][1] = c0[3];
                a0[g2][2] = c1[0]; a0[g2][3] = c1[1]; a1[g2][2] = c1[2]; a1[g2][3] = c1[3];
            }
        }
#pragma unroll
        for (int g2 = 0; g2 < 2; ++g2) {
            const int q = 2 * qp + g2;
            *reinterpret_cast<float4*>(out + r0 * KD + 16 * q + 4 * tig) = make_float4(a0[g2][0], a0[g2][1], a0[g2][2], a0[g2][3]);
            *reinterpret_cast<float4*>(out + r1 * KD + 16 * q + 4 * tig) = make_float4(a1[g2][0], a1[g2][1], a1[g2][2], a1[g2][3]);
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + s);                  // this warp has read the last of the stage
    if (!kda) {
        for (int j = tid; j < d.L; j += NT_LA) Wbuf[sh * d.L + j] = 0.f;
        if (tid == 0) {
            Pbuf[sh] = 1.f;
            hcnt[sh] = 0;
        }
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
    // two checkpoint stages, folded scales, factors, weights, barriers, window rows (bf16; KDA: decayed keys as head and remainder)
    const int kt = (3 * d->R + 15) / 16 * 16 + 8;               // operand row of the rank-R product, bf16 elements
    const size_t win = size_t((d->L + 15) & ~15) * (kda ? 3 * 136 * 2 + 128 * 2 : 2 * 136 * 2);
    const size_t smem = size_t(2) * dq_stage_bytes(d->R) + sizeof(float) * (2 * 128 + 64) + size_t(2) * 128 * kt * 2 + 4 * sizeof(uint64_t) +
                        2 * sizeof(DqInfo) + 16 + win;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nheads = N * d->HV;
    const int cap = 2 * device_sm_count();
    dim3 grid(unsigned(nheads < cap ? nheads : cap)), block(DQ_THREADS);
    if (d->R == 4) {
        if ((rc = ensure_smem((const void*)dequant_kernel<4>, smem))) return rc;
        dequant_kernel<4><<<grid, block, smem, st>>>(*d, (char*)ssm, (const uint16_t*)Kbuf, (const uint16_t*)Ubuf, Wbuf, Pbuf,
                                                     (const uint16_t*)Gbuf, hcnt, idx, nheads, kda);
    } else {
        if ((rc = ensure_smem((const void*)dequant_kernel<8>, smem))) return rc;
        dequant_kernel<8><<<grid, block, smem, st>>>(*d, (char*)ssm, (const uint16_t*)Kbuf, (const uint16_t*)Ubuf, Wbuf, Pbuf,
                                                     (const uint16_t*)Gbuf, hcnt, idx, nheads, kda);
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
