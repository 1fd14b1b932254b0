// GDN / KDA decode-step kernels (sm_100a).
//
// One "program" is one (row n, value head hv): it streams the head's INT8 checkpoint (codes, scales, factors) and the
// h live entries of its window buffer, and appends the new token.  A program is executed out of a shared-memory stage
// in two parts: a one-warp prologue (l2 norms, operand vectors, gates, window-weight decay, key append) and a body run
// by a group of GT threads (window dots, checkpoint matvec, contribution, output).  Two drivers share them:
//   * step_direct_kernel    : one CTA per program, cooperative 16-byte global loads into the stage;
//   * step_pipelined_kernel : persistent CTAs; a producer warp fills a ring of stages with bulk asynchronous copies
//                             (cp.async.bulk + mbarrier), a prologue warp prepares each stage, consumer groups compute.
//
// Thread mapping of the matvec: eight lanes share a row of the 128 x 128 INT8 tile; lane l8 = lane & 7 owns the
// 16 columns 16 l8 .. 16 l8 + 15, so a warp-wide 16-byte load covers four whole 128-byte rows and the operand
// vectors k_hat * Sk / 127 and q_hat * Sk / 127 for those columns stay in registers for the whole tile.
#include <string.h>

#include "lq_common.cuh"

#ifndef LQ_GW
#define LQ_GW 4       // warps per consumer group
#endif
#ifndef LQ_NG
#define LQ_NG 3       // consumer groups per CTA
#endif

namespace lq {

constexpr int GW = LQ_GW;                 // warps of one consumer group (a group executes one program at a time)
constexpr int GT = 32 * GW;               // its threads
static_assert(GW == 4 || GW == 8, "the reductions below are written for 4 or 8 warps per group");

// ---- stage layout (bytes) of a program with `rows` window rows; the checkpoint part mirrors the packed slot so that it
//      is ONE contiguous copy.  The pipelined driver sizes every stage for the program's live rows (rows = h), so that a
//      ring of 220 KB holds ~6 average programs instead of 4 worst-case ones. ----
struct StageLayout {
    int kb, ub, w, q, k, v, gb, pb, a, dtb, nrm, bop, bdk, sc, bytes;
};
__host__ __device__ inline StageLayout stage_layout(int rows, int L, int R, bool kda, bool qkv = true) {
    StageLayout s;
    int o = ck_bytes(R);
    s.kb = o; o += rows * 256;
    s.ub = o; o += rows * 256;
    s.w = o; o += L * 4;
    s.q = s.k = s.v = 0;
    if (qkv) {                               // the pipelined driver reads q, k, v straight from global memory into registers
        s.q = o; o += 256;
        s.k = o; o += 256;
        s.v = o; o += 256;
    }
    s.gb = s.pb = s.a = s.dtb = 0;
    if (kda) {
        s.gb = o; o += rows * 256;
        s.pb = o; o += 512;
        s.a = o; o += 256;
        s.dtb = o; o += 512;
    }
    s.nrm = o; o += (kda ? 4 : 2) * 512;    // prologue output: k_hat, q_hat, then KDA: pc, en  (f32[128] each)
    s.bop = o; o += 4 * 256;                // prologue output: matvec operands as f16[128] x {k hi, k lo, q hi, q lo}
    s.bdk = o; o += 4 * 256;                // prologue output: k_hat, q_hat as bf16[128] x {k head, k remainder, q head, q remainder}
    s.sc = o; o += 64;                      // ProgScalars (producer) + k_hat . q_hat and the operand unscale (prologue)
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
    // fused causal conv1d update (CONV kernels only): q | k | v are computed from the raw projections
    const uint16_t* cx;          // bf16 [N, cx_stride] raw projections, MIX = 2 H K + HV V channels per row
    uint16_t* cstate;            // bf16 conv state, element (slot, channel, tap) at slot * cs_slot + channel * cs_dim + tap * cs_tap
    const uint16_t* cw;          // bf16 [MIX][4] depthwise taps
    const uint16_t* cb;          // bf16 [MIX] bias or null
    int64_t cs_slot, cs_dim, cs_tap;
    int64_t cx_stride;
};

// ------------------------------------------------------------------------------------------------------------------
// causal conv1d update of NC consecutive channels of one row: out = silu(bias + sum_t w[c][t] window[t]) with
// window = (state[0], state[1], state[2], x), new state = (state[1], state[2], x).  The arithmetic is the serving engine's
// Triton kernel's: every tap product is rounded to bf16, the sum runs in fp32 from the bias on, taps in order, and the
// activation is x / (1 + exp(-x)) in fp32, rounded to bf16 at the end.
// ------------------------------------------------------------------------------------------------------------------
constexpr int CONV_W = 4;
// The raw words of NC consecutive channels (two bf16 per word), as loaded: nothing is unpacked before conv_eval(), and the
// loads of the contiguous layout are volatile asm, so that they are issued where the caller puts them -- a whole program
// ahead of their use -- and not next to it.
template <int NC>
struct ConvRegs {
    uint32_t x[NC / 2], st[CONV_W - 1][NC / 2], w[NC * CONV_W / 2], b[NC / 2];
};
__device__ __forceinline__ uint32_t ld_early_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ void ld_early_words(const void* p, uint32_t (&out)[1]) { out[0] = ld_early_u32(p); }
__device__ __forceinline__ void ld_early_words(const void* p, uint32_t (&out)[2]) {
    asm volatile("ld.global.v2.u32 {%0, %1}, [%2];" : "=r"(out[0]), "=r"(out[1]) : "l"(p));
}
__device__ __forceinline__ void ld_early_words(const void* p, uint32_t (&out)[4]) {
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3]) : "l"(p));
}
__device__ __forceinline__ void ld_early_words(const void* p, uint32_t (&out)[8]) {
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3]) : "l"(p));
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4+16];" : "=r"(out[4]), "=r"(out[5]), "=r"(out[6]), "=r"(out[7]) : "l"(p));
}
__device__ __forceinline__ void st_words(void* p, const uint32_t (&in)[1]) { *reinterpret_cast<uint32_t*>(p) = in[0]; }
__device__ __forceinline__ void st_words(void* p, const uint32_t (&in)[2]) { *reinterpret_cast<uint2*>(p) = make_uint2(in[0], in[1]); }
__device__ __forceinline__ uint16_t half_of(const uint32_t* w, int e) { return uint16_t(w[e >> 1] >> (16 * (e & 1))); }
template <int NC>
__device__ __forceinline__ ConvRegs<NC> conv_load(const StepParams& P, int n, int slot, int c0) {
    static_assert(NC == 2 || NC == 4, "two or four channels per thread");
    ConvRegs<NC> r;
    ld_early_words(P.cx + int64_t(n) * P.cx_stride + c0, r.x);
    const uint16_t* sb = P.cstate + int64_t(slot) * P.cs_slot;
    if (P.cs_dim == 1) {                                     // (slot, tap, channel): the channels of a tap are contiguous
#pragma unroll
        for (int t = 0; t < CONV_W - 1; ++t) ld_early_words(sb + t * P.cs_tap + c0, r.st[t]);
    } else {                                                 // (slot, channel, tap): one element at a time
#pragma unroll
        for (int t = 0; t < CONV_W - 1; ++t)
#pragma unroll
            for (int e = 0; e < NC; e += 2)
                r.st[t][e >> 1] = uint32_t(sb[int64_t(c0 + e) * P.cs_dim + t * P.cs_tap]) |
                                  (uint32_t(sb[int64_t(c0 + e + 1) * P.cs_dim + t * P.cs_tap]) << 16);
    }
    ld_early_words(P.cw + int64_t(c0) * CONV_W, r.w);
    if (P.cb) ld_early_words(P.cb + c0, r.b);
    else {
#pragma unroll
        for (int e = 0; e < NC / 2; ++e) r.b[e] = 0u;
    }
    return r;
}
template <int NC>
__device__ __forceinline__ void conv_eval(const ConvRegs<NC>& r, uint16_t (&out)[NC]) {
#pragma unroll
    for (int e = 0; e < NC; ++e) {
        float acc = bf16_to_f(half_of(r.b, e));
#pragma unroll
        for (int t = 0; t < CONV_W; ++t) {
            const float xv = bf16_to_f(t < CONV_W - 1 ? half_of(r.st[t], e) : half_of(r.x, e));
            acc += round_bf16(xv * bf16_to_f(half_of(r.w, e * CONV_W + t)));
        }
        out[e] = f_to_bf16(__fdividef(acc, 1.0f + __expf(-acc)));       // (the result is rounded to bf16: eight bits)
    }
}
// new state of the NC channels, tap by tap: nw[t] = the words of tap t
template <int NC>
__device__ __forceinline__ void conv_store_words(const StepParams& P, int slot, int c0, const uint32_t (&nw)[CONV_W - 1][NC / 2]) {
    uint16_t* sb = P.cstate + int64_t(slot) * P.cs_slot;
    if (P.cs_dim == 1) {
#pragma unroll
        for (int t = 0; t < CONV_W - 1; ++t) st_words(sb + t * P.cs_tap + c0, nw[t]);
    } else {
#pragma unroll
        for (int e = 0; e < NC; ++e) {
            uint16_t* cp = sb + int64_t(c0 + e) * P.cs_dim;
#pragma unroll
            for (int t = 0; t < CONV_W - 1; ++t) cp[t * P.cs_tap] = half_of(nw[t], e);
        }
    }
}
// new state (state[1], state[2], x)
template <int NC>
__device__ __forceinline__ void conv_store_state(const StepParams& P, int slot, int c0, const ConvRegs<NC>& r) {
    uint32_t nw[CONV_W - 1][NC / 2];
#pragma unroll
    for (int e = 0; e < NC / 2; ++e) { nw[0][e] = r.st[1][e]; nw[1][e] = r.st[2][e]; nw[2][e] = r.x[e]; }
    conv_store_words<NC>(P, slot, c0, nw);
}

// per-program scalars, produced once and read by the whole group
struct ProgScalars {
    int slot, h, n, hv;
    float alpha, beta, pold, ea;
};

// per-group scratch in shared memory
struct GroupScratch {
    float2* wd;      // [64 + 8]  (w_j dk_j, w_j dq_j) for j < L, then (dU_r . k, dU_r . q) at 64 + r
    float2* mqy;     // [128]     (mq, yq) per row
};
constexpr int SCRATCH_BYTES = 72 * 8 + 128 * 8;

__device__ __forceinline__ GroupScratch carve_scratch(char* p) {
    GroupScratch g;
    g.wd = reinterpret_cast<float2*>(p);
    g.mqy = reinterpret_cast<float2*>(p + 72 * 8);
    return g;
}

// The scalars of a program come from two levels of dependent global loads (row -> slot -> counters and gates).  They are
// split so that a caller can keep both levels of several programs in flight: load_raw() only issues loads (no branch, no
// arithmetic on what it loaded; a null row reads slot 0, which exists and is never used), finish_scalars() does the math.
struct RawScalars {
    int slot, h, n, hv;
    float alog, pold, dtb;
    uint16_t a, b;
};
__device__ __forceinline__ RawScalars load_raw(const StepParams& P, int n, int hv, int slot, bool kda) {
    RawScalars r;
    r.n = n; r.hv = hv;
    r.slot = (slot > 0 && slot < P.d.NS) ? slot : 0;
    const int64_t sh = int64_t(r.slot) * P.d.HV + hv;
    r.h = P.hcnt[sh];
    r.alog = P.A_log[hv];
    r.b = P.b[int64_t(n) * P.d.HV + hv];
    r.a = 0; r.dtb = 0.f; r.pold = 1.f;
    if (!kda) {
        r.a = P.a[int64_t(n) * P.d.HV + hv];
        r.dtb = P.dt_bias[hv];
        r.pold = P.Pbuf[sh];
    }
    return r;
}
__device__ __forceinline__ ProgScalars finish_scalars(const RawScalars& r, bool kda) {
    ProgScalars s;
    s.n = r.n; s.hv = r.hv; s.slot = r.slot;
    s.h = 0; s.alpha = 1.f; s.beta = 0.f; s.pold = 1.f; s.ea = 1.f;
    if (r.slot > 0) {
        s.h = r.h;
        s.ea = expf(r.alog);
        s.beta = round_bf16(sigmoidf_(bf16_to_f(r.b)));
        if (!kda) {
            const float xg = bf16_to_f(r.a) + r.dtb;
            s.alpha = expf(-s.ea * softplus_thr(xg));
            s.pold = r.pold;
        }
    }
    return s;
}
__device__ __forceinline__ ProgScalars load_scalars(const StepParams& P, int n, int hv, bool kda) {
    return finish_scalars(load_raw(P, n, hv, P.idx[n], kda), kda);
}
__device__ __forceinline__ bool prog_live(const ProgScalars& s, int L) { return s.slot > 0 && s.h >= 0 && s.h < L; }

// Transposed reductions over the eight lanes of a row group.  Every lane holds one partial sum per tile pass; the lanes
// add them up so that lane l8 ends with the total of pass l8 (mod the number of passes).
template <int N>
__device__ __forceinline__ float pass_transpose_sum(const float (&x)[N], int l8) {
    if constexpr (N == 8) {                       // 7 shuffles instead of 24
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
    } else {                                      // four passes: transposed over lane bits 1 and 0, summed over bit 2
        static_assert(N == 4, "4 or 8 passes");
        float y[2];
        const bool b1 = l8 & 2;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float keep = b1 ? x[2 + k] : x[k];
            const float send = b1 ? x[k] : x[2 + k];
            y[k] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        const bool b0 = l8 & 1;
        const float keep = b0 ? y[1] : y[0];
        const float send = b0 ? y[0] : y[1];
        const float z = keep + __shfl_xor_sync(0xffffffffu, send, 1);
        return z + __shfl_xor_sync(0xffffffffu, z, 4);
    }
}

// The four f32[128] vectors the prologue leaves in the stage are read back by eight lanes at a time, lane l8 taking the
// 64 bytes of its 16 channels as four 16-byte chunks.  Chunk c (0..31) is stored at c with its two low bits XORed by
// bits 3..4 of c, which spreads the eight lanes of a quarter-warp over all eight 16-byte bank groups.
__device__ __forceinline__ int nrm_chunk(int c) { return (c & ~3) | ((c & 3) ^ ((c >> 3) & 3)); }

// Four signed bytes -> two f16 pairs, exactly: byte ^ 0x80 is the code + 128 as an unsigned byte u, the f16 with bits
// 0x6400 | u is 1024 + u, and subtracting 1152 leaves the code.  lo gets bytes 0, 1 and hi bytes 2, 3.
__device__ __forceinline__ void s8x4_to_h2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t u = w ^ 0x80808080u;
    const uint32_t p0 = __byte_perm(u, 0x64646464u, 0x4140), p1 = __byte_perm(u, 0x64646464u, 0x4342);
    const __half2 off = __floats2half2_rn(1152.f, 1152.f);
    const __half2 r0 = __hsub2(*reinterpret_cast<const __half2*>(&p0), off), r1 = __hsub2(*reinterpret_cast<const __half2*>(&p1), off);
    lo = *reinterpret_cast<const uint32_t*>(&r0);
    hi = *reinterpret_cast<const uint32_t*>(&r1);
}
// D += A B for one m16n8k16 tile, f16 operands, f32 accumulator (warp-wide)
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ------------------------------------------------------------------------------------------------------------------
// prologue: ONE warp, lane owns key channels 4 lane .. 4 lane + 3
// ------------------------------------------------------------------------------------------------------------------
// `signal()` is called after the last shared-memory write and BEFORE the global stores (see step_body's `release`).
template <bool KDA, typename Signal>
__device__ __forceinline__ void step_prologue(const StepParams& P, const ProgScalars& sc, char* st, const StageLayout& lay,
                                              int lane, Signal signal, bool qk_regs = false,
                                              uint2 q_in = make_uint2(0u, 0u), uint2 k_in = make_uint2(0u, 0u)) {
    const int L = P.d.L, h = sc.h;
    const int64_t sh = int64_t(sc.slot) * P.d.HV + sc.hv;
    const uint2 qw = qk_regs ? q_in : reinterpret_cast<const uint2*>(st + lay.q)[lane];      // this lane's four channels of q
    const uint2 kw = qk_regs ? k_in : reinterpret_cast<const uint2*>(st + lay.k)[lane];
    float q[4], k[4];
    q[0] = bf16lo(qw.x); q[1] = bf16hi(qw.x); q[2] = bf16lo(qw.y); q[3] = bf16hi(qw.y);
    k[0] = bf16lo(kw.x); k[1] = bf16hi(kw.x); k[2] = bf16lo(kw.y); k[3] = bf16hi(kw.y);
    // KDA per-channel gate: log-decay g, cumulative log gate gn, pc = exp(gn), step factor en = exp(g)
    float gn[4], en[4], pc[4] = {1.f, 1.f, 1.f, 1.f};
    if (KDA) {
        const uint2 aw = reinterpret_cast<const uint2*>(st + lay.a)[lane];
        const float4 db = reinterpret_cast<const float4*>(st + lay.dtb)[lane];
        const float4 pb = reinterpret_cast<const float4*>(st + lay.pb)[lane];
        const float xa[4] = {bf16lo(aw.x) + db.x, bf16hi(aw.x) + db.y, bf16lo(aw.y) + db.z, bf16hi(aw.y) + db.w};
        const float pbv[4] = {pb.x, pb.y, pb.z, pb.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float gl;
            if (P.glb != 0.f) gl = P.glb * (1.0f / (1.0f + __expf(-sc.ea * xa[i])));
            else gl = -sc.ea * (xa[i] <= SOFTPLUS_THRESHOLD ? __logf(1.0f + __expf(xa[i])) : xa[i]);
            gn[i] = pbv[i] + gl;
            en[i] = __expf(gl);
            pc[i] = __expf(gn[i]);
        }
    }
    // column weights of the checkpoint matvec: Sk / 127 (KDA: times pc)
    const float4 s4 = reinterpret_cast<const float4*>(st + CK_SK)[lane];
    float s[4] = {s4.x * (1.0f / QMAX), s4.y * (1.0f / QMAX), s4.z * (1.0f / QMAX), s4.w * (1.0f / QMAX)};
    if (KDA) {
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] *= pc[i];
    }
    // one butterfly for |q|^2, |k|^2, k.q and the largest |k s|, |q s| (their maxima give the f16 operand scale)
    float sq = 0.f, sk = 0.f, skq = 0.f, mk = 0.f, mq = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sq = fmaf(q[i], q[i], sq);
        sk = fmaf(k[i], k[i], sk);
        skq = fmaf(k[i], q[i], skq);
        mk = fmaxf(mk, fabsf(k[i] * s[i]));
        mq = fmaxf(mq, fabsf(q[i] * s[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float a0 = __shfl_xor_sync(0xffffffffu, sq, o), a1 = __shfl_xor_sync(0xffffffffu, sk, o);
        const float a2 = __shfl_xor_sync(0xffffffffu, skq, o), a3 = __shfl_xor_sync(0xffffffffu, mk, o);
        const float a4 = __shfl_xor_sync(0xffffffffu, mq, o);
        sq += a0; sk += a1; skq += a2; mk = fmaxf(mk, a3); mq = fmaxf(mq, a4);
    }
    const float inq = rsqrtf(sq + 1e-6f) * P.scale, ink = rsqrtf(sk + 1e-6f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        q[i] *= inq;
        k[i] *= ink;
    }
    // The matvec runs on the tensor cores in f16 with an f32 accumulator.  The operands k_hat s and q_hat s are scaled by a
    // power of two that puts the largest of them in [2^13, 2^14) and split into an f16 head and an f16 remainder, which keeps
    // 22 bits of every operand that matters at the size of the largest one.
    const float mx = fmaxf(mk * ink, mq * inq);
    uint32_t eb = __float_as_uint(mx) & 0x7F800000u;
    eb = eb < 0x0C800000u ? 0x0C800000u : eb;
    const uint32_t sbits = (267u << 23) - eb;
    const float oscale = __uint_as_float(sbits);
    {
        uint32_t hw[4][2];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            float x[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] = (n == 0 ? k[i] : q[i]) * s[i] * oscale;
            const __half2 h01 = __floats2half2_rn(x[0], x[1]), h23 = __floats2half2_rn(x[2], x[3]);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(x[0] - f01.x, x[1] - f01.y), l23 = __floats2half2_rn(x[2] - f23.x, x[3] - f23.y);
            hw[2 * n][0] = *reinterpret_cast<const uint32_t*>(&h01); hw[2 * n][1] = *reinterpret_cast<const uint32_t*>(&h23);
            hw[2 * n + 1][0] = *reinterpret_cast<const uint32_t*>(&l01); hw[2 * n + 1][1] = *reinterpret_cast<const uint32_t*>(&l23);
        }
#pragma unroll
        for (int n = 0; n < 4; ++n) reinterpret_cast<uint2*>(st + lay.bop + n * 256)[lane] = make_uint2(hw[n][0], hw[n][1]);
    }
    {   // k_hat, q_hat as bf16 head + remainder (16 mantissa bits): the B operand of the window dots on the tensor cores
        float kh[4], kl[4], qh[4], ql[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            kh[i] = round_bf16(k[i]); kl[i] = k[i] - kh[i];
            qh[i] = round_bf16(q[i]); ql[i] = q[i] - qh[i];
        }
        uint2* bd = reinterpret_cast<uint2*>(st + lay.bdk);
        bd[lane] = make_uint2(f2_to_bf16x2(kh[0], kh[1]), f2_to_bf16x2(kh[2], kh[3]));
        bd[32 + lane] = make_uint2(f2_to_bf16x2(kl[0], kl[1]), f2_to_bf16x2(kl[2], kl[3]));
        bd[64 + lane] = make_uint2(f2_to_bf16x2(qh[0], qh[1]), f2_to_bf16x2(qh[2], qh[3]));
        bd[96 + lane] = make_uint2(f2_to_bf16x2(ql[0], ql[1]), f2_to_bf16x2(ql[2], ql[3]));
    }
    float4* nrm = reinterpret_cast<float4*>(st + lay.nrm);
    const int sl = nrm_chunk(lane);                       // swizzled 16-byte chunk of this lane's four channels
    nrm[sl] = make_float4(k[0], k[1], k[2], k[3]);
    nrm[32 + sl] = make_float4(q[0], q[1], q[2], q[3]);
    if (lane == 0) {
        *reinterpret_cast<float*>(st + lay.sc + 32) = skq * inq * ink;
        *reinterpret_cast<uint32_t*>(st + lay.sc + 36) = (254u << 23) - sbits;       // 1 / oscale
    }
    const uint2 kapp = make_uint2(f2_to_bf16x2(k[0], k[1]), f2_to_bf16x2(k[2], k[3]));      // k_hat (bf16) for the window
    if (KDA) {
        nrm[64 + sl] = make_float4(pc[0], pc[1], pc[2], pc[3]);
        nrm[96 + sl] = make_float4(en[0], en[1], en[2], en[3]);
        signal();
        reinterpret_cast<uint2*>(P.Kbuf + (sh * L + h) * KD)[lane] = kapp;
        reinterpret_cast<float4*>(P.Pbuf + sh * KD)[lane] = make_float4(gn[0], gn[1], gn[2], gn[3]);
        __half2 e01 = __floats2half2_rn(en[0], en[1]), e23 = __floats2half2_rn(en[2], en[3]);
        reinterpret_cast<uint2*>(P.Gbuf + (sh * L + h) * KD)[lane] =
            make_uint2(*reinterpret_cast<uint32_t*>(&e01), *reinterpret_cast<uint32_t*>(&e23));
    } else {
        // window weights decay: w_j <- w_j alpha for the live entries, in the stage and (after the signal) in global memory
        float* ws = reinterpret_cast<float*>(st + lay.w);
        float wj[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j = lane + 32 * i;
            if (j < h) {
                wj[i] = ws[j] * sc.alpha;
                ws[j] = wj[i];
            }
        }
        signal();
        reinterpret_cast<uint2*>(P.Kbuf + (sh * L + h) * KD)[lane] = kapp;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j = lane + 32 * i;
            if (j < h) P.Wbuf[sh * L + j] = wj[i];
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// body: GT threads, operands in the shared-memory stage `st` (prologue done)
// ------------------------------------------------------------------------------------------------------------------
// `release()` is called by every thread after its last read of the stage and BEFORE the program's global stores: the
// stage hand-back is an mbarrier arrive with release semantics, which would otherwise wait for those stores to drain.
constexpr int MT = (VD / GW) / 16;                 // m16 tiles of tile rows per warp
template <int R, bool KDA, bool CONV, typename Release>
__device__ __forceinline__ void step_body(const StepParams& P, const ProgScalars& sc, char* st, const StageLayout& lay,
                                          const GroupScratch& gs, int t, int bar, Release release) {
    const int w = t >> 5, lane = t & 31, l8 = lane & 7, g = lane >> 3;
    const int L = P.d.L, h = sc.h;
    const int64_t sh = int64_t(sc.slot) * P.d.HV + sc.hv;
    const float* nrm = reinterpret_cast<const float*>(st + lay.nrm);
    // this lane's two values of the token's v, straight from global memory: issued now, used in the last phase
    // (CONV: the two raw projections, their conv state and taps; the value follows from conv_eval() at the end)
    uint32_t vraw = 0u;
    ConvRegs<2> vconv = {};
    const int vch = 2 * P.d.H * KD + sc.hv * VD + 2 * ((64 / GW) * w + ((t & 31) % (64 / GW)));      // this lane's first channel of v
    if constexpr (CONV) {
        if ((t & 31) < 64 / GW) vconv = conv_load<2>(P, sc.n, sc.slot, vch);      // (the lanes that finish the program)
    } else vraw = __ldg(reinterpret_cast<const uint32_t*>(P.mixed + int64_t(sc.n) * (2 * P.d.H * KD + P.d.HV * VD) + vch));

    // ---- KDA: decayed window keys K_j D_j (bf16, in place), D_j = en prod_{j<i<h} e_i; thread per key channel ----
    if (KDA) {
        if (t < KD) {
            uint16_t* kb = reinterpret_cast<uint16_t*>(st + lay.kb);
            const uint16_t* gb = reinterpret_cast<const uint16_t*>(st + lay.gb);
            float dcur = nrm[384 + 4 * nrm_chunk(t >> 2) + (t & 3)];
            // eight rows per trip: their loads are issued together, only the running product is a serial chain
            int j = h - 1;
            for (; j >= 7; j -= 8) {
                float kv[8], gv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    kv[u] = bf16_to_f(kb[(j - u) * KD + t]);
                    gv[u] = f16_to_f(gb[(j - u) * KD + t]);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    kb[(j - u) * KD + t] = f_to_bf16(kv[u] * dcur);
                    dcur *= gv[u];
                }
            }
            for (; j >= 0; --j) {
                kb[j * KD + t] = f_to_bf16(bf16_to_f(kb[j * KD + t]) * dcur);
                dcur *= f16_to_f(gb[j * KD + t]);
            }
        }
        named_bar(bar, GT);
    }

    // ---- checkpoint matvec on the tensor cores: D[v][n] = sum_c codes[v][c] B[c][n], n = {k hi, k lo, q hi, q lo}.
    //      A warp owns 32 rows = two m16 tiles; lane (gid, tig) holds rows gid and gid + 8 of a tile and, of each row, the
    //      sixteen codes at columns 16 tig and the sixteen at 64 + 16 tig: word s of those eight words feeds k-step s, so
    //      the k index of the instruction is a permutation of the columns that the B fragments below follow. ----
    {
        const int gid = lane >> 2, tig = lane & 3;
        uint32_t bfr[16];
        {
            uint4 x[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
            if (gid < 4) {
                const uint4* bp = reinterpret_cast<const uint4*>(st + lay.bop + gid * 256);
                x[0] = bp[tig * 2]; x[1] = bp[tig * 2 + 1]; x[2] = bp[8 + tig * 2]; x[3] = bp[8 + tig * 2 + 1];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) { bfr[4 * i] = x[i].x; bfr[4 * i + 1] = x[i].y; bfr[4 * i + 2] = x[i].z; bfr[4 * i + 3] = x[i].w; }
        }
        const float unscale = *reinterpret_cast<const float*>(st + lay.sc + 36);
        uint4 ac[4 * MT];
        {
            const uint4* tile = reinterpret_cast<const uint4*>(st + CK_CODES);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int rlo = (VD / GW) * w + 16 * mt + gid, rhi = rlo + 8;
                ac[4 * mt] = tile[rlo * 8 + tig]; ac[4 * mt + 1] = tile[rlo * 8 + 4 + tig];
                ac[4 * mt + 2] = tile[rhi * 8 + tig]; ac[4 * mt + 3] = tile[rhi * 8 + 4 + tig];
            }
        }
        float* mqyf = reinterpret_cast<float*>(gs.mqy);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int rlo = (VD / GW) * w + 16 * mt + gid, rhi = rlo + 8;
            const uint4 l0 = ac[4 * mt], l1 = ac[4 * mt + 1], h0 = ac[4 * mt + 2], h1 = ac[4 * mt + 3];
            const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
            const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
            float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};      // two accumulator chains per tile
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a0, a1, a2, a3;
                s8x4_to_h2x2(lw[ks], a0, a2);
                s8x4_to_h2x2(hw[ks], a1, a3);
                mma_f16_16816((ks & 1) ? e : d, a0, a1, a2, a3, bfr[2 * ks], bfr[2 * ks + 1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) d[i] += e[i];
            if (tig < 2) {                                   // tig 0 holds (k hi, k lo), tig 1 holds (q hi, q lo)
                const float* svp = reinterpret_cast<const float*>(st + CK_SV);
                mqyf[2 * rlo + tig] = (d[0] + d[1]) * unscale * svp[rlo];
                mqyf[2 * rhi + tig] = (d[2] + d[3]) * unscale * svp[rhi];
            }
        }
    }

    // ---- window dots dk_j = K_j . k_hat, dq_j = K_j . q_hat on the tensor cores: D[j][n] = sum_c K_j[c] B[c][n] with
    //      n = {k head, k remainder, q head, q remainder} (bf16, fp32 accumulate).  Sixteen rows per m16 tile, tiles dealt
    //      round-robin to the warps; lane (gid, tig) reads rows gid and gid + 8 as four 16-byte chunks at 64 c + 16 tig, so
    //      the k index of the instruction is again a permutation of the columns that the B fragments follow. ----
    {
        const int gid = lane >> 2, tig = lane & 3;
        const int nmt = (h + 15) >> 4;
        if (w < nmt) {
            uint32_t bfr[16];
            {
                uint4 x[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                if (gid < 4) {
                    const uint4* bp = reinterpret_cast<const uint4*>(st + lay.bdk + gid * 256 + tig * 16);
                    x[0] = bp[0]; x[1] = bp[4]; x[2] = bp[8]; x[3] = bp[12];
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) { bfr[4 * i] = x[i].x; bfr[4 * i + 1] = x[i].y; bfr[4 * i + 2] = x[i].z; bfr[4 * i + 3] = x[i].w; }
            }
            const float* ws = reinterpret_cast<const float*>(st + lay.w);        // GDN: already decayed by the prologue
            float* wdf = reinterpret_cast<float*>(gs.wd);
            for (int mt = w; mt < nmt; mt += GW) {
                const int j0 = 16 * mt + gid, j1 = j0 + 8;
                const char* p0 = st + lay.kb + (j0 < h ? j0 : h - 1) * 256 + tig * 16;      // rows past h repeat the last row
                const char* p1 = st + lay.kb + (j1 < h ? j1 : h - 1) * 256 + tig * 16;
                uint4 x0[4], x1[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    x0[c] = *reinterpret_cast<const uint4*>(p0 + 64 * c);
                    x1[c] = *reinterpret_cast<const uint4*>(p1 + 64 * c);
                }
                float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    mma_bf16_16816(d, x0[c].x, x1[c].x, x0[c].y, x1[c].y, bfr[4 * c], bfr[4 * c + 1]);
                    mma_bf16_16816(e, x0[c].z, x1[c].z, x0[c].w, x1[c].w, bfr[4 * c + 2], bfr[4 * c + 3]);
                }
                if (tig < 2) {                               // tig 0 holds (k head, k remainder), tig 1 holds (q head, q remainder)
                    if (j0 < h) wdf[2 * j0 + tig] = ws[j0] * ((d[0] + e[0]) + (d[1] + e[1]));
                    if (j1 < h) wdf[2 * j1 + tig] = ws[j1] * ((d[2] + e[2]) + (d[3] + e[3]));
                }
            }
        }
    }
    // ---- factor dots dU_r . k_hat, dU_r . q_hat (KDA: U_r[c] pc[c]) ----
#pragma unroll
    for (int cr = 0; cr < R / 4; ++cr) {
        if (((((h + 15) >> 4) + cr) % GW) == w) {
            // k_hat, q_hat (fp32) of this lane's 16 columns: only the warp that takes this chunk of factor rows reads them
            float2 kn[8], qn[8];
            {
                const float4* kp = reinterpret_cast<const float4*>(nrm);
                const float4* qp = reinterpret_cast<const float4*>(nrm + 128);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 a = kp[nrm_chunk(l8 * 4 + i)], b = qp[nrm_chunk(l8 * 4 + i)];
                    kn[2 * i] = make_float2(a.x, a.y); kn[2 * i + 1] = make_float2(a.z, a.w);
                    qn[2 * i] = make_float2(b.x, b.y); qn[2 * i + 1] = make_float2(b.z, b.w);
                }
            }
            const int r = 4 * cr + g;
            const uint4 r0 = reinterpret_cast<const uint4*>(st + CK_UQ + r * 512)[l8 * 2];
            const uint4 r1 = reinterpret_cast<const uint4*>(st + CK_UQ + r * 512)[l8 * 2 + 1];
            const uint32_t ww[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            float2 ak = make_float2(0.f, 0.f), aq = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float2 x = f16x2_to_f2(ww[i]);
                if (KDA) x = __fmul2_rn(x, *reinterpret_cast<const float2*>(nrm + 256 + 4 * nrm_chunk(l8 * 4 + (i >> 1)) + 2 * (i & 1)));
                ak = __ffma2_rn(x, kn[i], ak);
                aq = __ffma2_rn(x, qn[i], aq);
            }
            const float dk = oct_sum(ak.x + ak.y), dq = oct_sum(aq.x + aq.y);
            if (l8 == 0) gs.wd[64 + r] = make_float2(dk, dq);
        }
    }

    named_bar(bar, GT);

    // ---- contribution of the window and of the rank-R part.  A warp owns VPW = 64 / GW value pairs; lane % VPW picks the
    //      pair and lane / VPW the phase of j; the phases are combined with shuffles. ----
    constexpr int VPW = 64 / GW;                             // value pairs per warp
    constexpr int NPH = 32 / VPW;                            // phases of j handled by the lanes of one value pair
    const int vp = VPW * w + (lane % VPW), jh = lane / VPW;
    float2 ck = make_float2(0.f, 0.f), cq = make_float2(0.f, 0.f), rk = make_float2(0.f, 0.f), rq = make_float2(0.f, 0.f);
    {
        const uint32_t* ub = reinterpret_cast<const uint32_t*>(st + lay.ub);
#pragma unroll 4
        for (int j = jh; j < h; j += NPH) {
            const float2 u2 = bf16x2_to_f2(ub[j * 64 + vp]);
            const float2 wd = gs.wd[j];
            ck = __ffma2_rn(u2, make_float2(wd.x, wd.x), ck);
            cq = __ffma2_rn(u2, make_float2(wd.y, wd.y), cq);
        }
        const uint32_t* uq = reinterpret_cast<const uint32_t*>(st + CK_UQ);
#pragma unroll
        for (int r = jh; r < R; r += NPH) {
            const float2 q2 = f16x2_to_f2(uq[r * 128 + 64 + vp]);
            const float2 dd = gs.wd[64 + r];
            rk = __ffma2_rn(q2, make_float2(dd.x, dd.x), rk);
            rq = __ffma2_rn(q2, make_float2(dd.y, dd.y), rq);
        }
    }
#pragma unroll
    for (int o = VPW; o < 32; o <<= 1) {
        ck.x += __shfl_xor_sync(0xffffffffu, ck.x, o); ck.y += __shfl_xor_sync(0xffffffffu, ck.y, o);
        cq.x += __shfl_xor_sync(0xffffffffu, cq.x, o); cq.y += __shfl_xor_sync(0xffffffffu, cq.y, o);
        rk.x += __shfl_xor_sync(0xffffffffu, rk.x, o); rk.y += __shfl_xor_sync(0xffffffffu, rk.y, o);
        rq.x += __shfl_xor_sync(0xffffffffu, rq.x, o); rq.y += __shfl_xor_sync(0xffffffffu, rq.y, o);
    }
    float u0 = 0.f, u1 = 0.f, y0 = 0.f, y1 = 0.f, pn = 0.f;
    if (jh == 0) {
        const float2 m0 = gs.mqy[2 * vp], m1 = gs.mqy[2 * vp + 1];
        if constexpr (CONV) {
            uint16_t vo[2];
            conv_eval<2>(vconv, vo);
            vraw = uint32_t(vo[0]) | (uint32_t(vo[1]) << 16);
        }
        const float2 vv = bf16x2_to_f2(vraw);
        const float beta = sc.beta;
        const float kq = *reinterpret_cast<const float*>(st + lay.sc + 32);
        if (KDA) {
            u0 = beta * (vv.x - (m0.x + rk.x + ck.x));
            u1 = beta * (vv.y - (m1.x + rk.y + ck.y));
            y0 = m0.y + rq.x + cq.x + kq * u0;
            y1 = m1.y + rq.y + cq.y + kq * u1;
        } else {
            pn = sc.pold * sc.alpha;
            u0 = beta * (vv.x - (pn * (m0.x + rk.x) + ck.x));
            u1 = beta * (vv.y - (pn * (m1.x + rk.y) + ck.y));
            y0 = pn * (m0.y + rq.x) + cq.x + kq * u0;
            y1 = pn * (m1.y + rq.y) + cq.y + kq * u1;
        }
    }
    release();
    if (jh == 0) {
        reinterpret_cast<uint32_t*>(P.o)[(int64_t(sc.n) * P.d.HV + sc.hv) * 64 + vp] = f2_to_bf16x2(y0, y1);
        reinterpret_cast<uint32_t*>(P.Ubuf)[(sh * L + h) * 64 + vp] = f2_to_bf16x2(u0, u1);
        if constexpr (CONV) conv_store_state<2>(P, sc.slot, vch, vconv);
        if (t == 0) {
            if (!KDA) P.Pbuf[sh] = pn;
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
__global__ void __launch_bounds__(GT, 2) step_direct_kernel(StepParams P) {
    extern __shared__ __align__(128) char stage_smem[];
    __shared__ ProgScalars s_sc;
    const int t = threadIdx.x;
    const int prog = blockIdx.x;
    const int n = prog / P.d.HV, hv = prog - n * P.d.HV;
    if (t == 0) s_sc = load_scalars(P, n, hv, KDA);
    __syncthreads();
    const ProgScalars sc = s_sc;
    const StageLayout lay = stage_layout(prog_live(sc, P.d.L) ? sc.h : 0, P.d.L, R, KDA);
    if (!prog_live(sc, P.d.L)) {
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
    if (t < 32) step_prologue<KDA>(P, sc, st, lay, t, [] {});
    __syncthreads();
    const GroupScratch gs = carve_scratch(stage_smem + stage_layout(P.d.L, P.d.L, R, KDA).bytes);
    step_body<R, KDA, false>(P, sc, st, lay, gs, t, 1, [] {});
}

#include "lq_step_warp.cuh"

// ------------------------------------------------------------------------------------------------------------------
// driver 2: persistent CTAs, producer warp + bulk asynchronous copies into a ring of stages
// ------------------------------------------------------------------------------------------------------------------
// warp 0: producer (places stages, publishes scalars), warp 1: copy issue, warp 2: prologue, warps 3 ..: NG consumer groups
// of GW warps.
// Shared memory: [ring of `ring_bytes`][NG group scratches][ND x (full, normed, empty) mbarriers][ND stage offsets][NG flags]
// [ND stage row counts].
// Program i (CTA-local sequence number) uses descriptor i % ND: three mbarriers and the offset of its stage in the ring.
// Stages are carved from the ring in order, each sized for its program's live window rows, and reclaimed in order.
// Tail of the fused decode kernel: after its last program a CTA flushes the heads whose window it has just filled.
struct FuseTail {
    const float* Q0;
    int iters;
    int teams;                                      // teams of 256 threads that fit in the ring side by side (1 or 2)
    int team_bytes;                                 // shared memory of one team
    int* work;                                      // mailboxes of due heads (global scratch, see WL_*) or null: every CTA flushes its own
};
// Shared mailboxes of the fused flush (global scratch of the caller, all zero between launches).  A serving batch fills the
// windows of a few rows per step, and the program -> CTA map puts two or three of their heads on some CTAs and none on
// others.  A CTA keeps the first head whose window it fills; the second and the third go into its own mailbox (a few slots
// per CTA: plain stores, no atomics) as soon as their program has run, while the CTA still has programs ahead of it, and any
// more stay with it.  A CTA that filled none scans the mailboxes when its programs are done and claims an entry with an
// atomic exchange, which also empties the slot.  The owner, when it has flushed what it kept, claims back whatever is still
// in its mailbox and flushes that too: every entry is flushed exactly once whether or not anybody helps, so nobody waits
// for anybody for correctness, helpers may give up at any time, and the slots are all zero again when the kernel ends.
// Helpers stop when the launch's reports are complete and a scan finds nothing: every CTA adds one to a counter when its
// programs are done; the CTA that makes it `grid` sets the counter back to zero and bumps a generation word, which every
// CTA read when it started (its own report, and therefore the last one, comes after that read).
// (When every window fills in the same step each CTA has dozens of heads: it posts two, nobody has time for them, and it
// takes them back at the end.)
constexpr int WL_DONE = 0, WL_GEN = 1, WL_BOX = 16;              // int offsets: reports of this launch, generation, mailboxes
constexpr int WL_SLOTS = 4;                                      // slots per CTA (at most two are used); entry = head + 1
constexpr int WL_EARLY = 2;                                      // heads after a CTA's first that are posted (the rest stay with it)
constexpr int WL_MAX_CTAS = 1024;                                // the scratch is sized for launches of up to this many CTAs
constexpr int WL_ITEMS = WL_BOX;                                 // (first int after the header)
constexpr uint32_t WL_HELP_POLLS = 4096;                         // a helper gives up after this many empty scans (about a millisecond)
__device__ __forceinline__ void st_volatile_i32(int* p, int v) { *reinterpret_cast<volatile int*>(p) = v; }
__device__ __forceinline__ int ld_volatile_i32(const int* p) { return *reinterpret_cast<const volatile int*>(p); }

#ifndef LQ_NPW
#define LQ_NPW 2
#endif
constexpr int NPW = LQ_NPW;                     // prologue warps; warp 2 + k takes the programs i = k (mod NPW)
constexpr int UT = 32 * (2 + NPW);              // utility threads ahead of the consumer groups: producer, copy issue, prologues
constexpr int ND = 16;                         // descriptors = most programs resident in the ring at once

// CONV: q | k | v come out of the fused causal conv1d update.  The q and k channels of a key head are shared by its GQA
// value heads, and their conv state may be rewritten only once every one of those programs has read it; so the CONV kernels
// deal out KEY-HEAD UNITS (row n, key head hk) to the CTAs instead of single programs: a CTA runs the GQA programs of a unit
// one after the other, and ONE prologue warp takes all of them, computes q and k once and then writes the state back.
template <int R, bool KDA, int NG, bool FUSE, bool CONV>
__global__ void __launch_bounds__(UT + NG * GT, 1) step_pipelined_kernel(StepParams P, int ring_bytes, FuseTail ft) {
    extern __shared__ __align__(128) char stage_smem[];
    char* scratch0 = stage_smem + ring_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(scratch0 + NG * SCRATCH_BYTES);
    uint64_t* normed = full + ND;
    uint64_t* empty = normed + ND;
    uint64_t* ready = empty + ND;                 // stage placed, scalars written: the copy-issue warp may go
    volatile int* doff = reinterpret_cast<volatile int*>(ready + ND);
    volatile int* gflag0 = doff + ND;
    ProgScalars* pbatch = reinterpret_cast<ProgScalars*>(const_cast<int*>(doff) + 2 * ND + NG + 2);      // [32], 8-byte aligned
    int* dl_n = reinterpret_cast<int*>(pbatch + 32);             // fused flush: number of due heads, abort flag, the heads
    volatile int* abortf = dl_n + 1;
    int* dl = dl_n + 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int HV = P.d.HV, H = P.d.H, L = P.d.L;
    const int grid = gridDim.x, bid = blockIdx.x;
    const int gqa = HV / H;
    // program i of this CTA: (row, value head).  Plain kernels: program index bid + i * grid.  CONV: unit bid + (i / gqa) * grid.
    const int nunits = CONV ? P.N * H : P.N * HV;
    const int nit = ((nunits - bid + grid - 1) / grid) * (CONV ? gqa : 1);
    auto row_head = [&](int i, int& n, int& hv) {
        if constexpr (CONV) {
            const int u = bid + (i / gqa) * grid;
            n = u / H;
            hv = (u - n * H) * gqa + (i % gqa);
        } else {
            const int pgm = bid + i * grid;
            n = pgm / HV;
            hv = pgm - n * HV;
        }
    };

    if (tid == 0) {
        *dl_n = 0;
        *abortf = 0;
        for (int s = 0; s < ND; ++s) {
            mbar_init(full + s, 1);
            mbar_init(normed + s, 32);
            mbar_init(empty + s, GT);
            mbar_init(ready + s, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    __syncthreads();
    pdl_trigger();
    pdl_wait();                                                  // everything below reads what earlier kernels of the stream wrote
    int gen0 = 0;                                                // (thread 0) generation of the mailboxes when this CTA started
    if (FUSE && tid == 0 && ft.work != nullptr) gen0 = ld_volatile_i32(ft.work + WL_GEN);

    auto run_roles = [&]() {
    if (warp == 0) {
        // ================= producer: scalars of 32 programs per batch, then one stage placement per program =================
        // Scalars of 32 programs per batch, one program per lane, fetched two levels ahead: while batch b is placed, the
        // counters and gates of batch b + 1 and the slots of batch b + 2 are in flight.
        ProgScalars cur;
        auto slot_of = [&](int i) -> int {
            if (i >= nit) return 0;
            int n, hv;
            row_head(i, n, hv);
            return P.idx[n];
        };
        auto raw_of = [&](int i, int slot) {
            int n, hv;
            row_head(i < nit ? i : 0, n, hv);
            return load_raw(P, n, hv, i < nit ? slot : 0, KDA);
        };
        int slot_b;
        RawScalars rnx;
        {
            const int s0 = slot_of(lane);
            slot_b = slot_of(32 + lane);
            rnx = raw_of(lane, s0);
        }
        // The ring is a FIFO: stages are placed in program order and reclaimed in program order.  Space is accounted in
        // virtual bytes: a stage that does not fit before the end of the ring starts at 0 and the skipped tail counts as
        // allocated, so the virtual position modulo the ring size is always the physical offset and the live programs
        // tail .. i-1 occupy the virtual range [start of tail, vhead), which must never exceed the ring size.
        int head = 0, tail = 0;                                  // next free ring byte; oldest program not yet reclaimed
        uint32_t vhead = 0, r_vs = 0;                            // virtual head; lane (i % ND) keeps the virtual start of program i
        bool ok = true;
        for (int base = 0; base < nit && ok; base += 32) {
            cur = finish_scalars(rnx, KDA);
            __syncwarp();
            pbatch[lane] = cur;                                  // the batch's scalars, one entry per lane
            __syncwarp();
            rnx = raw_of(base + 32 + lane, slot_b);
            slot_b = slot_of(base + 64 + lane);
            const int cnt = min(32, nit - base);
            for (int j = 0; j < cnt; ++j) {
                const int i = base + j;
                const int dsc = i % ND;
                const ProgScalars sc = *const_cast<const ProgScalars*>(&pbatch[j]);      // broadcast read
                const bool live = prog_live(sc, L);
                const int rows = live ? sc.h : 0;
                const StageLayout lay = stage_layout(rows, L, R, KDA, false);
                const int size = lay.bytes;
                int off = head;
                uint32_t v0 = vhead;
                if (head + size > ring_bytes) { v0 += uint32_t(ring_bytes - head); off = 0; }
                const uint32_t v1 = v0 + uint32_t(size);
                while (tail < i) {                               // reclaim in order until the stage and its descriptor are free
                    const uint32_t vt = __shfl_sync(0xffffffffu, r_vs, tail % ND);
                    if (v1 - vt <= uint32_t(ring_bytes) && i - tail < ND) break;
                    if (!warp_wait_bounded(empty + (tail % ND), uint32_t(tail / ND) & 1u, lane)) { ok = false; break; }
                    ++tail;
                }
                if (!ok) {
                    if (lane == 0) { atomicOr(&g_status, ST_PRODUCER_TIMEOUT); *abortf = 1; }
                    break;
                }
                if (lane == dsc) r_vs = v0;
                head = off + size;
                vhead = v1;
                char* st = stage_smem + off;
                if (lane == 0) {
                    doff[dsc] = off;
                    doff[ND + NG + dsc] = rows;
                    *reinterpret_cast<ProgScalars*>(st + lay.sc) = sc;
                    if (live) {
                        uint32_t bytes = uint32_t(ck_bytes(R)) + 2u * uint32_t(sc.h) * 256u + uint32_t(L) * 4u;
                        if (KDA) bytes += uint32_t(sc.h) * 256u + 512u + 256u + 512u;
                        mbar_arrive_expect_tx(full + dsc, bytes);
                    }                                            // a dead program's `full` is completed by the copy-issue warp
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(ready + dsc);
            }
        }
        return;
    }

    if (warp == 1) {
        // ================= copy issue: one bulk asynchronous copy per lane and program =================
        // Per-lane copy descriptor, fixed for the whole kernel: lane k < ncopy issues copy k of every program from
        //   src = base + slot * c_slot + hv * c_hv + n * c_n + hk * c_hk,   bytes = b_fix + h * b_h,
        // into stage + o_fix + h * o_h (the stage layout moves with the live rows h).
        const char* c_base = nullptr;
        uint32_t c_slot = 0, c_hv = 0, c_n = 0, c_hk = 0, b_fix = 0, b_h = 0, o_fix = 0, o_h = 0;
        {
            const uint32_t rowb = uint32_t(L) * 256u;                    // one head's window rows (bf16 / f16) in bytes
            const StageLayout l0 = stage_layout(0, L, R, KDA, false), l1 = stage_layout(1, L, R, KDA, false);
            int which = -1;                                              // member of the layout this lane copies into
            switch (lane) {
                case 0: c_base = P.ssm; c_slot = uint32_t(P.d.SS) * 4u; c_hv = VD * KD * 4u; b_fix = ck_bytes(R); break;
                case 1: c_base = reinterpret_cast<const char*>(P.Kbuf); c_slot = uint32_t(HV) * rowb; c_hv = rowb; b_h = 256u; which = 0; break;
                case 2: c_base = reinterpret_cast<const char*>(P.Ubuf); c_slot = uint32_t(HV) * rowb; c_hv = rowb; b_h = 256u; which = 1; break;
                case 3: c_base = reinterpret_cast<const char*>(P.Wbuf); c_slot = uint32_t(HV * L) * 4u; c_hv = uint32_t(L) * 4u; b_fix = uint32_t(L) * 4u; which = 2; break;
                case 7: if (KDA) { c_base = reinterpret_cast<const char*>(P.Gbuf); c_slot = uint32_t(HV) * rowb; c_hv = rowb; b_h = 256u; which = 6; } break;
                case 8: if (KDA) { c_base = reinterpret_cast<const char*>(P.Pbuf); c_slot = uint32_t(HV) * 512u; c_hv = 512u; b_fix = 512u; which = 7; } break;
                case 9: if (KDA) { c_base = reinterpret_cast<const char*>(P.a); c_n = uint32_t(HV) * 256u; c_hv = 256u; b_fix = 256u; which = 8; } break;
                case 10: if (KDA) { c_base = reinterpret_cast<const char*>(P.dt_bias); c_hv = 512u; b_fix = 512u; which = 9; } break;
                default: break;
            }
            const int m0[10] = {l0.kb, l0.ub, l0.w, l0.q, l0.k, l0.v, l0.gb, l0.pb, l0.a, l0.dtb};
            const int m1[10] = {l1.kb, l1.ub, l1.w, l1.q, l1.k, l1.v, l1.gb, l1.pb, l1.a, l1.dtb};
#pragma unroll
            for (int k = 0; k < 10; ++k)
                if (which == k) { o_fix = uint32_t(m0[k]); o_h = uint32_t(m1[k] - m0[k]); }
            __syncwarp();
        }
        const uint64_t keep_policy = l2_policy_evict_last();
        for (int i = 0; i < nit; ++i) {
            const int dsc = i % ND;
            if (!warp_wait_bounded(ready + dsc, uint32_t(i / ND) & 1u, lane)) {
                if (lane == 0) { atomicOr(&g_status, ST_PRODUCER_TIMEOUT); *abortf = 1; }
                return;
            }
            char* st = stage_smem + doff[dsc];
            const int rows = doff[ND + NG + dsc];
            const ProgScalars sc = *reinterpret_cast<const ProgScalars*>(st + stage_layout(rows, L, R, KDA, false).sc);
            if (prog_live(sc, L)) {
                // The ring bytes under this stage were read and written through the generic proxy by the previous tenants'
                // prologue and consumers; their accesses are visible here through the empty -> ready barrier chain, and this
                // fence orders them before the asynchronous-proxy writes issued below.
                fence_async_smem();
                const uint32_t hk = uint32_t(sc.hv) / uint32_t(gqa);
                const char* src = c_base + uint64_t(uint32_t(sc.slot)) * c_slot + uint64_t(uint32_t(sc.hv)) * c_hv +
                                  uint64_t(uint32_t(sc.n)) * c_n + uint64_t(hk) * c_hk;
                const uint32_t bytes = b_fix + uint32_t(sc.h) * b_h;
                // a program that fills its window is followed, at the end of this launch, by the flush of the same head, which
                // reads the same checkpoint and window rows again: its copies ask L2 to keep those lines
                if (bytes) {
                    if (FUSE && sc.h + 1 == L) bulk_g2s_hint(st + o_fix + uint32_t(sc.h) * o_h, src, bytes, full + dsc, keep_policy);
                    else bulk_g2s(st + o_fix + uint32_t(sc.h) * o_h, src, bytes, full + dsc);
                }
            } else if (lane == 0) {
                // nothing to copy (padding row, null slot or full window): this warp completes the phase itself.  Doing it here
                // and not in the producer keeps this warp inside the full -> normed -> empty chain for every program, so the
                // producer can never run a whole round of descriptors ahead of it, however long a run of dead programs is.
                mbar_arrive(full + dsc);
            }
        }
        return;
    }

    if (warp < 2 + NPW) {
        // ================= prologue warps: programs dealt round-robin, each warp in fill order =================
        // q and k of a program come straight from global memory into this warp's registers (lane = four channels), fetched
        // one program of this warp ahead: row and key head follow from the program index alone
        auto run_prologue = [&](int i, const uint2& q_cur, const uint2& k_cur) -> bool {
            const int dsc = i % ND;
            if (!warp_wait_bounded(full + dsc, uint32_t(i / ND) & 1u, lane)) {
                if (lane == 0) { atomicOr(&g_status, ST_PROLOGUE_TIMEOUT); *abortf = 1; }
                return false;
            }
            char* st = stage_smem + doff[dsc];
            const int rows = doff[ND + NG + dsc];                  // rows the stage was sized for (h, or 0 for a dead program)
            const ProgScalars sc = *reinterpret_cast<const ProgScalars*>(st + stage_layout(rows, L, R, KDA, false).sc);
            if (prog_live(sc, L)) {
                const StageLayout lay = stage_layout(sc.h, L, R, KDA, false);
                step_prologue<KDA>(P, sc, st, lay, lane, [&] { mbar_arrive(normed + dsc); }, true, q_cur, k_cur);
            } else {
                mbar_arrive(normed + dsc);
            }
            return true;
        };
        if constexpr (CONV) {
            // warp k takes the units k, k + NPW, ... of this CTA: the raw q and k projections of the unit, their conv state and
            // taps are fetched one unit ahead; the conv runs once, the new state is written back at once (every reader of the
            // old one is this warp), and the unit's GQA programs all use the result
            const int nun = nit / gqa;
            // The conv inputs of a unit are loaded one unit of this warp ahead and its slot two units ahead, so that no
            // load waits for another: index -> slot one trip, slot -> conv state and projections the next.
            ConvRegs<4> cq = {}, ck = {};
            int slot_nx = 0, raw_nx2 = 0;
            auto slot_fetch = [&](int uu) { raw_nx2 = uu < nun ? P.idx[(bid + uu * grid) / H] : 0; };      // (a load, nothing else)
            auto unit_fetch = [&](int uu, int raw) {
                slot_nx = 0;
                if (uu >= nun || raw <= 0 || raw >= P.d.NS) return;
                const int u = bid + uu * grid, n2 = u / H, hk2 = u - n2 * H;
                slot_nx = raw;
                cq = conv_load<4>(P, n2, raw, hk2 * KD + 4 * lane);
                ck = conv_load<4>(P, n2, raw, (H + hk2) * KD + 4 * lane);
            };
            slot_fetch(warp - 2);
            unit_fetch(warp - 2, raw_nx2);
            slot_fetch(warp - 2 + NPW);
            for (int uu = warp - 2; uu < nun; uu += NPW) {
                uint2 q_cur = make_uint2(0u, 0u), k_cur = make_uint2(0u, 0u);
                if (slot_nx > 0) {
                    const int u = bid + uu * grid, n1 = u / H, hk1 = u - n1 * H;
                    uint16_t qo[4], ko[4];
                    conv_eval<4>(cq, qo);
                    conv_eval<4>(ck, ko);
                    q_cur = make_uint2(uint32_t(qo[0]) | (uint32_t(qo[1]) << 16), uint32_t(qo[2]) | (uint32_t(qo[3]) << 16));
                    k_cur = make_uint2(uint32_t(ko[0]) | (uint32_t(ko[1]) << 16), uint32_t(ko[2]) | (uint32_t(ko[3]) << 16));
                }
                // the new conv state of q and k: three words per tap, kept until the unit's programs have been signalled
                // (the signal is a release, and would wait for these stores to drain)
                const int slot_cur = slot_nx;
                uint32_t nq[3][2], nk[3][2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    nq[0][e] = cq.st[1][e]; nq[1][e] = cq.st[2][e]; nq[2][e] = cq.x[e];
                    nk[0][e] = ck.st[1][e]; nk[1][e] = ck.st[2][e]; nk[2][e] = ck.x[e];
                }
                const int raw = raw_nx2;
                slot_fetch(uu + 2 * NPW);
                unit_fetch(uu + NPW, raw);
                bool ok = true;
                for (int g2 = 0; g2 < gqa && ok; ++g2) ok = run_prologue(uu * gqa + g2, q_cur, k_cur);
                if (slot_cur > 0) {
                    const int u = bid + uu * grid, n1 = u / H, hk1 = u - n1 * H;
                    conv_store_words<4>(P, slot_cur, hk1 * KD + 4 * lane, nq);
                    conv_store_words<4>(P, slot_cur, (H + hk1) * KD + 4 * lane, nk);
                }
                if (!ok) return;
            }
        } else {
            const int MIXq = 2 * H * KD + HV * VD;
            uint2 q_nx = make_uint2(0u, 0u), k_nx = make_uint2(0u, 0u);
            auto qk_fetch = [&](int i2) {
                if (i2 >= nit) return;
                int n2, hv2;
                row_head(i2, n2, hv2);
                const int hk2 = hv2 / gqa;
                const uint2* mrow = reinterpret_cast<const uint2*>(P.mixed + int64_t(n2) * MIXq);
                q_nx = __ldg(mrow + hk2 * 32 + lane);
                k_nx = __ldg(mrow + (H + hk2) * 32 + lane);
            };
            qk_fetch(warp - 2);
            for (int i = warp - 2; i < nit; i += NPW) {
                const uint2 q_cur = q_nx, k_cur = k_nx;
                qk_fetch(i + NPW);
                if (!run_prologue(i, q_cur, k_cur)) return;
            }
        }
        return;
    }

    // ================= consumers: group g takes programs g, g + NG, ... =================
    const int g = (warp - 2 - NPW) / GW;
    const int t = tid - UT - g * GT;
    const int bar = 1 + g;
    const GroupScratch gs = carve_scratch(scratch0 + g * SCRATCH_BYTES);
    volatile int* gflag = gflag0 + g;
    // A head whose window is full goes on this CTA's list.  With the mailboxes the second and the third head of the list are
    // posted at once, while the CTA still has programs to run: a CTA that ends its programs with nothing to flush then finds
    // them in its first look.  (Called by the whole group; `wrote`: the group has just written the head's new window entry.)
    auto note_due = [&](int head, bool wrote) {
        if (ft.work == nullptr) {
            if (t == 0) dl[atomicAdd(dl_n, 1)] = head;
            return;
        }
        if (wrote) named_bar(bar, GT);                          // every thread's stores to the head are issued
        if (t == 0) {
            const int k = atomicAdd(dl_n, 1);
            dl[k] = head;
            if (k >= 1 && k <= WL_EARLY) {
                __threadfence();                                 // the head's data comes before its entry
                st_volatile_i32(ft.work + WL_BOX + bid * WL_SLOTS + (k - 1), head + 1);
            }
        }
    };
    for (int i = g; i < nit; i += NG) {
        const int dsc = i % ND;
        // one warp polls and publishes the outcome; the other warps sleep at the group barrier
        if (t < 32) {
            const bool got = warp_wait_bounded(normed + dsc, uint32_t(i / ND) & 1u, t);
            if (t == 0) *gflag = got ? 1 : 0;
        }
        named_bar(bar, GT);
        if (*gflag == 0) {                              // uniform decision: nobody enters the body unless the data is there
            if (t == 0) { atomicOr(&g_status, ST_CONSUMER_TIMEOUT); *abortf = 1; }
            return;
        }
        char* st = stage_smem + doff[dsc];
        const int rows = doff[ND + NG + dsc];
        const StageLayout lay = stage_layout(rows, L, R, KDA, false);
        const ProgScalars sc = *reinterpret_cast<const ProgScalars*>(st + lay.sc);
        auto release = [&] { mbar_arrive(empty + dsc); };
        if (prog_live(sc, L)) {
            step_body<R, KDA, CONV>(P, sc, st, lay, gs, t, bar, release);
            if (FUSE && sc.h + 1 == L) note_due(sc.slot * HV + sc.hv, true);                        // window just filled
        } else {
            if (FUSE && sc.slot > 0 && sc.h == L) note_due(sc.slot * HV + sc.hv, false);             // was full already
            release();
            int n0, hv0;
            row_head(i, n0, hv0);
            if (t < 64) reinterpret_cast<uint32_t*>(P.o)[(int64_t(n0) * HV + hv0) * 64 + t] = 0u;
            if constexpr (CONV) {                           // the row still advances its conv state (v channels of this head)
                if (t < 64 && sc.slot > 0) {
                    const int vch = 2 * H * KD + hv0 * VD + 2 * t;
                    const ConvRegs<2> r2 = conv_load<2>(P, n0, sc.slot, vch);
                    conv_store_state<2>(P, sc.slot, vch, r2);
                }
            }
        }
    }
    };
    run_roles();

    // ================= fused flush: the heads whose window this CTA just filled =================
    // While at least two heads are left the CTA works as two teams of 8 warps, each flushing one head in its own work area
    // (carved from the dead ring) with its own 128 columns of tensor memory; a last single head -- or every head, when the
    // ring has room for one work area only -- is flushed by all 16 warps as one team, which halves the stages that are
    // parallel over the tile.  A serving batch whose sequences fill their windows at different steps gives most CTAs exactly
    // one head per step, and the latency of that flush is what the step pays.
    if constexpr (FUSE) {
        __shared__ uint32_t tm_slot;
        __shared__ int s_pop[4];
        __shared__ int s_list[24];                               // mailbox slots a scan found occupied
        static_assert(UT + NG * GT == 512, "the fused flush is written for two teams of 256 threads");
        const int nteams = ft.teams;                             // work areas that fit in the ring: 1 or 2
        const int team = tid >> 8, ttid = tid & 255;
        FlushArgs A;
        A.d = P.d; A.ssm = P.ssm; A.Kbuf = P.Kbuf; A.Ubuf = P.Ubuf; A.Wbuf = P.Wbuf; A.Pbuf = P.Pbuf; A.Gbuf = P.Gbuf;
        A.hcnt = P.hcnt; A.Q0 = ft.Q0; A.iters = ft.iters;
        __syncthreads();                                         // every role is done; the ring is dead, this CTA's global writes are issued
        const int ndl = *abortf ? 0 : *dl_n;
        int* const wl = ft.work;
        if (wl == nullptr && ndl == 0) return;                   // (before any tensor memory is held)
        // dl[1 .. npub] were posted by the consumers when they found them; the CTA keeps dl[0] and dl[npub + 1 ..]
        const int nfound = *dl_n;                               // (also after an abort: what was posted has to be taken back)
        const int npub = wl == nullptr ? 0 : (nfound - 1 < WL_EARLY ? (nfound > 1 ? nfound - 1 : 0) : WL_EARLY);
        int* const box = wl + WL_BOX;
        if (tid == 0) {
            s_pop[2] = 0; s_pop[3] = 0;                          // [2]: occupied slots found by a scan, [3]: 1 = nothing was posted in this launch
            if (npub > 0) dl[npub] = dl[0];                      // the kept heads, contiguous: dl[npub .. nfound - 1]
        }
        if (wl != nullptr) {
            __syncthreads();
            if (tid == 0) {
                // one word counts the reports (low 16 bits) and the heads posted (above them)
                const int old = atomicAdd(wl + WL_DONE, 1 + (npub << 16));
                if ((old & 0xffff) == grid - 1) {                // the last CTA to report closes the launch's count at once: the others
                    const int any = ((old >> 16) + npub) > 0;    // learn from the generation that no more heads will be posted, and from
                    st_volatile_i32(wl + WL_DONE, 0);            // its low bit whether any was.  (This thread reaches the first barrier
                    st_volatile_i32(wl + WL_GEN, (gen0 & ~1) + 2 + any);      // of its flush a round trip late; the flush starts with
                    if (!any) s_pop[3] = 1;                      // global loads that take as long.)
                }
            }
        }
        // Rounds of heads: first what this CTA keeps of its own list; with the mailboxes, then one head per round -- its own
        // posted heads that nobody took, or, for a CTA that filled nothing, heads from other CTAs' mailboxes.
        __syncthreads();                                         // (dl[npub] is in place)
        const int* heads = dl + npub;
        int nh = ndl > 0 ? ndl - npub : 0;
        int reclaim = 0;                                         // (thread 0) next slot of the own mailbox to look at
        const int total = grid * WL_SLOTS;
        bool inited = false;
        bool more = true;
        while (more) {
            if (nh == 0) {                                       // (mailboxes only) find the next head
                if (tid == 0) {
                    int q = -1;
                    if (!*abortf) {
                        for (; reclaim < npub && q < 0; ++reclaim) {
                            const int x = atomicExch(box + bid * WL_SLOTS + reclaim, 0);
                            if (x > 0) q = x - 1;
                        }
                    } else {                                     // a wait ran out somewhere in this CTA (the status word says so): what it
                        for (; reclaim < npub; ++reclaim) atomicExch(box + bid * WL_SLOTS + reclaim, 0);       // posted must not outlive the launch
                    }
                    s_pop[0] = q;
                }
                __syncthreads();
                int q = s_pop[0];
                if (q < 0 && *abortf == 0 && s_pop[3] == 0) {    // nothing (left) of its own: help the others
                    // One trip = the generation and every mailbox slot, read side by side.  A scan that races with the last
                    // postings may miss one: its owner flushes it.  Occupied slots go to a short list and the CTA tries the one
                    // its number picks, so that helpers spread over the entries.
                    for (uint32_t it = 0; it < WL_HELP_POLLS; ++it) {
                        int g = 0;
                        if (tid == 0) g = ld_volatile_i32(wl + WL_GEN);
                        for (int i = tid; i < total; i += UT + NG * GT)
                            if (ld_volatile_i32(box + i) != 0) {
                                const int pos = atomicAdd(&s_pop[2], 1);
                                if (pos < 24) s_list[pos] = i;
                            }
                        __syncthreads();
                        if (tid == 0) {
                            int got = -1;                        // -1: nothing yet, -2: lost the race for an entry, -3: nothing more to come
                            const int nfound = min(s_pop[2], 24);
                            if (nfound > 0) {
                                const int x = atomicExch(box + s_list[(bid * 7 + int(it)) % nfound], 0);
                                got = x > 0 ? x - 1 : -2;
                                if (x > 0) __threadfence();      // the head's data is read after its entry
                            } else if (g != gen0) {
                                got = -3;
                            }
                            if (got < 0 && g != gen0 && (g & 1) == 0) got = -3;         // the launch closed with nothing posted
                            s_pop[0] = got;
                            s_pop[2] = 0;                        // (for the next scan)
                        }
                        __syncthreads();
                        const int got = s_pop[0];
                        if (got >= 0) q = got;
                        // leave the loop with a head, when the launch is over, or -- a CTA that had heads of its own comes late, when
                        // the postings are in -- as soon as a scan finds nothing; only a CTA that filled no window waits for more
                        if (got >= 0 || got == -3 || (got == -1 && ndl > 0)) it = WL_HELP_POLLS;
                        else if (got == -1) __nanosleep(100);
                    }
                    __syncthreads();
                    if (tid == 0) s_pop[0] = q;
                    __syncthreads();
                }
                heads = s_pop;
                nh = q >= 0 ? 1 : 0;
                if (nh == 0) more = false;
            }
            if (nh > 0) {
                if (!inited) {                                   // first head of this CTA: tensor memory and the per-team constants
                    if (warp == 0) tmem_alloc(&tm_slot, 2 * TMEM_COLS);
                    const FlushSmem fi = flush_carve<R>(stage_smem + (team < nteams ? team : 0) * ft.team_bytes, L, KDA);
                    if (team < nteams) flush_init<R>(fi, ft.Q0, ttid, 256);
                    tc_fence_before_sync();
                    __syncthreads();
                    tc_fence_after_sync();
                    inited = true;
                }
                const uint32_t tm = tm_slot;
                int k = 0;
                if (nteams == 2 && nh >= 2) {                    // pairs: each team of 8 warps goes through its own heads
                    const FlushSmem fs = flush_carve<R>(stage_smem + team * ft.team_bytes, L, KDA);
                    auto tsync = [&] { named_bar(8 + team, 256); };
                    const int npair = nh >> 1;
                    bool ok = true;
                    for (int i = 0; i < npair && ok; ++i) ok = flush_head<R, KDA, 8>(fs, A, heads[2 * i + team], ttid, tm + team * TMEM_COLS, tsync);
                    if (!ok && ttid == 0) *abortf = 1;
                    k = 2 * npair;
                    __syncthreads();
                }
                if (k < nh && *abortf == 0) {                    // a last single head: all 16 warps
                    const FlushSmem f0 = flush_carve<R>(stage_smem, L, KDA);
                    for (; k < nh; ++k)
                        if (!flush_head<R, KDA, 16>(f0, A, heads[k], tid, tm, [] { __syncthreads(); })) {
                            if (tid == 0) *abortf = 1;
                            k = nh;
                        }
                }
                __syncthreads();                                 // (s_pop is rewritten by the next round; abort flag settled)
            }
            if (wl == nullptr) more = false;
            nh = 0;
        }
        tc_fence_before_sync();
        __syncthreads();
        if (inited && warp == 0) tmem_dealloc(tm_slot, 2 * TMEM_COLS);
    }
}

// 0 = pipelined, 1 = direct, 2 = one warp per program (GDN; KDA falls back to the pipelined driver)
static std::atomic<int> g_step_impl{0};
// fewest (row, head) programs of a decode call for which the mailboxes are used; -1 = sixteen per SM
static std::atomic<int> g_work_list_min{-1};

// fuse != nullptr: the pipelined driver also flushes, in the same launch, the heads whose window it fills (Q0, iters from
// *fuse).  Returns LQ_ERR_UNSUPPORTED when the fused form is not available for the configuration (debug drivers, a flush
// team that does not fit in the ring): the caller then launches the two kernels separately.
// conv: q | k | v come from the fused causal conv1d update (P.cx etc. are set); only the fused pipelined form exists for it.
template <int R, bool KDA>
static int launch_step(const StepParams& P, cudaStream_t st, const FuseTail* fuse, bool conv = false) {
    const StageLayout lay = stage_layout(P.d.L, P.d.L, R, KDA);
    const int impl = (conv && fuse) ? 0 : g_step_impl.load(std::memory_order_relaxed);      // read once: one call never mixes two drivers
    if (conv && !fuse) return LQ_ERR_UNSUPPORTED;
    if (impl != 0 && fuse && !(impl == 2 && KDA)) return LQ_ERR_UNSUPPORTED;
    if (impl == 1) {
        const size_t smem = size_t(lay.bytes) + SCRATCH_BYTES;
        int rc = ensure_smem((const void*)step_direct_kernel<R, KDA>, smem);
        if (rc) return rc;
        step_direct_kernel<R, KDA><<<unsigned(P.N) * P.d.HV, GT, smem, st>>>(P);
        return finish_launch();
    }
    if (impl == 2 && !KDA) {
        const int nprog = P.N * P.d.HV;
        const int want = (nprog + WK_WARPS - 1) / WK_WARPS;
        const int cap = device_sm_count() * 4;
        step_warp_gdn_kernel<R><<<want < cap ? want : cap, 32 * WK_WARPS, 0, st>>>(P);
        return finish_launch();
    }
    constexpr int NG = LQ_NG;
    const int nprog = P.N * P.d.HV;
    const int nunits = conv ? P.N * P.d.H : nprog;               // what the CTAs are dealt: key-head units (conv) or programs
    const int grid = nunits < device_sm_count() ? nunits : device_sm_count();
    const int nit_max = ((nunits + grid - 1) / grid) * (conv ? P.d.HV / P.d.H : 1);
    const size_t budget = 227 * 1024 - 256;                      // (the kernel also has a few bytes of static shared memory)
    const size_t fixed = size_t(NG) * SCRATCH_BYTES + 4 * ND * sizeof(uint64_t) + (2 * ND + NG + 4) * sizeof(int) + 32 * sizeof(ProgScalars) +
                         (4 + size_t(nit_max)) * sizeof(int);
    const int lay_p = stage_layout(P.d.L, P.d.L, R, KDA, false).bytes;
    if (fixed + size_t(lay_p) > budget) return LQ_ERR_UNSUPPORTED;
    const int ring_bytes = int((budget - fixed) & ~size_t(127));
    if (ring_bytes < lay_p) return LQ_ERR_UNSUPPORTED;
    const size_t smem = size_t(ring_bytes) + fixed;
    FuseTail ft = {nullptr, 0, 0, 0, nullptr};
    cudaError_t le;
    if (fuse) {
        ft = *fuse;
        ft.team_bytes = int((flush_smem_bytes<R>(P.d.L, 0, KDA) + 127) & ~size_t(127));
        ft.teams = (2 * ft.team_bytes <= ring_bytes) ? 2 : (ft.team_bytes <= ring_bytes ? 1 : 0);
        if (ft.teams == 0) return LQ_ERR_UNSUPPORTED;
        // the mailboxes cost an atomic round trip or two per launch: they pay once a CTA has many programs
        const int wl_min = g_work_list_min.load(std::memory_order_relaxed);
        if (int64_t(P.N) * P.d.HV < (wl_min >= 0 ? int64_t(wl_min) : int64_t(16) * device_sm_count())) ft.work = nullptr;
        if (device_sm_count() > WL_MAX_CTAS) ft.work = nullptr;
        if (conv) {
            int rc = ensure_smem((const void*)step_pipelined_kernel<R, KDA, NG, true, true>, smem);
            if (rc) return rc;
            le = launch_dependent(step_pipelined_kernel<R, KDA, NG, true, true>, unsigned(grid), unsigned(UT + NG * GT), smem, st, P, ring_bytes, ft);
        } else {
            int rc = ensure_smem((const void*)step_pipelined_kernel<R, KDA, NG, true, false>, smem);
            if (rc) return rc;
            le = launch_dependent(step_pipelined_kernel<R, KDA, NG, true, false>, unsigned(grid), unsigned(UT + NG * GT), smem, st, P, ring_bytes, ft);
        }
    } else {
        int rc = ensure_smem((const void*)step_pipelined_kernel<R, KDA, NG, false, false>, smem);
        if (rc) return rc;
        le = launch_dependent(step_pipelined_kernel<R, KDA, NG, false, false>, unsigned(grid), unsigned(UT + NG * GT), smem, st, P, ring_bytes, ft);
    }
    if (le != cudaSuccess) { set_last_cuda_error(le); return LQ_ERR_LAUNCH; }
    return finish_launch();
}

static int check_conv(const lq_conv1d* c, int channels) {
    if (!c->x || !c->state || !c->weight) return LQ_ERR_NULL;
    if (c->width != CONV_W) return LQ_ERR_UNSUPPORTED;
    if (c->x_stride < channels || (c->x_stride & 7)) return LQ_ERR_RANGE;
    if (misaligned16({c->x, c->weight}) || (reinterpret_cast<uintptr_t>(c->state) & 7) || (c->bias && (reinterpret_cast<uintptr_t>(c->bias) & 7)))
        return LQ_ERR_ALIGN;
    // channels contiguous per tap: the kernels move four channels of a tap with one 8-byte access
    if (c->stride_dim == 1 && ((c->stride_tap & 3) || (c->stride_slot & 3))) return LQ_ERR_ALIGN;
    return LQ_OK;
}
static void set_conv(StepParams& P, const lq_conv1d* c) {
    P.cx = (const uint16_t*)c->x; P.cx_stride = c->x_stride; P.cstate = (uint16_t*)c->state; P.cw = (const uint16_t*)c->weight;
    P.cb = (const uint16_t*)c->bias; P.cs_slot = c->stride_slot; P.cs_dim = c->stride_dim; P.cs_tap = c->stride_tap;
}

static int step_common(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                       int32_t* hcnt, const void* mixed, const void* a, const void* b, const float* A_log,
                       const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale, float glb, bool kda,
                       void* stream, const FuseTail* fuse = nullptr, const lq_conv1d* conv = nullptr) {
    int rc = check_dims(d);
    if (rc) return rc;
    if (conv) {
        rc = check_conv(conv, 2 * d->H * d->K + d->HV * d->V);
        if (rc) return rc;
        mixed = conv->x;                                         // (takes the place of the q | k | v rows in the checks below)
    }
    if (!ssm || !Kbuf || !Ubuf || !Wbuf || !Pbuf || !hcnt || !A_log || !dt_bias || (kda && !Gbuf)) return LQ_ERR_NULL;
    if (N < 0) return LQ_ERR_RANGE;
    if (N == 0) return LQ_OK;
    if (!mixed || !a || !b || !idx || !o) return LQ_ERR_NULL;
    if (misaligned16({ssm, Kbuf, Ubuf, Wbuf, mixed, o})) return LQ_ERR_ALIGN;
    if (kda && misaligned16({Gbuf, Pbuf, a, dt_bias})) return LQ_ERR_ALIGN;
    StepParams P;
    P.d = *d; P.ssm = (char*)ssm; P.Kbuf = (uint16_t*)Kbuf; P.Ubuf = (uint16_t*)Ubuf; P.Wbuf = Wbuf; P.Pbuf = Pbuf;
    P.Gbuf = (uint16_t*)Gbuf; P.hcnt = hcnt; P.mixed = (const uint16_t*)mixed; P.a = (const uint16_t*)a;
    P.b = (const uint16_t*)b; P.A_log = A_log; P.dt_bias = dt_bias; P.idx = idx; P.o = (uint16_t*)o; P.N = N;
    P.scale = scale > 0.f ? scale : 1.0f / sqrtf(float(d->K));
    P.glb = glb;
    P.cx = nullptr; P.cstate = nullptr; P.cw = nullptr; P.cb = nullptr; P.cs_slot = P.cs_dim = P.cs_tap = 0; P.cx_stride = 0;
    if (conv) set_conv(P, conv);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool cv = conv != nullptr;
    if (kda) return d->R == 4 ? launch_step<4, true>(P, s, fuse, cv) : launch_step<8, true>(P, s, fuse, cv);
    return d->R == 4 ? launch_step<4, false>(P, s, fuse, cv) : launch_step<8, false>(P, s, fuse, cv);
}

// standalone conv update: one thread per two channels of a row, the arithmetic of the fused kernels
__global__ void __launch_bounds__(256) conv1d_update_kernel(StepParams P, int C, uint16_t* out, int64_t out_stride) {
    const int n = blockIdx.y, c0 = 2 * (blockIdx.x * 256 + threadIdx.x);
    if (c0 >= C) return;
    const int slot = P.idx[n];
    if (slot <= 0 || slot >= P.d.NS) return;                     // padding row: nothing read, nothing written
    const ConvRegs<2> r = conv_load<2>(P, n, slot, c0);
    uint16_t o2[2];
    conv_eval<2>(r, o2);
    *reinterpret_cast<uint32_t*>(out + int64_t(n) * out_stride + c0) = uint32_t(o2[0]) | (uint32_t(o2[1]) << 16);
    conv_store_state<2>(P, slot, c0, r);
}

}  // namespace lq

extern "C" int lq_set_option(const char* name, int32_t value) {
    if (!name) return LQ_ERR_NULL;
    if (strcmp(name, "step_impl") == 0) {
        if (value < 0 || value > 2) return LQ_ERR_RANGE;
        lq::g_step_impl.store(value, std::memory_order_relaxed);
        return LQ_OK;
    }
    if (strcmp(name, "work_list_min_programs") == 0) {
        lq::g_work_list_min.store(value < 0 ? -1 : value, std::memory_order_relaxed);
        return LQ_OK;
    }
    if (strcmp(name, "pdl") == 0) {
        lq::g_pdl.store(value != 0, std::memory_order_relaxed);
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

// Fused decode = step + flush of the heads that fill up, one launch; falls back to the two launches where the fused form
// is not available.  Same results as lq_*_step followed by lq_flush on the same rows.
static int decode_common(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf, int32_t* hcnt,
                         const void* mixed, const void* a, const void* b, const float* A_log, const float* dt_bias,
                         const int32_t* idx, void* o, int32_t N, float scale, float glb, bool kda, const float* Q0, int32_t iters,
                         void* work, int64_t work_bytes, void* stream, const lq_conv1d* conv = nullptr) {
    if (!Q0) return LQ_ERR_NULL;
    if (iters < 0) return LQ_ERR_RANGE;
    if (work) {                                                  // shared mailboxes of due heads
        if (reinterpret_cast<uintptr_t>(work) & 7) return LQ_ERR_ALIGN;
        if (d && N > 0 && work_bytes < lq_decode_work_bytes(N < d->NS ? N : d->NS, d->HV)) return LQ_ERR_RANGE;
    }
    lq::FuseTail ft = {Q0, iters, 0, 0, static_cast<int*>(work)};
    int rc = lq::step_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, idx, o, N, scale, glb, kda,
                             stream, &ft, conv);
    if (rc != LQ_ERR_UNSUPPORTED || conv) return rc;           // (the conv form exists as one fused launch only)
    rc = lq::step_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, idx, o, N, scale, glb, kda, stream);
    if (rc) return rc;
    return lq_flush(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Q0, idx, N, kda ? 1 : 0, iters, stream);
}

extern "C" int64_t lq_decode_work_bytes(int32_t rows, int32_t HV) {
    (void)rows;                                                  // (the scratch does not grow with the call: a few slots per CTA)
    (void)HV;
    return 4 * (int64_t(lq::WL_BOX) + int64_t(lq::WL_SLOTS) * lq::WL_MAX_CTAS);
}

extern "C" int lq_gdn_decode(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                             const void* mixed, const void* a, const void* b, const float* A_log, const float* dt_bias,
                             const int32_t* idx, void* o, int32_t N, float scale, const float* Q0, int32_t iters, void* work,
                             int64_t work_bytes, void* stream) {
    return decode_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, nullptr, hcnt, mixed, a, b, A_log, dt_bias, idx, o, N, scale, 0.f, false, Q0,
                         iters, work, work_bytes, stream);
}

extern "C" int lq_kda_decode(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                             int32_t* hcnt, const void* mixed, const void* a, const void* b, const float* A_log,
                             const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale, float glb, const float* Q0,
                             int32_t iters, void* work, int64_t work_bytes, void* stream) {
    return decode_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, idx, o, N, scale, glb, true, Q0,
                         iters, work, work_bytes, stream);
}

extern "C" int lq_gdn_decode_conv(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                                  const lq_conv1d* conv, const void* a, const void* b, const float* A_log, const float* dt_bias,
                                  const int32_t* idx, void* o, int32_t N, float scale, const float* Q0, int32_t iters, void* work,
                                  int64_t work_bytes, void* stream) {
    if (!conv) return LQ_ERR_NULL;
    return decode_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, nullptr, hcnt, nullptr, a, b, A_log, dt_bias, idx, o, N, scale, 0.f, false, Q0,
                         iters, work, work_bytes, stream, conv);
}

extern "C" int lq_kda_decode_conv(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                                  int32_t* hcnt, const lq_conv1d* conv, const void* a, const void* b, const float* A_log,
                                  const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale, float glb,
                                  const float* Q0, int32_t iters, void* work, int64_t work_bytes, void* stream) {
    if (!conv) return LQ_ERR_NULL;
    return decode_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, nullptr, a, b, A_log, dt_bias, idx, o, N, scale, glb, true, Q0,
                         iters, work, work_bytes, stream, conv);
}

// ------------------------------------------------------------------------------------------------------------------
// GDN decode for callers that must not allocate.  The mailboxes of due heads that lq_gdn_decode takes as `work` live
// here in a file-scope device array of fixed size, which every GPU that loads the library holds until the process exits.
// In host code the array's name only stands for the symbol: its device address comes from cudaGetSymbolAddress(), asked
// once per device with that device current, and is what the kernel is given.
// ------------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) int g_noalloc_work[lq::WL_BOX + lq::WL_SLOTS * lq::WL_MAX_CTAS];
static std::atomic<int*> g_noalloc_ptr[64];                     // per device: the array's address on that device (null = not asked yet)

extern "C" int lq_gdn_decode_noalloc(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                                     const void* mixed, const void* a, const void* b, const float* A_log, const float* dt_bias,
                                     const int32_t* idx, void* o, int32_t N, float scale, const float* Q0, int32_t iters,
                                     void* stream) {
    if (!d) return LQ_ERR_NULL;
    if (N < 0) return LQ_ERR_RANGE;
    const int64_t rows = N < d->NS ? N : d->NS;
    if (d->HV <= 0 || rows * int64_t(d->HV) > LQ_NOALLOC_MAX_HEADS) return LQ_ERR_LIMIT;        // larger than the largest call this entry takes
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        lq::set_last_cuda_error(e == cudaSuccess ? cudaErrorInvalidDevice : e);
        return LQ_ERR_LAUNCH;
    }
    int* ptr = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (!ptr) {                                                  // first call on this device (two threads may both ask: same answer)
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_work);
        if (e != cudaSuccess || !ptr) {
            lq::set_last_cuda_error(e == cudaSuccess ? cudaErrorInvalidSymbol : e);
            return LQ_ERR_LAUNCH;
        }
        g_noalloc_ptr[dev].store(ptr, std::memory_order_release);
    }
    if (N == 0) return LQ_OK;
    // the array keeps what the last call left (all zero after a call that ran to its end): the part this call uses starts at zero
    const size_t bytes = size_t(lq_decode_work_bytes(int32_t(rows), d->HV));
    e = cudaMemsetAsync(ptr, 0, bytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        lq::set_last_cuda_error(e);
        return LQ_ERR_LAUNCH;
    }
    return decode_common(d, ssm, Kbuf, Ubuf, Wbuf, Pbuf, nullptr, hcnt, mixed, a, b, A_log, dt_bias, idx, o, N, scale, 0.f, false, Q0,
                         iters, ptr, int64_t(sizeof(int)) * (lq::WL_BOX + lq::WL_SLOTS * lq::WL_MAX_CTAS), stream);
}

extern "C" int lq_causal_conv1d_update(const lq_conv1d* conv, const int32_t* idx, int32_t N, int32_t channels, int32_t NS, void* out,
                                       int64_t out_stride, void* stream) {
    if (!conv || !out || (N > 0 && !idx)) return LQ_ERR_NULL;
    if (N < 0 || channels <= 0 || (channels & 7) || NS < 1 || out_stride < channels || (out_stride & 1)) return LQ_ERR_RANGE;
    int rc = lq::check_conv(conv, channels);
    if (rc) return rc;
    if (reinterpret_cast<uintptr_t>(out) & 3) return LQ_ERR_ALIGN;
    if (N == 0) return LQ_OK;
    lq::StepParams P = {};
    P.d.NS = NS;
    P.idx = idx;
    lq::set_conv(P, conv);
    dim3 grid(unsigned((channels / 2 + 255) / 256), unsigned(N));
    lq::conv1d_update_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(P, channels, (uint16_t*)out, out_stride);
    return lq::finish_launch();
}
