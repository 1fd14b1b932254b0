// Shared device helpers for the leapquant_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <atomic>
#include <initializer_list>

#include "../../include/leapquant_b200.h"

namespace lq {

constexpr int KD = 128;                 // key dim
constexpr int VD = 128;                 // value dim
constexpr float QMAX = 127.0f;
constexpr float EPS = 1e-12f;
constexpr float SOFTPLUS_THRESHOLD = 20.0f;
constexpr float PNMIN = 1e-20f;
constexpr float RNE_MAGIC = 12582912.0f;   // 1.5 * 2^23

// ---- packed checkpoint layout inside one (slot, head) region (byte offsets) ----
constexpr int CK_CODES = 0;
constexpr int CK_SK = VD * KD;                       // f32 Sk[K]
constexpr int CK_SV = CK_SK + 4 * KD;                // f32 Sv[V]
constexpr int CK_UQ = CK_SV + 4 * VD;                // f16 [R][K+V]
__host__ __device__ constexpr int ck_bytes(int R) { return CK_UQ + 2 * R * (KD + VD); }

__device__ __forceinline__ char* head_base(void* ssm, int64_t SS, int slot, int hv) {
    return reinterpret_cast<char*>(ssm) + 4 * (int64_t(slot) * SS + int64_t(hv) * VD * KD);
}

// device-side status word: a kernel that gives up a bounded wait ORs a code in here and returns.
// The library is built as ONE translation unit, so this is the single copy every kernel and lq_device_status() see.
static __device__ int g_status = 0;

// ---- conversions ----
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t w) { return make_float2(bf16lo(w), bf16hi(w)); }
__device__ __forceinline__ uint32_t f2_to_bf16x2(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint16_t f_to_bf16(float x) {
    __nv_bfloat16 r = __float2bfloat16_rn(x);
    return *reinterpret_cast<uint16_t*>(&r);
}
__device__ __forceinline__ float bf16_to_f(uint16_t x) { return __uint_as_float(uint32_t(x) << 16); }
__device__ __forceinline__ float2 f16x2_to_f2(uint32_t w) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    return __half22float2(h);
}
__device__ __forceinline__ float f16_to_f(uint16_t x) {
    __half h = *reinterpret_cast<__half*>(&x);
    return __half2float(h);
}
__device__ __forceinline__ uint16_t f_to_f16(float x) {
    __half h = __float2half_rn(x);
    return *reinterpret_cast<uint16_t*>(&h);
}
__device__ __forceinline__ float round_f16(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// D += A B for one m16n8k16 tile, bf16 operands, f32 accumulator (warp-wide)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Four int8 codes packed in `w` -> four floats, exactly.  The word is flipped to offset binary, each byte is dropped
// into the low mantissa byte of 2^23 and 2^23 + 128 is subtracted.
__device__ __forceinline__ void s8x4_to_f4(uint32_t w, float& f0, float& f1, float& f2, float& f3) {
    const uint32_t x = w ^ 0x80808080u;
    const float m = 8388736.0f;
    f0 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650)) - m;
    f1 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651)) - m;
    f2 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652)) - m;
    f3 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653)) - m;
}
// same, as two packed pairs (for the f32x2 pipe)
__device__ __forceinline__ void s8x4_to_f2x2(uint32_t w, float2& a, float2& b) {
    const uint32_t x = w ^ 0x80808080u;
    const float2 m = make_float2(-8388736.0f, -8388736.0f);
    a = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650)),
                               __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651))), m);
    b = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652)),
                               __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653))), m);
}

// round-to-nearest-even integer of x * s in [-127, 127] as the low byte of fma(x, s, 1.5 * 2^23)
__device__ __forceinline__ uint32_t rne_code(float x, float s) { return __float_as_uint(__fmaf_rn(x, s, RNE_MAGIC)); }
__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// ---- gates ----
__device__ __forceinline__ float softplus_thr(float x) { return x <= SOFTPLUS_THRESHOLD ? logf(1.0f + expf(x)) : x; }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- warp helpers ----
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// sum over the 8 lanes that share lane >> 3
__device__ __forceinline__ float oct_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}
__device__ __forceinline__ void named_bar(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- global loads that bypass L1 allocation (streamed once) ----
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// ---- mbarriers, bounded waits, bulk copies (shared by the step and the flush kernels) ----
constexpr uint32_t WAIT_LIMIT = 1u << 22;      // bounded spin: ~seconds at worst, then the kernel records a status and leaves
constexpr int ST_PRODUCER_TIMEOUT = 1, ST_CONSUMER_TIMEOUT = 2, ST_PROLOGUE_TIMEOUT = 4, ST_FLUSH_TIMEOUT = 8;

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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// A whole warp waits for the phase with the given parity: lane 0 tests the barrier, the outcome is broadcast, and every
// lane takes the same branch, so the warp stays converged (a lane that spins alone leaves the warp split in two, and every
// later warp-synchronous shuffle then costs a rendezvous of the halves).  Gives up after WAIT_LIMIT polls.
__device__ __forceinline__ bool warp_wait_bounded(uint64_t* bar, uint32_t parity, int lane) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        uint32_t ok = 0;
        if (lane == 0) ok = mbar_try_wait(bar, parity) ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) return true;
    }
    return false;
}
// bulk asynchronous copy global -> this CTA's shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// the same copy with an L2 eviction-priority hint for the lines it reads
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- host-side helpers ----
int device_sm_count();
int ensure_smem(const void* func, size_t bytes);
int check_dims(const lq_dims* d);
// true if any of the (non-null) pointers is not 16-byte aligned: the kernels read and write them with 128-bit accesses
inline bool misaligned16(std::initializer_list<const void*> ptrs) {
    uintptr_t acc = 0;
    for (const void* p : ptrs) acc |= reinterpret_cast<uintptr_t>(p);
    return (acc & 15) != 0;
}
void set_last_cuda_error(cudaError_t e);

// Programmatic dependent launch.  The decode path is a chain of short kernels on one stream (step, flush, step, ...); a
// kernel launched with this attribute may be scheduled while its predecessor is still draining, runs its set-up
// (shared-memory carve, barrier initialisation) and then blocks in pdl_wait() until the predecessor has completed and its
// writes are visible.  Every kernel launched this way calls pdl_trigger() and pdl_wait() before it touches global memory.
static std::atomic<int> g_pdl{1};       // set by lq_set_option from any thread, read by every launch
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_pdl.load(std::memory_order_relaxed) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
inline int finish_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        return LQ_ERR_LAUNCH;
    }
    return LQ_OK;
}

}  // namespace lq
