// Host-side utilities shared by the C-ABI entry points: argument checks, error strings, per-device caches.
#include <mutex>

#include "lq_common.cuh"

namespace lq {

static thread_local int tl_last_cuda_error = 0;
void set_last_cuda_error(cudaError_t e) { tl_last_cuda_error = int(e); }

int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Raises a kernel's dynamic shared-memory limit once per (device, kernel); later calls are a table lookup.
int ensure_smem(const void* func, size_t bytes) {
    struct Entry { int dev; const void* f; size_t bytes; };
    static Entry table[256];
    static int used = 0;
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
        if (table[i].dev == dev && table[i].f == func) {
            if (table[i].bytes >= bytes) return LQ_OK;
            cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
            if (e != cudaSuccess) { set_last_cuda_error(e); return LQ_ERR_LAUNCH; }
            table[i].bytes = bytes;
            return LQ_OK;
        }
    cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
    if (e != cudaSuccess) { set_last_cuda_error(e); return LQ_ERR_LAUNCH; }
    if (used < 256) table[used++] = Entry{dev, func, bytes};
    return LQ_OK;
}

int check_dims(const lq_dims* d) {
    if (!d) return LQ_ERR_NULL;
    if (d->K != KD || d->V != VD) return LQ_ERR_UNSUPPORTED;
    if (d->R != 4 && d->R != 8) return LQ_ERR_UNSUPPORTED;
    if (d->L < 4 || d->L > 64 || (d->L & 3)) return LQ_ERR_UNSUPPORTED;
    if (d->NS < 1 || d->HV < 1 || d->H < 1 || d->HV % d->H != 0) return LQ_ERR_RANGE;
    if (d->SS < int64_t(d->HV) * d->V * d->K) return LQ_ERR_RANGE;
    if (d->SS & 3) return LQ_ERR_ALIGN;
    return LQ_OK;
}

}  // namespace lq

extern "C" int lq_version(void) { return 100; }

extern "C" const char* lq_strerror(int code) {
    switch (code) {
        case LQ_OK: return "ok";
        case LQ_ERR_NULL: return "a required pointer is NULL";
        case LQ_ERR_UNSUPPORTED: return "unsupported shape (need K = V = 128, R in {4, 8}, L % 4 == 0, 4 <= L <= 64)";
        case LQ_ERR_ALIGN: return "state tensor must be 16-byte aligned with a slot stride that is a multiple of 4 floats";
        case LQ_ERR_RANGE: return "a size argument is negative or inconsistent";
        case LQ_ERR_LAUNCH: return "CUDA launch failed (see lq_last_cuda_error)";
        case LQ_ERR_LIMIT: return "more (row, head) pairs than one call of lq_gdn_decode_noalloc takes (LQ_NOALLOC_MAX_HEADS)";
        default: return "unknown leapquant_b200 error code";
    }
}

extern "C" int lq_last_cuda_error(void) { return lq::tl_last_cuda_error; }

extern "C" int lq_device_status(int* status) {
    if (!status) return LQ_ERR_NULL;
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, lq::g_status, sizeof(int));
    if (e != cudaSuccess) { lq::set_last_cuda_error(e); return LQ_ERR_LAUNCH; }
    int zero = 0;
    e = cudaMemcpyToSymbol(lq::g_status, &zero, sizeof(int));
    if (e != cudaSuccess) { lq::set_last_cuda_error(e); return LQ_ERR_LAUNCH; }
    *status = v;
    return LQ_OK;
}
