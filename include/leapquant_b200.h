/*
 * leapquant_b200 -- C ABI of the B200 (sm_100a) kernels for LeapQuant's quantized recurrent-state decode path.
 *
 * Every entry point takes raw DEVICE pointers, plain sizes and the CUDA stream to launch on (a cudaStream_t passed as
 * void*; NULL = the legacy default stream).  Nothing here allocates, frees, synchronises or reads device data on the
 * host, so every call is legal while the stream is being captured into a CUDA graph.  All memory belongs to the caller.
 *
 * The LeapQuant reference has no native interface: its kernels are TileLang programs compiled at run time and called
 * with torch tensors.  Each function below replaces one of those compiled kernels; the comment above it names the
 * reference kernel factory (file:line in the reference tree) whose launch it stands in for, and the argument order
 * follows that kernel's tensor order with the aliasing views of the state tensor collapsed into `ssm` + `SS`.
 *
 * Packed state layout (reference leapquant/state.py:1-6,29-40).  `ssm` points at element [0,0,0,0] of the fp32 state
 * tensor [NS, HV, V, K]; `SS` is its slot stride in floats (inner dims packed).  Inside each (slot, head) region of
 * 4*V*K bytes:   int8 codes [V][K]  |  f32 Sk[K]  |  f32 Sv[V]  |  f16 [R][K+V] = U^T | Q^T   (rest unused).
 * Window buffers (reference leapquant/state.py:61-70): Kbuf bf16 [NS,HV,L,K], Ubuf bf16 [NS,HV,L,V], Wbuf f32 [NS,HV,L],
 * Pbuf f32 [NS,HV,1] (GDN, running decay) or [NS,HV,K] (KDA, cumulative log gate), Gbuf f16 [NS,HV,L,K] (KDA only),
 * hcnt i32 [NS,HV].  Slot indices `idx` are int32; idx <= 0 marks a padding row.
 *
 * Supported shapes: K = V = 128; R in {4, 8}; L a multiple of 4 with 4 <= L <= 64; HV a multiple of H;
 * ssm 16-byte aligned and SS a multiple of 4.  Anything else returns LQ_ERR_UNSUPPORTED / LQ_ERR_ALIGN and launches nothing.
 *
 * Return value: LQ_OK (0) or a negative LQ_ERR_* code.  Errors are argument or launch errors found on the host; the
 * kernels themselves never trap.  lq_strerror() gives a static description.
 */
#ifndef LEAPQUANT_B200_H
#define LEAPQUANT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LQ_OK 0
#define LQ_ERR_NULL (-1)         /* a required pointer is NULL */
#define LQ_ERR_UNSUPPORTED (-2)  /* shape outside the supported set */
#define LQ_ERR_ALIGN (-3)        /* pointer or stride alignment */
#define LQ_ERR_RANGE (-4)        /* a size is negative or inconsistent (e.g. HV % H != 0, N < 0) */
#define LQ_ERR_LAUNCH (-5)       /* the CUDA runtime refused the launch; see lq_last_cuda_error() */
#define LQ_ERR_LIMIT (-6)        /* a call larger than lq_gdn_decode_noalloc takes */

/* Shape of one layer's state, shared by all entry points. */
typedef struct lq_dims {
    int32_t NS;   /* slots in the state tensor (slot 0 is the null slot) */
    int32_t HV;   /* value heads */
    int32_t H;    /* key heads (HV % H == 0) */
    int32_t K;    /* key dim   (128) */
    int32_t V;    /* value dim (128) */
    int32_t L;    /* window length */
    int32_t R;    /* Compensator Tokens per head */
    int64_t SS;   /* slot stride of the state tensor in floats */
} lq_dims;

int lq_version(void);
const char* lq_strerror(int code);
/* cudaError_t value of the most recent LQ_ERR_LAUNCH on this thread (0 if none). */
int lq_last_cuda_error(void);
/* Copies the device-side status word (0 = no kernel gave up a bounded wait) to *status and clears it.  Synchronises
 * the device: debugging / tests only.  No reference counterpart. */
int lq_device_status(int* status);

/* Tuning / debugging switch; no reference counterpart.  The setting is process-wide (it applies to every layer and every
 * later call in the process, not to one call), stored atomically, and read once per launch: it may be set from any
 * thread, but calls already in progress on other threads may still use the previous value.  "step_impl": 0 = persistent CTAs fed by bulk
 * asynchronous copies (default), 1 = one CTA per (row, head) with plain loads and the same arithmetic, 2 = one warp per
 * (row, head) in registers (GDN only; KDA keeps the default).  1 and 2 exist for debugging and comparison.
 * "pdl": 1 (default) launches the step and flush kernels with programmatic stream serialisation, so that the launch and
 * set-up of one overlap the tail of its predecessor on the stream; 0 = plain launches.
 * "work_list_min_programs": the fewest (row, head) programs of a fused decode call for which the `work` list passed to it
 * is used (-1 = default, sixteen per SM; 0 = whenever `work` is given).  The mailboxes cost an atomic round trip or two
 * per launch and save the flush of one head when the due heads sit unevenly on the CTAs. */
int lq_set_option(const char* name, int32_t value);

/* GDN decode step.  Replaces the kernel built by make_gdn_step (reference leapquant/kernels.py:27-692, launch
 * signature :80-89).  One token per row n < N: reads the INT8 checkpoint and the h live window entries of
 * (idx[n], hv), writes o[n,hv,:] (bf16) and appends (k_hat, u, w = 1) to the window; hcnt += 1.
 * mixed bf16 [N, 2*H*K + HV*V] = q | k | v;  a bf16 [N,HV];  b bf16 [N,HV];  A_log f32 [HV];  dt_bias f32 [HV];
 * o bf16 [N,HV,V].  scale <= 0 selects K^-1/2.  A head whose window is already full (hcnt == L) is skipped: o = 0. */
int lq_gdn_step(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                const void* mixed, const void* a, const void* b, const float* A_log, const float* dt_bias,
                const int32_t* idx, void* o, int32_t N, float scale, void* stream);

/* KDA decode step.  Replaces the kernel built by make_kda_step (reference leapquant/kernels.py:694-1075, launch
 * signature :732-741).  As lq_gdn_step with a gate per key channel: a bf16 [N,HV,K], dt_bias f32 [HV,K],
 * Pbuf f32 [NS,HV,K], Gbuf f16 [NS,HV,L,K].  gate_lower_bound != 0 selects the bounded gate
 * g = glb * sigmoid(exp(A_log) (a + dt_bias)); 0 selects g = -exp(A_log) softplus(a + dt_bias). */
int lq_kda_step(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                int32_t* hcnt, const void* mixed, const void* a, const void* b, const float* A_log,
                const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale, float gate_lower_bound,
                void* stream);

/* Window flush.  Replaces the kernel built by make_flush (reference leapquant/kernels.py:1077-2033, launch
 * signature :1139-1148).  For every (idx[n] > 0, hv) with hcnt == L: rebuilds the state from checkpoint + window,
 * extracts R new Compensator Tokens by `iters` rounds of subspace iteration from Q0 (f32 [V,R]) with CholeskyQR2,
 * recomputes Sk / Sv, requantises the residual to INT8 and resets the window.  Due heads are found on the device;
 * the launch shape does not depend on how many are due.  (Row n, head hv) is handled by CTA (n * HV + hv) % grid, which
 * reads that head's counter once: no CTA depends on what another one reads or resets, nor on all CTAs being resident.  kda != 0 selects the per-channel-gate variant (Gbuf used). */
int lq_flush(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
             int32_t* hcnt, const float* Q0, const int32_t* idx, int32_t N, int32_t kda, int32_t iters, void* stream);

/* Fused decode: lq_gdn_step / lq_kda_step followed by lq_flush on the same rows, in ONE launch.  Replaces the two
 * launches of LeapQuantState.decode (reference leapquant/state.py:99-116): the persistent CTA that fills a head's window
 * flushes that head itself after its last program, so the flush needs no due scan, no second launch and finds the
 * head's window rows in cache.  Same arguments as the step plus the flush's Q0 and iters; same results as the two calls.
 * Where the fused form is not available (a debug step driver is selected, or the working set of one flush team does not
 * fit in the shared memory the step pipeline leaves behind) the two kernels are launched one after the other.
 *
 * `work` (optional, may be NULL): device scratch of at least lq_decode_work_bytes(N, HV) bytes (16 KiB), 8-byte aligned, ALL
 * ZERO before the first call that uses it; every call leaves it ready for the next (all zero but for a generation counter).  It holds a small mailbox per CTA: a CTA
 * that filled the windows of two or three heads in this call flushes the first and posts the others; a CTA that filled none
 * takes posted heads over (a serving batch fills the windows of a few rows per step, and the program-to-CTA map puts their
 * heads on the same CTAs now and then); what nobody took, the poster flushes itself, so no CTA ever waits for another.
 * Results do not depend on it.  Calls that use the same `work` must not overlap on the GPU.  Small calls ignore it (see
 * "work_list_min_programs"). */
int lq_gdn_decode(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                  const void* mixed, const void* a, const void* b, const float* A_log, const float* dt_bias,
                  const int32_t* idx, void* o, int32_t N, float scale, const float* Q0, int32_t iters, void* work,
                  int64_t work_bytes, void* stream);
int lq_kda_decode(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                  int32_t* hcnt, const void* mixed, const void* a, const void* b, const float* A_log,
                  const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale, float gate_lower_bound,
                  const float* Q0, int32_t iters, void* work, int64_t work_bytes, void* stream);
/* Bytes of the `work` scratch: 16 KiB (a mailbox per CTA for launches of up to 1 024 CTAs), whatever `rows` and `HV`. */
int64_t lq_decode_work_bytes(int32_t rows, int32_t HV);

/* lq_gdn_decode for callers that cannot allocate device memory.  (No counterpart in the reference: its kernels get every
 * buffer from torch.)  Some hosts of this library must not call cudaMalloc once they are running: a serving engine that
 * has measured free memory and given all of it to its cache pool, so that a later allocation may fail or push it over;
 * a plugin that lives under an allocator it does not own; a latency-bound thread for which the device-wide
 * synchronisation inside cudaMalloc / cudaFree is a stall.  lq_gdn_decode leaves the mailboxes of due heads (`work`) to
 * the caller, which is one more buffer to allocate; this entry point keeps them inside the library instead, in a device
 * array of fixed size that is part of the library image: every GPU that loads the library holds lq_decode_work_bytes()
 * = 16 KiB for it until the process exits, used or not.
 *   - Arguments and results are those of lq_gdn_decode without `work` / `work_bytes`; inputs and outputs are still the
 *     caller's.  It calls no cudaMalloc, cudaFree or other allocating routine.
 *   - Limit: calls of at most LQ_NOALLOC_MAX_HEADS (row, head) pairs, min(N, NS) * HV, and GPUs of at most 1 024 SMs (one
 *     mailbox per CTA); a larger call returns LQ_ERR_LIMIT and nothing is launched.
 *   - The first call on a device asks the runtime for the array's address on that device (cudaGetSymbolAddress, with the
 *     caller's current device): make that first call outside any stream capture.
 *   - Every call on a device shares the one array.  The call zeroes the part it uses (a memset on `stream` ahead of the
 *     kernel), so a call that was cut short leaves nothing behind; two calls that overlap on the GPU (different streams,
 *     or different threads without ordering) race on it and must not be made. */
#define LQ_NOALLOC_MAX_HEADS 65536
int lq_gdn_decode_noalloc(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                          const void* mixed, const void* a, const void* b, const float* A_log, const float* dt_bias,
                          const int32_t* idx, void* o, int32_t N, float scale, const float* Q0, int32_t iters, void* stream);

/* Operands of the causal conv1d update that precedes every decode step in the serving engine (the reference plugin calls
 * vLLM's causal_conv1d_update right before LeapQuantState.decode: reference leapquant/vllm/gdn.py:31-33, glm.py:72-73).
 * Per row with slot = idx[n] > 0 and per channel c of the q | k | v projection:
 *     window = (state[slot][c][0], state[slot][c][1], state[slot][c][2], x[n][c])
 *     y      = bias[c] + sum_t bf16(weight[c][t] * window[t])      (fp32 sum, taps in order: the engine kernel's arithmetic)
 *     out    = bf16(y / (1 + exp(-y)))                             (SiLU)
 *     state[slot][c][:] <- (window[1], window[2], window[3])
 * All tensors are bf16.  The state is addressed through three element strides, so both layouts of the engine's cache work:
 * (slot, channel, tap) and (slot, tap, channel); the second one (stride_dim == 1) is read with 8-byte accesses and then
 * needs stride_tap and stride_slot to be multiples of 4.  width must be 4. */
typedef struct lq_conv1d {
    const void* x;          /* bf16 [N, x_stride]: raw projections of the N rows; channels 0 .. 2*H*K + HV*V - 1 are used */
    int64_t x_stride;       /* elements between rows: >= the channel count, a multiple of 8; x 16-byte aligned */
    void* state;            /* bf16 conv state, element (slot, channel, tap) at slot*stride_slot + channel*stride_dim + tap*stride_tap */
    int64_t stride_slot, stride_dim, stride_tap;
    const void* weight;     /* bf16 [channels, width] contiguous (a depthwise conv1d weight [channels, 1, width] viewed 2-D) */
    const void* bias;       /* bf16 [channels] or NULL */
    int32_t width;          /* taps: 4 (the state keeps width - 1 = 3 past inputs) */
} lq_conv1d;

/* Fused conv1d update + decode: lq_gdn_decode / lq_kda_decode with the q | k | v row computed inside the kernel from the raw
 * projections (see lq_conv1d) instead of read from `mixed`; the conv state of every row with idx[n] > 0 is advanced.  Replaces
 * the pair causal_conv1d_update -> LeapQuantState.decode of the reference plugin (leapquant/vllm/gdn.py:25-36,
 * leapquant/vllm/glm.py:71-75) by ONE launch that never writes the intermediate q | k | v row to memory.  Results equal
 * lq_causal_conv1d_update followed by lq_*_decode bit for bit.  Only the fused single-launch form exists: a configuration
 * whose flush work area does not fit beside the step pipeline returns LQ_ERR_UNSUPPORTED.  When to use it: the conv
 * arithmetic of the single launch runs on the warps that feed the step pipeline, and replayed from a CUDA graph the two
 * calls lq_causal_conv1d_update + lq_*_decode are the faster form (86 against 96 microseconds per step at 256 rows of 32
 * heads on a B200); the single launch saves a launch where launches are issued one by one from the host. */
int lq_gdn_decode_conv(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, int32_t* hcnt,
                       const lq_conv1d* conv, const void* a, const void* b, const float* A_log, const float* dt_bias,
                       const int32_t* idx, void* o, int32_t N, float scale, const float* Q0, int32_t iters, void* work,
                       int64_t work_bytes, void* stream);
int lq_kda_decode_conv(const lq_dims* d, void* ssm, void* Kbuf, void* Ubuf, float* Wbuf, float* Pbuf, void* Gbuf,
                       int32_t* hcnt, const lq_conv1d* conv, const void* a, const void* b, const float* A_log,
                       const float* dt_bias, const int32_t* idx, void* o, int32_t N, float scale, float gate_lower_bound,
                       const float* Q0, int32_t iters, void* work, int64_t work_bytes, void* stream);

/* The conv1d update alone (same arithmetic as inside the fused kernels): out bf16 [N, out_stride] receives the activated
 * q | k | v rows, the state is advanced.  Stands in for vLLM's causal_conv1d_update on single-token rows (call sites
 * reference leapquant/vllm/gdn.py:32, glm.py:72).  Rows with idx[n] <= 0 are skipped (nothing read or written).  `channels`
 * must be a multiple of 8; NS is the number of slots of the state. */
int lq_causal_conv1d_update(const lq_conv1d* conv, const int32_t* idx, int32_t N, int32_t channels, int32_t NS, void* out,
                            int64_t out_stride, void* stream);

/* Standalone quantize.  Replaces the kernel built by make_quantize (reference leapquant/kernels.py:2126-2242);
 * with kda != 0 it also stands in for LeapQuantState._kda_checkpoint (reference leapquant/state.py:130-142, which
 * calls lowrank_factor with 3 iterations).  For every idx[n] > 0 and every head: reads the fp32 state [V][K] that
 * fills the slot and writes the 8-bit checkpoint over it; resets the window (Wbuf = 0, hcnt = 0, Pbuf = 1 for GDN;
 * Pbuf = 0 and Gbuf = 1 for KDA).  Orthogonalisation is modified Gram-Schmidt, as in the reference kernel. */
int lq_quantize(const lq_dims* d, void* ssm, float* Wbuf, float* Pbuf, void* Gbuf, int32_t* hcnt, const float* Q0,
                const int32_t* idx, int32_t N, int32_t kda, int32_t iters, void* stream);

/* Dequantize in place.  Replaces the kernel built by make_dequant (reference leapquant/kernels.py:2041-2123, GDN
 * branch); with kda != 0 it stands in for LeapQuantState._kda_rebuild (reference leapquant/state.py:118-128).
 * For every idx[n] > 0 and every head: fp32 state = decay * (deq + Q U^T) + live window entries, written over the
 * slot.  GDN then resets the window (Wbuf = 0, Pbuf = 1, hcnt = 0); KDA leaves the window buffers untouched, as the
 * reference does (its quantize after the prefill resets them). */
int lq_dequant(const lq_dims* d, void* ssm, const void* Kbuf, const void* Ubuf, float* Wbuf, float* Pbuf,
               const void* Gbuf, int32_t* hcnt, const int32_t* idx, int32_t N, int32_t kda, void* stream);

/* Rank-r factors of x f32 [n, K, V] (contiguous): `iters` rounds of P = x Q -> MGS, Q = x^T P -> MGS from Q0
 * f32 [V, r]; U = x Q f32 [n, K, r], Q f32 [n, V, r].  Replaces the kernel built by make_lowrank (reference
 * leapquant/kernels.py:2246-2314) as called by lowrank_factor (:2321-2331). */
int lq_lowrank(const float* x, const float* Q0, float* U, float* Q, int32_t n, int32_t K, int32_t V, int32_t r,
               int32_t iters, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LEAPQUANT_B200_H */
