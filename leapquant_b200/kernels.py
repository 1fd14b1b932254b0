"""Kernel factories of the 8-bit recurrent state, with the names and call signatures of the reference's
leapquant/kernels.py, backed by hand-written sm_100a CUDA behind a C ABI (include/leapquant_b200.h).

  make_gdn_step    GDN decode step            (reference leapquant/kernels.py:28,   launch signature :80-89)
  make_kda_step    KDA decode step            (reference leapquant/kernels.py:695,  launch signature :732-741)
  make_flush       end-of-window flush        (reference leapquant/kernels.py:1078, launch signature :1139-1148)
  make_dequant     8-bit -> fp32 in place     (reference leapquant/kernels.py:2042, launch signature :2053-2062)
  make_quantize    fp32 -> 8-bit in place     (reference leapquant/kernels.py:2127, launch signature :2136-2142)
  make_lowrank / lowrank_factor               (reference leapquant/kernels.py:2247, :2321)

Each factory returns a callable that takes the same tensors in the same order as the reference's compiled kernel.
The several aliasing views of the state tensor the reference passes (Sq, Sk, Sv, Skv, UQ, Sq16) all point into one
fp32 tensor; the callable takes the base address from the first of them and the slot stride SS from the factory.
The reference's tuning keywords (SMS, NSTAGE, NSTAGEQ, NCG, NNW, MAXIT, NMAX, NTP, RSG, PAD, MMT, BV, threads) are
accepted and ignored: scheduling is decided inside the library.  Shapes outside K = V = 128 raise NotImplementedError.
"""
import functools

import torch

from . import _lib

F32, BF16, I32, I8 = "float32", "bfloat16", "int32", "int8"
QMAX = 127.0
SOFTPLUS_THRESHOLD = 20.0
EPS = 1e-12
STEP_CFG = {(128, 128): (6, 3, 2), (64, 128): (10, 5, 5), (64, 64): (8, 4, 4)}


def _need_128(K, V, who):
    if (K, V) != (128, 128):
        raise NotImplementedError(f"{who}: (K, V) = ({K}, {V}); this build implements 128 x 128 heads only")


def _launch(fn, what, dev_tensor, *args):
    with _lib.on_device(dev_tensor):
        _lib.check(fn(*args, _lib.stream_of(dev_tensor)), what)


def _work(work):
    """(pointer, bytes) of the optional mailbox scratch of the fused decode (an int32 tensor, zeroed once), or (None, 0)."""
    if work is None:
        return None, 0
    return _lib.ptr(work), work.numel() * work.element_size()


def decode_work_ints(rows, HV):
    """int32 elements of the `work` tensor of the fused decode (mailboxes of due heads: a fixed 16 KiB, whatever the call)."""
    return int(_lib.lib().lq_decode_work_bytes(int(rows), int(HV))) // 4


def make_gdn_step(NS, HV, H, K, V, L, SS, R=4, SMS=148, NSTAGE=None, NCG=None, NNW=None, scale=None, MAXIT=256):
    """Gated DeltaNet decode step on the 8-bit state.  Returns
    step(Sq, Sk, Sv, Skv, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, mixed, a, b, A_log, dt_bias, UQ, idx, o)."""
    _need_128(K, V, "make_gdn_step")
    d = _lib.dims(NS, HV, H, K, V, L, R, SS)
    sc = float(K ** -0.5 if scale is None else scale)
    fn = _lib.lib().lq_gdn_step
    p = _lib.ptr

    def step(Sq, Sk, Sv, Skv, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, mixed, a, b, A_log, dt_bias, UQ, idx, o):
        _launch(fn, "lq_gdn_step", Sq, d, p(Sq), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(hcnt), p(mixed), p(a), p(b),
                p(A_log), p(dt_bias), p(idx), p(o), int(mixed.shape[0]), sc)

    return step


def make_kda_step(NS, HV, H, K, V, L, SS, R=4, SMS=148, NSTAGE=6, NSTAGEQ=4, NCG=2, NNW=2, scale=128 ** -0.5, MAXIT=256,
                  GLB=0.0):
    """Kimi Delta Attention decode step (gate per key channel).  GLB != 0 selects the bounded gate.  Returns
    step(Sq, Sk, Sv, Skv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, UQ, idx, o)."""
    _need_128(K, V, "make_kda_step")
    d = _lib.dims(NS, HV, H, K, V, L, R, SS)
    sc, glb = float(scale), float(GLB)
    fn = _lib.lib().lq_kda_step
    p = _lib.ptr

    def step(Sq, Sk, Sv, Skv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, UQ, idx, o):
        _launch(fn, "lq_kda_step", Sq, d, p(Sq), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(Gbuf), p(hcnt), p(mixed), p(a),
                p(b), p(A_log), p(dt_bias), p(idx), p(o), int(mixed.shape[0]), sc, glb)

    return step


def make_decode(NS, HV, H, K, V, L, SS, R=4, ITERS=1, KDA=False, GLB=0.0, scale=None):
    """Step and flush in one launch (no counterpart factory in the reference, whose LeapQuantState.decode launches the two
    kernels one after the other, leapquant/state.py:99-116).  Returns, for GDN,
    decode(Sq, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, mixed, a, b, A_log, dt_bias, Q0, idx, o) and for KDA the same with Gbuf
    after Pbuf; results equal those of the step followed by the flush."""
    _need_128(K, V, "make_decode")
    d = _lib.dims(NS, HV, H, K, V, L, R, SS)
    sc = float(K ** -0.5 if scale is None else scale)
    iters, glb = int(ITERS), float(GLB)
    p = _lib.ptr
    if KDA:
        fn = _lib.lib().lq_kda_decode

        def decode(Sq, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, Q0, idx, o, work=None):
            _launch(fn, "lq_kda_decode", Sq, d, p(Sq), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(Gbuf), p(hcnt), p(mixed), p(a), p(b),
                    p(A_log), p(dt_bias), p(idx), p(o), int(mixed.shape[0]), sc, glb, p(Q0), iters, *_work(work))
    else:
        fn = _lib.lib().lq_gdn_decode

        def decode(Sq, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, mixed, a, b, A_log, dt_bias, Q0, idx, o, work=None):
            _launch(fn, "lq_gdn_decode", Sq, d, p(Sq), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(hcnt), p(mixed), p(a), p(b),
                    p(A_log), p(dt_bias), p(idx), p(o), int(mixed.shape[0]), sc, p(Q0), iters, *_work(work))

    return decode


def make_decode_conv(NS, HV, H, K, V, L, SS, R=4, ITERS=1, KDA=False, GLB=0.0, scale=None):
    """causal conv1d update + step + flush in one launch (no counterpart factory in the reference, whose plugin calls vLLM's
    causal_conv1d_update and then LeapQuantState.decode: leapquant/vllm/gdn.py:31-36, leapquant/vllm/glm.py:71-75).  Returns, for
    GDN, decode(Sq, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, x, conv_state, conv_weight, conv_bias, a, b, A_log, dt_bias, Q0, idx, o) and
    for KDA the same with Gbuf after Pbuf.  x holds the raw q | k | v projections (bf16 [N, >= 2HK + HV V]); conv_state is the
    engine's conv cache viewed (slot, channel, width - 1) and is advanced in place; results equal make_conv1d_update followed by
    make_decode bit for bit."""
    _need_128(K, V, "make_decode_conv")
    d = _lib.dims(NS, HV, H, K, V, L, R, SS)
    sc = float(K ** -0.5 if scale is None else scale)
    iters, glb = int(ITERS), float(GLB)
    p = _lib.ptr
    if KDA:
        fn = _lib.lib().lq_kda_decode_conv

        def decode(Sq, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, x, conv_state, conv_weight, conv_bias, a, b, A_log, dt_bias, Q0, idx, o,
                   work=None):
            cv = _lib.conv1d(x, conv_state, conv_weight, conv_bias)
            _launch(fn, "lq_kda_decode_conv", Sq, d, p(Sq), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(Gbuf), p(hcnt), cv, p(a), p(b),
                    p(A_log), p(dt_bias), p(idx), p(o), int(x.shape[0]), sc, glb, p(Q0), iters, *_work(work))
    else:
        fn = _lib.lib().lq_gdn_decode_conv

        def decode(Sq, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, x, conv_state, conv_weight, conv_bias, a, b, A_log, dt_bias, Q0, idx, o, work=None):
            cv = _lib.conv1d(x, conv_state, conv_weight, conv_bias)
            _launch(fn, "lq_gdn_decode_conv", Sq, d, p(Sq), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(hcnt), cv, p(a), p(b),
                    p(A_log), p(dt_bias), p(idx), p(o), int(x.shape[0]), sc, p(Q0), iters, *_work(work))

    return decode


def make_conv1d_update(NS, channels):
    """The causal conv1d update alone, with the arithmetic of the fused kernels.  Returns
    update(x, conv_state, conv_weight, conv_bias, idx, out): out bf16 [N, channels] receives the activated rows, conv_state
    (slot, channel, width - 1) is advanced; rows with idx <= 0 are skipped.  Stands in for vLLM's causal_conv1d_update on
    single-token rows (call sites reference leapquant/vllm/gdn.py:32, leapquant/vllm/glm.py:72)."""
    fn = _lib.lib().lq_causal_conv1d_update
    p = _lib.ptr

    def update(x, conv_state, conv_weight, conv_bias, idx, out):
        cv = _lib.conv1d(x, conv_state, conv_weight, conv_bias)
        _launch(fn, "lq_causal_conv1d_update", x, cv, p(idx), int(x.shape[0]), int(channels), int(NS), p(out), out.stride(0))

    return update


def make_flush(NS, HV, K, V, L, SS, R=4, ITERS=1, SMS=148, NCG=3, MAXIT=128, PAD=8, KDA=False, MMT="bf16", PNMIN=1e-20,
               NMAX=0, NTP=0, RSG=None):
    """End-of-window flush of every head of the rows idx whose window is full.  Returns
    flush(Sq, Sk, Sv, Skv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Sq16, UQ, Q0, idx)."""
    _need_128(K, V, "make_flush")
    d = _lib.dims(NS, HV, HV, K, V, L, R, SS)
    kda, iters = int(bool(KDA)), int(ITERS)
    fn = _lib.lib().lq_flush
    p = _lib.ptr

    def flush(Sq, Sk, Sv, Skv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, Sq16, UQ, Q0, idx):
        _launch(fn, "lq_flush", Sq, d, p(Sq), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(Gbuf) if kda else None, p(hcnt),
                p(Q0), p(idx), int(idx.shape[0]), kda, iters)

    return flush


def make_dequant(NS, HV, K, V, L, SS, BV=32, threads=128, kda=False, buf_dtype=F32, R=0):
    """fp32 S[slot] <- decay * deq(checkpoint) + live window entries, in place, for the listed slots.  Returns
    dequant(S0, Sq, Sk, Sv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, UQ, idx).  Window buffers must be bf16 (buf_dtype=BF16).
    kda=True rebuilds a KDA state (per-channel decay, Gbuf holding fp16 step factors) and leaves the window untouched."""
    _need_128(K, V, "make_dequant")
    if buf_dtype != BF16:
        raise NotImplementedError("make_dequant: the window buffers are bf16 in this build (buf_dtype=BF16)")
    if R not in (4, 8):
        raise NotImplementedError(f"make_dequant: R = {R}; supported 4 and 8")
    d = _lib.dims(NS, HV, HV, K, V, L, R, SS)
    kd = int(bool(kda))
    fn = _lib.lib().lq_dequant
    p = _lib.ptr

    def dequant(S0, Sq, Sk, Sv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, UQ, idx):
        _launch(fn, "lq_dequant", S0, d, p(S0), p(Kbuf), p(Ubuf), p(Wbuf), p(Pbuf), p(Gbuf) if kd else None, p(hcnt),
                p(idx), int(idx.shape[0]), kd)

    return dequant


def make_quantize(NS, HV, K, V, L, SS, R=4, ITERS=1, threads=128, kda=False):
    """8-bit checkpoint of the fp32 states in the listed slots, then window reset.  Returns
    quantize(S0, Sq, Sk, Sv, UQ, Wbuf, Pbuf, hcnt, Q0, idx[, Gbuf]).  kda=True (not in the reference's factory) resets a KDA
    window instead (Pbuf = 0, Gbuf = 1) and needs Gbuf as the last argument."""
    _need_128(K, V, "make_quantize")
    d = _lib.dims(NS, HV, HV, K, V, L, R, SS)
    kd, iters = int(bool(kda)), int(ITERS)
    fn = _lib.lib().lq_quantize
    p = _lib.ptr

    def quantize(S0, Sq, Sk, Sv, UQ, Wbuf, Pbuf, hcnt, Q0, idx, Gbuf=None):
        _launch(fn, "lq_quantize", S0, d, p(S0), p(Wbuf), p(Pbuf), p(Gbuf) if kd else None, p(hcnt), p(Q0), p(idx),
                int(idx.shape[0]), kd, iters)

    return quantize


def make_lowrank(K, V, R, ITERS, threads=128):
    """Rank-R subspace iteration with modified Gram-Schmidt.  Returns lowrank(S [N,K,V] f32, Q0 [V,R], U [N,K,R], Q [N,V,R])."""
    _need_128(K, V, "make_lowrank")
    fn = _lib.lib().lq_lowrank
    p = _lib.ptr
    iters = int(ITERS)

    def lowrank(S, Q0, U, Q):
        _launch(fn, "lq_lowrank", S, p(S), p(Q0), p(U), p(Q), int(S.shape[0]), K, V, R, iters)

    return lowrank


_mk_lowrank = functools.lru_cache(maxsize=None)(make_lowrank)
_Q0_LR = {}


def lowrank_factor(x, r, iters=3):
    """x: [..., K, V] fp32 CUDA -> U [..., K, r], Q [..., V, r] (one fused kernel)."""
    *lead, K, V = x.shape
    key = (str(x.device), V, r)
    if key not in _Q0_LR:
        _Q0_LR[key] = torch.randn(V, r, generator=torch.Generator().manual_seed(0)).to(x.device)
    xf = x.reshape(-1, K, V).contiguous().float()
    U = torch.empty(xf.shape[0], K, r, device=x.device, dtype=torch.float32)
    Q = torch.empty(xf.shape[0], V, r, device=x.device, dtype=torch.float32)
    _mk_lowrank(K, V, r, iters)(xf, _Q0_LR[key], U, Q)
    return U.reshape(*lead, K, r), Q.reshape(*lead, V, r)
