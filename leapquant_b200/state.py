"""Per-layer quantized recurrent state: the 8-bit checkpoint lives inside the engine's fp32 state slot, the window
buffers next to it.  Same names, constructor and methods as the reference's leapquant/state.py, so the plugin layer
and any caller of `get_state(...).decode / .dequantize / .quantize` work unchanged.

Packed layout of one (slot, value head) inside the fp32 [V, K] slot (reference leapquant/state.py:1-6):

    int8 codes [V][K] | f32 Sk[K] | f32 Sv[V] | f16 [R][K+V] = U^T | Q^T | (unused)

What differs from the reference, by design:
  * kernels are prebuilt CUDA behind a C ABI: construction compiles nothing and needs no device query;
  * L up to 64 and R in {4, 8} are supported for both GDN and KDA;
  * the KDA prefill round trip (`dequantize` / `quantize` with kda=True) runs as CUDA kernels with the arithmetic of the
    reference's torch code (leapquant/state.py:118-142) instead of a chain of torch ops.
"""
import torch

from . import kernels as KN

WINDOW = 16          # tokens per window (L), reference leapquant/state.py:16
RANK = 4             # Compensator Tokens per head (R), reference leapquant/state.py:17


def _ident(t):
    """Identity of a state tensor: same storage and same view means same layer state (reference leapquant/state.py:20-22)."""
    return (t.untyped_storage().data_ptr(), t.storage_offset(), tuple(t.shape), tuple(t.stride()))


def _alias(ssm, dtype, shape, stride, offset):
    v = torch.empty(0, dtype=dtype, device=ssm.device)
    return v.set_(ssm.untyped_storage()).as_strided(shape, stride, offset)


def state_views(ssm, R):
    """Views of the packed checkpoint aliasing the fp32 state tensor [NS, HV, V, K]; no allocation, works on any device.

    Keys, dtypes, shapes and strides are those of the reference (leapquant/state.py:29-40): Sq int8, q32 int32, sq16 int16
    over the codes; Sk, Sv, skv float32 over the scales; uq float16 over the factors."""
    NS, HV, V, K = ssm.shape
    SS, HS = ssm.stride(0), V * K                       # slot / head strides in floats
    f0 = ssm.storage_offset()                           # first float of the tensor inside its storage
    fs = f0 + HS // 4                                   # scales start after V*K code bytes
    hu = 2 * (fs + K + V)                               # factors start (in halves) after the K + V scales
    return {
        "Sq": _alias(ssm, torch.int8, (NS, HV, V, K), (4 * SS, 4 * HS, K, 1), 4 * f0),
        "q32": _alias(ssm, torch.int32, (NS, HV, V, K // 4), (SS, HS, K // 4, 1), f0),
        "sq16": _alias(ssm, torch.int16, (NS, HV, V, K // 2), (2 * SS, 2 * HS, K // 2, 1), 2 * f0),
        "Sk": _alias(ssm, torch.float32, (NS, HV, K), (SS, HS, 1), fs),
        "Sv": _alias(ssm, torch.float32, (NS, HV, V), (SS, HS, 1), fs + K),
        "skv": _alias(ssm, torch.float32, (NS, HV, K + V), (SS, HS, 1), fs),
        "uq": _alias(ssm, torch.float16, (NS, HV, R, K + V), (2 * SS, 2 * HS, K + V, 1), hu),
    }


class LeapQuantState:
    """Window buffers + kernel handles of one linear-attention layer (reference leapquant/state.py:43-165).

    kda=False: Gated DeltaNet.  kda=True: Kimi Delta Attention; gate_lower_bound != 0 selects the bounded gate.
    nmax is accepted for signature compatibility (the flush sizes its work list from the call's row count)."""

    def __init__(self, ssm, H, kda=False, gate_lower_bound=0.0, nmax=0, L=WINDOW, R=RANK):
        if not ssm.is_cuda:
            raise RuntimeError("LeapQuantState needs the state tensor on a CUDA device (no CPU path exists)")
        assert ssm.dtype == torch.float32, f"LeapQuant needs the fp32 recurrent state cache, got {ssm.dtype}"
        NS, HV, V, K = ssm.shape
        SS = ssm.stride(0)
        assert ssm.stride()[1:] == (V * K, K, 1), f"state inner dims must be packed, got strides {ssm.stride()}"
        assert V * K // 4 + K + V + R * (K + V) // 2 <= V * K, "checkpoint must fit inside the fp32 slot"
        dev = ssm.device
        self.key = _ident(ssm)
        self.gen = 0
        self.kda, self.NS, self.HV, self.H, self.K, self.V, self.L, self.R = bool(kda), NS, HV, H, K, V, L, R
        KA = K if kda else 1

        # initial values as in reference leapquant/state.py:61-70
        self.Kbuf = torch.zeros(NS, HV, L, K, device=dev, dtype=torch.bfloat16)
        self.Ubuf = torch.zeros(NS, HV, L, V, device=dev, dtype=torch.bfloat16)
        self.Wbuf = torch.zeros(NS, HV, L, device=dev)
        self.Pbuf = torch.zeros(NS, HV, KA, device=dev) if kda else torch.ones(NS, HV, 1, device=dev)
        self.Gbuf = (torch.ones(NS, HV, L, KA, device=dev, dtype=torch.float16) if kda
                     else torch.zeros(NS, HV, L, 1, device=dev))
        self.Gd = torch.zeros(1, 1, 1, 1, dtype=torch.bfloat16, device=dev)
        self.hcnt = torch.zeros(NS, HV, dtype=torch.int32, device=dev)
        self.Q0 = torch.randn(V, R, generator=torch.Generator().manual_seed(0)).to(dev)

        if kda:
            self.kstep = KN.make_kda_step(NS, HV, H, K, V, L, SS, R=R, GLB=float(gate_lower_bound))
        else:
            self.kstep = KN.make_gdn_step(NS, HV, H, K, V, L, SS, R=R)
        self.kflush = KN.make_flush(NS, HV, K, V, L, SS, R=R, ITERS=1, KDA=kda, NMAX=nmax)
        self.kdecode = KN.make_decode(NS, HV, H, K, V, L, SS, R=R, ITERS=1, KDA=kda, GLB=float(gate_lower_bound),
                                      scale=(128 ** -0.5 if kda else None))
        self.kdecode_conv = KN.make_decode_conv(NS, HV, H, K, V, L, SS, R=R, ITERS=1, KDA=kda, GLB=float(gate_lower_bound),
                                                scale=(128 ** -0.5 if kda else None))
        self.fused = True                                     # decode() = one fused launch; False = step then flush
        # decode_conv(): False = the conv1d update kernel, then decode (two launches); True = the update inside the decode
        # launch.  Replayed from a CUDA graph the two launches are the faster form at every batch size measured (the conv
        # arithmetic of the single launch sits on the warps that feed its pipeline); the single launch saves a launch where
        # launches are issued one by one from the host.
        self.conv_one_launch = False
        self._kconv = None
        self._mixed = None
        # mailboxes for the heads whose window fills in a call (zeroed once, here): let a CTA without such a head take over a
        # head of a CTA that has several.  No counterpart in the reference.
        self.work = torch.zeros(KN.decode_work_ints(NS, HV), dtype=torch.int32, device=dev)
        self.kdeq = KN.make_dequant(NS, HV, K, V, L, SS, buf_dtype=KN.BF16, R=R, kda=kda)
        self.kquant = KN.make_quantize(NS, HV, K, V, L, SS, R=R, ITERS=3 if kda else 1, kda=kda)
        self._vkey = None
        self._v = None
        self._f32 = {}

    def _p32(self, t):
        """fp32 copy of a layer parameter, cached per tensor (several layers can share one state tensor)."""
        c = self._f32.get(t.data_ptr())
        if c is None:
            c = self._f32[t.data_ptr()] = t.detach().to(torch.float32).contiguous()
        return c

    def views(self, ssm):
        k = _ident(ssm)
        if self._vkey != k:
            self._vkey, self._v = k, state_views(ssm, self.R)
        return self._v

    def decode(self, ssm, mixed, a, b, A_log, dt_bias, idx, out):
        """One decode token per row: step kernel, then the flush of every head whose window just filled.

        mixed bf16 [N, 2HK + HV*V]; a: GDN (N, HV) | KDA (N, HV, K) raw gate; b (N, HV); dt_bias: GDN (HV,) | KDA (HV*K,);
        idx int (N,); out bf16 (N, HV, V) written in place.  No host synchronisation, no allocation when the dtypes match."""
        A_log = A_log if A_log.dtype == torch.float32 else self._p32(A_log)
        dt_bias = dt_bias if dt_bias.dtype == torch.float32 else self._p32(dt_bias)
        KA = self.K if self.kda else 1
        a = a.reshape(a.shape[0], self.HV, KA).contiguous()
        dt_bias = dt_bias.reshape(self.HV, KA).contiguous()
        idx = idx if idx.dtype == torch.int32 else idx.to(torch.int32)
        v = self.views(ssm)
        if self.fused:
            if self.kda:
                self.kdecode(v["q32"], self.Kbuf, self.Ubuf, self.Wbuf, self.Pbuf, self.Gbuf, self.hcnt, mixed, a, b, A_log,
                             dt_bias, self.Q0, idx, out, self.work)
            else:
                self.kdecode(v["q32"], self.Kbuf, self.Ubuf, self.Wbuf, self.Pbuf, self.hcnt, mixed, a, b, A_log, dt_bias,
                             self.Q0, idx, out, self.work)
            return
        if self.kda:
            self.kstep(v["q32"], v["Sk"], v["Sv"], v["skv"], self.Kbuf, self.Ubuf, self.Wbuf, self.Pbuf, self.Gbuf,
                       self.hcnt, mixed, a, b, A_log, dt_bias, v["uq"], idx, out)
            G = self.Gbuf
        else:
            self.kstep(v["q32"], v["Sk"], v["Sv"], v["skv"], self.Kbuf, self.Ubuf, self.Wbuf, self.Pbuf, self.hcnt,
                       mixed, a, b, A_log, dt_bias, v["uq"], idx, out)
            G = self.Gd
        self.kflush(v["q32"], v["Sk"], v["Sv"], v["skv"], self.Kbuf, self.Ubuf, self.Wbuf, self.Pbuf, G, self.hcnt,
                    v["sq16"], v["uq"], self.Q0, idx)

    def decode_conv(self, ssm, x, conv_state, conv_weight, conv_bias, a, b, A_log, dt_bias, idx, out):
        """The causal conv1d update of the step and decode(): x bf16 [N, >= 2HK + HV*V] holds the RAW q | k | v projections,
        conv_state is the engine's conv cache viewed (slot, channel, width - 1) (any strides; advanced in place), conv_weight
        bf16 [channels, 4], conv_bias bf16 [channels] or None.  Two launches of this library (update kernel, decode), or, with
        conv_one_launch, one, in which the activated q | k | v row is never written to memory; the results are the same bit for
        bit.  No counterpart in the reference, whose plugin calls vLLM's causal_conv1d_update first."""
        if not self.conv_one_launch:
            C = 2 * self.H * self.K + self.HV * self.V
            N = x.shape[0]
            if self._kconv is None:
                self._kconv = KN.make_conv1d_update(self.NS, C)
            if self._mixed is None or self._mixed.shape[0] < N:
                self._mixed = torch.empty(max(N, 64), C, dtype=torch.bfloat16, device=x.device)
            mixed = self._mixed[:N]
            i32 = idx if idx.dtype == torch.int32 else idx.to(torch.int32)
            self._kconv(x, conv_state, conv_weight, conv_bias, i32, mixed)
            return self.decode(ssm, mixed, a, b, A_log, dt_bias, i32, out)
        A_log = A_log if A_log.dtype == torch.float32 else self._p32(A_log)
        dt_bias = dt_bias if dt_bias.dtype == torch.float32 else self._p32(dt_bias)
        KA = self.K if self.kda else 1
        a = a.reshape(a.shape[0], self.HV, KA).contiguous()
        dt_bias = dt_bias.reshape(self.HV, KA).contiguous()
        idx = idx if idx.dtype == torch.int32 else idx.to(torch.int32)
        v = self.views(ssm)
        bufs = (self.Kbuf, self.Ubuf, self.Wbuf, self.Pbuf) + ((self.Gbuf,) if self.kda else ()) + (self.hcnt,)
        self.kdecode_conv(v["q32"], *bufs, x, conv_state, conv_weight, conv_bias, a, b, A_log, dt_bias, self.Q0, idx, out, self.work)

    def dequantize(self, ssm, idx):
        """Materialize the fp32 state of the slots idx in place (before the engine's own prefill kernel runs on them)."""
        if idx.numel() == 0:
            return
        v = self.views(ssm)
        self.kdeq(ssm, v["Sq"], v["Sk"], v["Sv"], self.Kbuf, self.Ubuf, self.Wbuf, self.Pbuf, self.Gbuf, self.hcnt,
                  v["uq"], idx.to(torch.int32).contiguous())

    def quantize(self, ssm, idx):
        """Write the 8-bit checkpoint of the fp32 states in the slots idx and reset their windows (after a prefill)."""
        if idx.numel() == 0:
            return
        v = self.views(ssm)
        self.kquant(ssm, v["Sq"], v["Sk"], v["Sv"], v["uq"], self.Wbuf, self.Pbuf, self.hcnt, self.Q0,
                    idx.to(torch.int32).contiguous(), self.Gbuf if self.kda else None)


_STATES = {}
_GEN = [0]


def get_state(layer, ssm, **kw):
    """The LeapQuantState of `layer` for its current state tensor; rebuilt when the engine swaps the cache after
    profiling (reference leapquant/state.py:172-189).  Refuses prefix caching of the recurrent state."""
    st = layer.__dict__.get("_leapquant")
    k = _ident(ssm)
    if st is not None and st.key == k:
        return st
    if st is not None and st.gen == _GEN[0]:            # cache re-allocated: drop every buffer of the old one
        _GEN[0] += 1
        _STATES.clear()
        torch.cuda.empty_cache()
    st = _STATES.get(k)
    if st is None:
        cc = getattr(layer, "cache_config", None)
        if cc is not None and getattr(cc, "mamba_cache_mode", "none") != "none":
            raise RuntimeError("LeapQuant keeps each sequence's window buffer next to its state slot and does not support "
                               "prefix caching of the recurrent state: run vLLM with --no-enable-prefix-caching")
        st = _STATES[k] = LeapQuantState(ssm, **kw)
        st.gen = _GEN[0]
    layer._leapquant = st
    return st
