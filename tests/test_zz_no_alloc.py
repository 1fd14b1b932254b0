"""GPU test of lq_gdn_decode_noalloc, the decode entry point for callers that cannot allocate device memory: the mailboxes
of due heads live in a fixed device array inside the library instead of a buffer of the caller's.  Called through the C
ABI, twice in a row, against lq_gdn_decode with a caller-owned list on the same inputs: outputs, window buffers and packed
state must agree bit for bit (the mailboxes never change a result, only which CTA flushes a head).

The file sorts after the other test files on purpose: it has to pass both in a fresh process and after everything else has
used the device.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
K = V = 128


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


class Side:
    """One copy of the state of a GDN layer on the device, driven through raw C-ABI calls."""

    def __init__(self, base, NS, HV, H, L, R):
        from leapquant_b200 import _lib
        from leapquant_b200.state import LeapQuantState
        self.ssm = base.clone()
        st = LeapQuantState(self.ssm, H, L=L, R=R)                       # allocates the window buffers; its kernels quantize
        st.quantize(self.ssm, torch.arange(1, NS, dtype=torch.int32, device="cuda"))
        self.st, self.L, self.HV = st, L, HV
        self.dims = _lib.dims(NS, HV, H, K, V, L, R, self.ssm.stride(0))
        self.lib = _lib.lib()

    def args(self, mixed, a, b, A_log, dtb, idx, out):
        st = self.st
        return (self.dims, _ptr(self.ssm), _ptr(st.Kbuf), _ptr(st.Ubuf), _ptr(st.Wbuf), _ptr(st.Pbuf), _ptr(st.hcnt), _ptr(mixed),
                _ptr(a), _ptr(b), _ptr(A_log), _ptr(dtb), _ptr(idx), _ptr(out), int(mixed.shape[0]), ctypes.c_float(0.0),
                _ptr(st.Q0), 1)


def test_noalloc_decode_matches_decode_twice_in_a_row():
    from leapquant_b200 import _lib
    from oracle import lq_oracle as O
    NS, N, HV, H, L, R = 81, 80, 32, 16, 8, 4                  # 2 560 programs: the mailboxes are in use by default
    g = torch.Generator(device="cuda").manual_seed(41)
    base = torch.randn(NS, HV, V, K, device="cuda", generator=g) * 0.5
    ours, ref = Side(base, NS, HV, H, L, R), Side(base, NS, HV, H, L, R)
    T = 2 * L                                                   # every window fills twice: two calls flush through the list
    mixed, a, b, A_log, dtb = O.synth_inputs(N, H, HV, K, V, T, 42, kda=False)
    a = (a.float() - 3.0).to(a.dtype)
    A_log, dtb = A_log.cuda(), dtb.cuda()
    idx = torch.arange(1, N + 1, dtype=torch.int32, device="cuda")
    o_n = torch.zeros(N, HV, V, dtype=torch.bfloat16, device="cuda")
    o_r = torch.zeros_like(o_n)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    bits = lambda x: x.view(torch.int32) if x.dtype == torch.float32 else x.view(torch.int16) if x.element_size() == 2 else x
    flushed = 0
    for t in range(T):
        m, aa, bb = mixed[t].cuda(), a[t].reshape(N, HV, 1).contiguous().cuda(), b[t].cuda()
        # consecutive calls of the entry point under test: each one re-uses the one fixed array
        rc = ours.lib.lq_gdn_decode_noalloc(*ours.args(m, aa, bb, A_log, dtb, idx, o_n), stream)
        assert rc == 0, _lib.lib().lq_strerror(rc)
        rc = ref.lib.lq_gdn_decode(*ref.args(m, aa, bb, A_log, dtb, idx, o_r), _ptr(ref.st.work),
                                   ref.st.work.numel() * 4, stream)
        assert rc == 0, _lib.lib().lq_strerror(rc)
        assert torch.equal(bits(o_n), bits(o_r)), t
        assert torch.equal(ours.st.hcnt, ref.st.hcnt), t
        flushed += int((ref.st.hcnt[1:] == 0).all())
    assert flushed == 2, "the windows must have filled (and been flushed) twice"
    for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf"):
        assert torch.equal(bits(getattr(ours.st, name)), bits(getattr(ref.st, name))), name
    assert torch.equal(bits(ours.ssm), bits(ref.ssm))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def test_noalloc_rejects_more_heads_than_its_array():
    from leapquant_b200 import _lib
    L = _lib.lib()
    one = ctypes.c_void_p(256)
    big = _lib.dims(4096, 32, 16, K, V, 16, 4, 32 * K * V)      # 4096 rows x 32 heads > 65 536 entries
    rc = L.lq_gdn_decode_noalloc(big, one, one, one, one, one, one, one, one, one, one, one, one, one, 4096, ctypes.c_float(0.0),
                                 one, 1, None)
    assert rc == -6 and b"lq_gdn_decode_noalloc" in L.lq_strerror(rc)
