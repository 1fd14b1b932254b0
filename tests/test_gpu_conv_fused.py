"""GPU parity tests of the conv1d update that precedes the decode step: the standalone kernel against the oracle, and the
fused conv + decode launch against the standalone kernel followed by decode (bit for bit), for both layouts of the conv
state, GQA and non-GQA head layouts, null rows and windows that fill inside the call."""
import pytest
import torch

from lq_testlib import CpuSide, GpuSide, random_states
from oracle import lq_oracle as O
from test_gpu_parity import make_pair, step_inputs, work_list  # noqa: F401 (work_list is a fixture)

pytestmark = pytest.mark.gpu
K = V = 128


def conv_operands(NS, C, seed, dim_first):
    """bf16 conv state (viewed slot, channel, tap), taps and bias; dim_first: stored (slot, channel, tap), else (slot, tap, channel)."""
    g = torch.Generator().manual_seed(seed)
    store = torch.randn(NS, C, 3, generator=g).bfloat16() if dim_first else torch.randn(NS, 3, C, generator=g).bfloat16()
    w = (torch.randn(C, 4, generator=g) * 0.5).bfloat16()
    b = (torch.randn(C, generator=g) * 0.1).bfloat16()
    return store, w, b


def view_sct(store, dim_first):
    return store if dim_first else store.transpose(-1, -2)


@pytest.mark.parametrize("dim_first", [False, True], ids=["slot_tap_channel", "slot_channel_tap"])
def test_conv1d_update_against_oracle(dim_first):
    from leapquant_b200.kernels import make_conv1d_update
    NS, N, C = 9, 7, 2 * 2 * K + 4 * V
    store, w, b = conv_operands(NS, C, 3, dim_first)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(N, C + 64, generator=g).bfloat16()                  # rows wider than the channels: a row stride
    idx = torch.tensor([3, 0, 8, 1, -1, 5, 2], dtype=torch.int32)
    st_c = view_sct(store.clone(), dim_first)
    out_c = O.causal_conv1d_update(x, st_c, w, b, idx)
    store_g = store.cuda()
    out_g = torch.full((N, C), 7.0, dtype=torch.bfloat16, device="cuda")
    make_conv1d_update(NS, C)(x.cuda(), view_sct(store_g, dim_first), w.cuda(), b.cuda(), idx.cuda(), out_g)
    live = idx > 0
    # exp() of the device and of the host may differ in the last place of fp32: one bf16 ulp on a few outputs at most
    d = (out_g.cpu()[live].float() - out_c[live].float()).abs()
    assert bool((d <= 8e-3 * out_c[live].float().abs() + 1e-6).all()), float(d.max())
    assert float((d > 0).float().mean()) < 1e-3
    assert float((out_g.cpu()[~live].float() - 7.0).abs().max()) == 0.0, "rows without a slot must not be written"
    assert torch.equal(view_sct(store_g.cpu(), dim_first), st_c), "conv state after the update"
    # without a bias
    out_c2 = O.causal_conv1d_update(x, st_c, w, None, idx)
    make_conv1d_update(NS, C)(x.cuda(), view_sct(store_g, dim_first), w.cuda(), None, idx.cuda(), out_g)
    d2 = (out_g.cpu()[live].float() - out_c2[live].float()).abs()
    assert bool((d2 <= 8e-3 * out_c2[live].float().abs() + 1e-6).all())


@pytest.mark.parametrize("kda,L,R,H,HV,N", [(False, 16, 4, 2, 4, 11), (False, 64, 4, 16, 32, 40), (False, 16, 4, 1, 4, 9),
                                            (True, 16, 4, 2, 2, 11), (True, 32, 8, 32, 32, 40)])
@pytest.mark.parametrize("dim_first", [False, True], ids=["slot_tap_channel", "slot_channel_tap"])
def test_fused_conv_decode_equals_conv_then_decode(kda, L, R, H, HV, N, dim_first, work_list):
    """decode_conv as one launch == decode_conv as it runs by default (two launches) == the conv1d update kernel called by
    hand, then decode: outputs, window buffers, packed state and conv state, bit for bit, over more than a window, with null
    rows and rows that sit out some steps."""
    from leapquant_b200.kernels import make_conv1d_update
    NS, T = N + 2, L + 5
    C = 2 * H * K + HV * V
    cpu, gpu_f = make_pair(NS, HV, H, L, R, kda=kda, glb=(-5.0 if kda else 0.0), seed=8)
    gpu_s, gpu_d = GpuSide(cpu), GpuSide(cpu)
    store, w, b = conv_operands(NS, C, 5, dim_first)
    st_f, st_s, st_d = store.cuda(), store.clone().cuda(), store.clone().cuda()
    wg, bg = w.cuda(), b.cuda()
    g = torch.Generator().manual_seed(6)
    idx = torch.randperm(NS - 1, generator=g)[:N].int() + 1
    idx[2] = 0
    idx[N - 1] = -1
    idx = idx.cuda()
    _, a, b_, A_log, dtb = step_inputs(N, H, HV, T, 9, kda, gate_shift=2.0)
    conv = make_conv1d_update(NS, C)
    gpu_f.st.conv_one_launch = True
    assert not gpu_d.st.conv_one_launch
    o_f = torch.zeros(N, HV, V, dtype=torch.bfloat16, device="cuda")
    o_s, o_d = torch.zeros_like(o_f), torch.zeros_like(o_f)
    mixed = torch.zeros(N, C, dtype=torch.bfloat16, device="cuda")
    bits = lambda t: t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.int16) if t.element_size() == 2 else t
    for t in range(T):
        x = (torch.randn(N, C, generator=g) * 0.7).bfloat16().cuda()
        n = N if t % 3 else N // 2                                         # half of the rows skip every third step
        at, bt = a[t][:n].cuda(), b_[t][:n].cuda()
        gpu_f.st.decode_conv(gpu_f.ssm, x[:n], view_sct(st_f, dim_first), wg, bg, at, bt, A_log.cuda(), dtb.cuda(), idx[:n], o_f[:n])
        gpu_d.st.decode_conv(gpu_d.ssm, x[:n], view_sct(st_d, dim_first), wg, bg, at, bt, A_log.cuda(), dtb.cuda(), idx[:n], o_d[:n])
        conv(x[:n], view_sct(st_s, dim_first), wg, bg, idx[:n], mixed[:n])
        gpu_s.st.decode(gpu_s.ssm, mixed[:n], at, bt, A_log.cuda(), dtb.cuda(), idx[:n], o_s[:n])
        assert torch.equal(bits(o_f[:n]), bits(o_s[:n])) and torch.equal(bits(o_d[:n]), bits(o_s[:n])), t
        assert torch.equal(gpu_f.st.hcnt, gpu_s.st.hcnt), t
    assert torch.equal(bits(st_f), bits(st_s)) and torch.equal(bits(st_d), bits(st_s)), "conv state"
    assert torch.equal(bits(gpu_d.ssm), bits(gpu_s.ssm))
    for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf") + (("Gbuf",) if kda else ()):
        assert torch.equal(bits(getattr(gpu_f.st, name)), bits(getattr(gpu_s.st, name))), name
    assert torch.equal(bits(gpu_f.ssm), bits(gpu_s.ssm))
    from leapquant_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def test_conv_argument_errors():
    from leapquant_b200 import _lib
    from leapquant_b200.kernels import make_conv1d_update
    x = torch.zeros(2, 1024, dtype=torch.bfloat16, device="cuda")
    st = torch.zeros(4, 1024, 3, dtype=torch.bfloat16, device="cuda")
    w5 = torch.zeros(1024, 5, dtype=torch.bfloat16, device="cuda")
    idx = torch.ones(2, dtype=torch.int32, device="cuda")
    out = torch.zeros(2, 1024, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.LeapQuantError):                                 # conv state of the wrong depth for 5 taps
        make_conv1d_update(4, 1024)(x, st, w5, None, idx, out)
    st4 = torch.zeros(4, 1024, 4, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.LeapQuantError):                                 # 5 taps: unsupported width
        make_conv1d_update(4, 1024)(x, st4, w5, None, idx, out)
    with pytest.raises(_lib.LeapQuantError):                                 # fp32 operands
        make_conv1d_update(4, 1024)(x.float(), st, w5[:, :4].contiguous(), None, idx, out)
