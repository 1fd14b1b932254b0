"""GPU parity tests at the shape the benchmark runs: many programs per persistent CTA and many flushed heads per CTA.

A B200 has 148 SMs and the step / decode kernels run one persistent CTA per SM, so a call with 1 280 (row, head) programs
gives every CTA eight or nine programs: the byte ring wraps, the sixteen stage descriptors are reused with flipped
parities, and -- when every window fills in the same call -- each CTA flushes eight or nine heads, four or five per team,
in the shared memory the ring leaves behind.  The standalone flush with 1 280 due heads gives each of its 296 CTAs four or
five heads.  The configurations are the benchmark's: GDN L = 64, R = 4, 16 key / 32 value heads and KDA L = 32, R = 8,
32 heads.
"""
import pytest
import torch

from lq_testlib import CpuSide, GpuSide, assert_close, random_states
from oracle import lq_oracle as O
from test_gpu_parity import check_flush, compare_window, make_pair, step_inputs, work_list  # noqa: F401 (fixture)

pytestmark = pytest.mark.gpu
K = V = 128
CONFIGS = [pytest.param(False, 64, 4, 16, 32, id="gdn_L64_R4_gqa2"), pytest.param(True, 32, 8, 32, 32, id="kda_L32_R8")]
N_ROWS = 40                                   # 40 rows x 32 heads = 1 280 programs: 8.6 per CTA on 148 SMs


def fill_windows(cpu, fill, seed):
    """Plausible window contents with `fill[slot, head]` live entries per head (ragged or uniform)."""
    b = cpu.bufs
    NS, HV, L = cpu.NS, cpu.HV, cpu.L
    g = torch.Generator().manual_seed(seed)
    live = torch.arange(L)[None, None, :] < fill[..., None]
    b.hcnt.copy_(fill.int())
    b.Kbuf.copy_((torch.randn(NS, HV, L, K, generator=g) * 0.09).bfloat16())
    b.Ubuf.copy_(torch.randn(NS, HV, L, V, generator=g).bfloat16())
    b.Wbuf.copy_(torch.where(live, 0.2 + 0.8 * torch.rand(NS, HV, L, generator=g), torch.zeros(NS, HV, L)))
    if cpu.kda:
        b.Pbuf.copy_(-1.5 * torch.rand(NS, HV, K, generator=g))                             # cumulative log gate
        e = (0.5 + 0.5 * torch.rand(NS, HV, L, K, generator=g)).half()                      # per-entry step factors
        b.Gbuf.copy_(torch.where(live[..., None], e, torch.ones_like(e)))
    else:
        b.Pbuf.copy_(0.1 + 0.9 * torch.rand(NS, HV, 1, generator=g))


def launch_step(gpu, kda, mixed, a, b_, A_log, dtb, idx, o):
    st, vv = gpu.st, gpu.st.views(gpu.ssm)
    N = mixed.shape[0]
    args = (mixed.cuda(), a.reshape(N, st.HV, -1).contiguous().cuda(), b_.cuda(), A_log.cuda(),
            dtb.reshape(st.HV, -1).contiguous().cuda(), vv["uq"], idx.cuda(), o)
    if kda:
        st.kstep(vv["q32"], vv["Sk"], vv["Sv"], vv["skv"], st.Kbuf, st.Ubuf, st.Wbuf, st.Pbuf, st.Gbuf, st.hcnt, *args)
    else:
        st.kstep(vv["q32"], vv["Sk"], vv["Sv"], vv["skv"], st.Kbuf, st.Ubuf, st.Wbuf, st.Pbuf, st.hcnt, *args)


@pytest.mark.parametrize("kda,L,R,H,HV", CONFIGS)
def test_step_ragged_fill_many_programs_per_cta(kda, L, R, H, HV):
    """(i) One step of 1 280 programs at ragged fill levels (stages of 22 KB to 55 KB wrap the ring), null rows in between,
    against the oracle from bit-identical inputs."""
    N, NS = N_ROWS, N_ROWS + 2
    cpu, gpu = make_pair(NS, HV, H, L, R, kda=kda, seed=11)
    g = torch.Generator().manual_seed(1)
    fill = torch.randint(0, L, (NS, HV), generator=g)
    fill_windows(cpu, fill, 2)
    gpu.sync_from(cpu)
    idx = torch.arange(1, N + 1, dtype=torch.int32)
    idx[torch.randperm(N, generator=g)[:3]] = 0
    mixed, a, b_, A_log, dtb = step_inputs(N, H, HV, 1, 5, kda)
    A_log = A_log + 0.05 * torch.arange(HV)
    o_c = torch.zeros(N, HV, V, dtype=torch.bfloat16)
    o_g = torch.full((N, HV, V), 3.0, dtype=torch.bfloat16, device="cuda")
    cpu.step(mixed[0], a[0], b_[0], A_log, dtb, idx, o_c)
    launch_step(gpu, kda, mixed[0], a[0], b_[0], A_log, dtb, idx, o_g)
    mag = float(o_c.float().abs().max())
    assert_close(o_g.cpu(), o_c, 8e-3, 1e-4 + 1e-3 * mag, "outputs")
    compare_window(cpu, gpu, list(range(NS)), "ragged batch")
    from leapquant_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("kda,L,R,H,HV", CONFIGS)
def test_step_long_padded_tail(kda, L, R, H, HV):
    """A CUDA-graph batch padded far beyond its live rows: 296 rows of which 40 are live, so every CTA meets runs of more
    than sixteen consecutive dead programs (more than the stage descriptors it has)."""
    N, NL, NS = 296, N_ROWS, N_ROWS + 1
    cpu, gpu = make_pair(NS, HV, H, L, R, kda=kda, seed=12)
    g = torch.Generator().manual_seed(3)
    fill_windows(cpu, torch.randint(0, L, (NS, HV), generator=g), 4)
    gpu.sync_from(cpu)
    idx = torch.zeros(N, dtype=torch.int32)
    idx[:NL // 2] = torch.arange(1, NL // 2 + 1, dtype=torch.int32)        # live rows at both ends, padding in between
    idx[-(NL - NL // 2):] = torch.arange(NL // 2 + 1, NL + 1, dtype=torch.int32)
    mixed, a, b_, A_log, dtb = step_inputs(N, H, HV, 1, 6, kda)
    o_c = torch.zeros(N, HV, V, dtype=torch.bfloat16)
    o_g = torch.full((N, HV, V), 3.0, dtype=torch.bfloat16, device="cuda")
    cpu.step(mixed[0], a[0], b_[0], A_log, dtb, idx, o_c)
    launch_step(gpu, kda, mixed[0], a[0], b_[0], A_log, dtb, idx, o_g)
    mag = float(o_c.float().abs().max())
    assert_close(o_g.cpu(), o_c, 8e-3, 1e-4 + 1e-3 * mag, "outputs")
    assert float(o_g[NL // 2: N - (NL - NL // 2)].float().abs().max()) == 0.0, "padding rows must write zeros"
    compare_window(cpu, gpu, list(range(NS)), "padded batch")
    from leapquant_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def all_windows_one_short(kda, L, R, H, HV, seed):
    """CPU state with every window of slots 1 .. N_ROWS one entry short of full, filled by running the oracle for L - 1
    steps (mild decay, so that the rebuilt state keeps a well-conditioned spectrum), and the inputs of the filling step."""
    N, NS = N_ROWS, N_ROWS + 1
    cpu = CpuSide(NS, HV, H, K, V, L, R, kda=kda)
    cpu.ssm.copy_(random_states(NS, HV, V, K, seed))
    idx = torch.arange(1, N + 1, dtype=torch.int32)
    cpu.quantize(idx)
    mixed, a, b_, A_log, dtb = step_inputs(N, H, HV, L, seed + 1, kda, gate_shift=4.0)
    o = torch.zeros(N, HV, V, dtype=torch.bfloat16)
    for t in range(L - 1):
        cpu.step(mixed[t], a[t], b_[t], A_log, dtb, idx, o)
    return cpu, idx, (mixed[L - 1], a[L - 1], b_[L - 1], A_log, dtb)


@pytest.mark.parametrize("kda,L,R,H,HV", CONFIGS)
def test_decode_every_window_fills(kda, L, R, H, HV, work_list):
    """(ii) One decode call in which all 1 280 windows fill: every CTA of the fused kernel flushes eight or nine heads, each
    team four or five, one after the other in the same shared memory (with the mailboxes too: a CTA that filled four or more
    windows keeps them all).  Bit-identical to the step kernel followed by the flush kernel."""
    cpu, idx, (mixed, a, b_, A_log, dtb) = all_windows_one_short(kda, L, R, H, HV, 21)
    gpu_f, gpu_s = GpuSide(cpu), GpuSide(cpu)
    gpu_s.st.fused = False
    N = idx.numel()
    o_f = torch.zeros(N, HV, V, dtype=torch.bfloat16, device="cuda")
    o_s = torch.zeros_like(o_f)
    for gsd, o in ((gpu_f, o_f), (gpu_s, o_s)):
        gsd.st.decode(gsd.ssm, mixed.cuda(), a.cuda(), b_.cuda(), A_log.cuda(), dtb.cuda(), idx.cuda(), o)
    bits = lambda x: x.view(torch.int32) if x.dtype == torch.float32 else x.view(torch.int16) if x.element_size() == 2 else x
    assert int(gpu_f.st.hcnt[1:].abs().max()) == 0, "every window must have been flushed"
    assert torch.equal(bits(o_f), bits(o_s))
    for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf", "hcnt") + (("Gbuf",) if kda else ()):
        assert torch.equal(bits(getattr(gpu_f.st, name)), bits(getattr(gpu_s.st, name))), name
    assert torch.equal(bits(gpu_f.ssm), bits(gpu_s.ssm))
    from leapquant_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("kda,L,R,H,HV", CONFIGS)
def test_flush_many_due_heads_per_cta(kda, L, R, H, HV):
    """(iii) The standalone flush with 1 280 due heads (more than its 296 CTAs: each flushes four or five), stage by stage
    against the oracle from bit-identical inputs."""
    cpu, idx, (mixed, a, b_, A_log, dtb) = all_windows_one_short(kda, L, R, H, HV, 23)
    o = torch.zeros(idx.numel(), HV, V, dtype=torch.bfloat16)
    cpu.step(mixed, a, b_, A_log, dtb, idx, o)                             # the filling step, on the oracle
    assert int(cpu.bufs.hcnt[1:].min()) == L
    gpu = GpuSide(cpu)
    # (21 million codes: the worst evaluation noise of the rebuilt state over that many elements is several times the typical
    #  one, so the distance from a rounding boundary within which a code may differ is 0.05 code units here)
    check_flush(cpu, gpu, idx, list(range(1, N_ROWS + 1)), f"flush of 1280 heads kda={kda}", code_tol=5e-2)
    assert int(gpu.st.hcnt.abs().max()) == 0


@pytest.mark.parametrize("kda,L,R,H,HV", CONFIGS)
def test_shared_work_list_staggered_fill(kda, L, R, H, HV):
    """(iv) A serving batch: 200 sequences whose windows fill at different steps (sequence n starts with n mod L entries), so
    every step fills the windows of a few rows and their heads land on a few CTAs.  The fused decode that shares one list of
    due heads among the CTAs, the fused decode in which every CTA flushes its own heads, and step-then-flush give the same
    bits at every step; the list is left all zero by every launch."""
    from leapquant_b200 import _lib
    from leapquant_b200.state import LeapQuantState
    N, NS = 200, 201                               # 6 400 programs: above the size from which the list is used by default
    g = torch.Generator(device="cuda").manual_seed(31)
    base = torch.randn(NS, HV, V, K, device="cuda", generator=g) * 0.5
    idx = torch.arange(1, N + 1, dtype=torch.int32, device="cuda")
    arms = []
    for name in ("shared", "own", "split"):
        ssm = base.clone()
        st = LeapQuantState(ssm, H, kda=kda, gate_lower_bound=-5.0 if kda else 0.0, L=L, R=R)
        st.quantize(ssm, idx)
        if name == "own":
            st.work = None
        if name == "split":
            st.fused = False
        arms.append((ssm, st, torch.zeros(N, HV, V, dtype=torch.bfloat16, device="cuda")))
    T = 2 * L + 3
    mixed, a, b_, A_log, dtb = step_inputs(N, H, HV, T, 32, kda, gate_shift=3.0)
    A_log, dtb = A_log.cuda(), dtb.cuda()
    bits = lambda x: x.view(torch.int32) if x.dtype == torch.float32 else x.view(torch.int16) if x.element_size() == 2 else x
    start = torch.arange(N) % L
    for t in range(T):
        # the first L - 1 steps build the stagger: row n joins at step L - 1 - (n mod L)
        rows = torch.nonzero(start >= L - 1 - t).flatten() if t < L - 1 else torch.arange(N)
        m, aa, bb = mixed[t][rows].cuda(), a[t][rows].cuda(), b_[t][rows].cuda()
        for ssm, st, o in arms:
            st.decode(ssm, m, aa, bb, A_log, dtb, idx[rows.cuda()].contiguous(), o[: rows.numel()])
        n = rows.numel()
        for ssm, st, o in arms[1:]:
            assert torch.equal(bits(arms[0][2][:n]), bits(o[:n])), t
            assert torch.equal(arms[0][1].hcnt, st.hcnt), t
        w = arms[0][1].work
        assert int(w[0]) == 0 and int(w[2:].abs().max()) == 0, t
    assert int(arms[0][1].hcnt.max()) < L
    for ssm, st, o in arms[1:]:
        for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf") + (("Gbuf",) if kda else ()):
            assert torch.equal(bits(getattr(arms[0][1], name)), bits(getattr(st, name))), name
        assert torch.equal(bits(arms[0][0]), bits(ssm))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("kda,L,R,H,HV,N", [pytest.param(False, 16, 4, 16, 32, 200, id="gdn_L16"), pytest.param(True, 8, 8, 32, 32, 300, id="kda_L8")])
def test_mailboxes_with_random_batches(kda, L, R, H, HV, N):
    """(v) Short windows and a random 90 % of the rows in every call: the number of heads that fill per step, and the CTAs they
    land on, change from call to call.  Over twenty windows the decode with mailboxes and the decode in which every CTA
    flushes its own heads stay bit-identical, the mailboxes are empty after every call and no wait runs out."""
    from leapquant_b200 import _lib
    from leapquant_b200.state import LeapQuantState
    NS = N + 1
    g = torch.Generator(device="cuda").manual_seed(51)
    base = torch.randn(NS, HV, V, K, device="cuda", generator=g) * 0.5
    idx = torch.arange(1, N + 1, dtype=torch.int32, device="cuda")
    arms = []
    for name in ("mailboxes", "own"):
        ssm = base.clone()
        st = LeapQuantState(ssm, H, kda=kda, gate_lower_bound=-5.0 if kda else 0.0, L=L, R=R)
        st.quantize(ssm, idx)
        if name == "own":
            st.work = None
        arms.append((ssm, st, torch.zeros(N, HV, V, dtype=torch.bfloat16, device="cuda")))
    T = 4 * L
    mixed, a, b_, A_log, dtb = step_inputs(N, H, HV, T, 52, kda, gate_shift=3.0)
    mixed, a, b_, A_log, dtb = mixed.cuda(), a.cuda(), b_.cuda(), A_log.cuda(), dtb.cuda()
    bits = lambda x: x.view(torch.int32) if x.dtype == torch.float32 else x.view(torch.int16) if x.element_size() == 2 else x
    gen = torch.Generator().manual_seed(53)
    for s in range(20 * L):
        t = s % T
        rows = torch.nonzero(torch.rand(N, generator=gen) < 0.9).flatten().cuda()
        n = rows.numel()
        for ssm, st, o in arms:
            st.decode(ssm, mixed[t][rows].contiguous(), a[t][rows].contiguous(), b_[t][rows].contiguous(), A_log, dtb,
                      idx[rows].contiguous(), o[:n])
        if s % 8 == 0:
            assert torch.equal(bits(arms[0][2][:n]), bits(arms[1][2][:n])), s
            assert torch.equal(arms[0][1].hcnt, arms[1][1].hcnt), s
            w = arms[0][1].work
            assert int(w[0]) == 0 and int(w[2:].abs().max()) == 0, s
    for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf") + (("Gbuf",) if kda else ()):
        assert torch.equal(bits(getattr(arms[0][1], name)), bits(getattr(arms[1][1], name))), name
    assert torch.equal(bits(arms[0][0]), bits(arms[1][0]))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("kda,L,R,H,HV", CONFIGS)
def test_dequantize_many_heads_per_cta(kda, L, R, H, HV):
    """(vi) The dequantize kernel is persistent: with 10 560 heads every CTA walks 35 or 36 of them, so its two stages are
    reused many times and the warp that looks ahead fetches a second batch of 32 heads.  Windows of every length (empty,
    short enough to travel with the stage, longer), padding rows in the batch.  One call over the whole batch gives the bits
    of calls of eight rows each -- one head per CTA, the shape the oracle tests cover -- and no wait runs out."""
    from leapquant_b200 import _lib
    from leapquant_b200.state import LeapQuantState
    N, NS = 330, 331
    g = torch.Generator(device="cuda").manual_seed(61)
    base = torch.randn(NS, HV, V, K, device="cuda", generator=g) * 0.5
    idx_all = torch.arange(1, N + 1, dtype=torch.int32, device="cuda")
    st0 = LeapQuantState(base, H, kda=kda, gate_lower_bound=-5.0 if kda else 0.0, L=L, R=R)
    st0.quantize(base, idx_all)
    # windows: a third empty, a third with at most 8 entries, the rest anything up to L
    kind = torch.randint(0, 3, (NS, HV), device="cuda", generator=g)
    short = torch.randint(1, 9, (NS, HV), device="cuda", generator=g)
    long_ = torch.randint(1, L + 1, (NS, HV), device="cuda", generator=g)
    st0.hcnt.copy_(torch.where(kind == 0, torch.zeros_like(short), torch.where(kind == 1, short, long_)).to(torch.int32))
    st0.Kbuf.copy_((torch.randn(st0.Kbuf.shape, device="cuda", generator=g) * 0.1).to(torch.bfloat16))
    st0.Ubuf.copy_((torch.randn(st0.Ubuf.shape, device="cuda", generator=g) * 0.5).to(torch.bfloat16))
    st0.Wbuf.copy_(torch.rand(st0.Wbuf.shape, device="cuda", generator=g))
    if kda:
        st0.Pbuf.copy_(-torch.rand(st0.Pbuf.shape, device="cuda", generator=g))
        st0.Gbuf.copy_((0.9 + 0.1 * torch.rand(st0.Gbuf.shape, device="cuda", generator=g)).to(torch.float16))
    else:
        st0.Pbuf.copy_(0.5 + 0.5 * torch.rand(st0.Pbuf.shape, device="cuda", generator=g))
    names = ("Kbuf", "Ubuf", "Wbuf", "Pbuf", "hcnt") + (("Gbuf",) if kda else ())
    snap = {n: getattr(st0, n).clone() for n in names}
    # the batch: every slot once, in a shuffled order, with padding rows (slot 0) in between
    perm = (torch.randperm(N, generator=torch.Generator().manual_seed(62)) + 1).to(torch.int32)
    rows = torch.cat([perm[:100], torch.zeros(3, dtype=torch.int32), perm[100:], torch.zeros(1, dtype=torch.int32)]).cuda()
    results = []
    for chunk in (rows.numel(), 8):
        ssm = base.clone()
        for n in names:
            getattr(st0, n).copy_(snap[n])
        for i in range(0, rows.numel(), chunk):
            st0.dequantize(ssm, rows[i:i + chunk].contiguous())
        results.append((ssm, {n: getattr(st0, n).clone() for n in names}))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    (s_all, b_all), (s_8, b_8) = results
    assert torch.equal(s_all.view(torch.int32), s_8.view(torch.int32))
    for n in names:
        a, b = b_all[n], b_8[n]
        assert torch.equal(a.view(torch.int16) if a.element_size() == 2 else a.view(torch.int32), b.view(torch.int16) if b.element_size() == 2 else b.view(torch.int32)), n
    assert not torch.equal(s_all[1:], base[1:])                  # (something was dequantized)
    if not kda:
        assert int(b_all["hcnt"][1:].abs().max()) == 0           # the GDN dequantize folds the window in and empties it
