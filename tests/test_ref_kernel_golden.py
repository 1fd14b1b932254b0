"""The oracle and the CUDA library against OUTPUTS OF THE REFERENCE'S OWN KERNELS.

tests/golden/ref_kernels/*.npz were produced on a B200 by tests/golden/make_ref_kernel_golden.py, which builds the
reference's plain-SIMT TileLang kernels -- make_quantize (leapquant/kernels.py:2126-2242), make_dequant (:2041-2123) and
make_lowrank (:2246-2331) -- and runs them on seeded inputs (tilelang 0.1.9; log.json records the versions).  The fixtures
hold the inputs too, so nothing here needs the reference, tilelang, or (for the CPU half) a GPU.

What "equal" means: the rank-R factors of quantize and lowrank come out of a subspace iteration in fp32 whose summation
order differs between implementations, so factors are compared through their products Q U^T and through the dequantised
state (rtol 1e-3 and an absolute term of 2e-3 of the state's magnitude).  Given the REFERENCE'S stored factors, the scales
and the INT8 codes are a deterministic function of the input, and there the oracle must reproduce the reference's bytes:
Sk / Sv to 1e-5 relative, codes exactly except +-1 where the pre-rounding value sits on a rounding boundary.
"""
import glob
import json
import os

import numpy as np
import pytest
import torch

from oracle import lq_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels")
K = V = 128
bf16 = lambda a: torch.from_numpy(a).view(torch.bfloat16)
f16 = lambda a: torch.from_numpy(a).view(torch.float16)
QUANT = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "quantize_*.npz")))
DEQ = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "dequant_*.npz")))
LOWR = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "lowrank_*.npz")))


def test_fixtures_present_and_complete():
    log = json.load(open(os.path.join(GOLD, "log.json")))
    assert all(v == "ok" for v in log["kernels"].values()), log["kernels"]
    assert len(QUANT) == 4 and len(DEQ) == 2 and len(LOWR) == 2


def close(a, b, rtol, atol, what):
    err = (a.float() - b.float()).abs()
    lim = atol + rtol * b.float().abs()
    assert bool((err <= lim).all()), f"{what}: max err {float(err.max()):.3e}, {int((err > lim).sum())} of {err.numel()} off"


def codes_match(code, x, slack, what, max_frac=2e-3):
    """code == round-half-even(x) except +-1 where x is within `slack` (code units, per element) of a half-integer."""
    want = torch.round(x.double())
    d = code.double() - want
    bad = d != 0
    if not bool(bad.any()):
        return
    assert int(d.abs().max()) <= 1, what + ": a code differs by more than one LSB"
    frac = (x.double()[bad] - torch.floor(x.double()[bad]) - 0.5).abs()
    assert bool((frac <= slack[bad].double()).all()), f"{what}: {int((frac > slack[bad].double()).sum())} codes differ away from a boundary"
    assert int(bad.sum()) <= max_frac * code.numel(), f"{what}: {int(bad.sum())} boundary codes"


def quant_fixture(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    NS, HV, _, _, L, R = (int(x) for x in z["dims"])
    S = bf16(z["S"]).float()                                         # [2, HV, V, K] inputs of slots 1, 2
    ref = dict(Sq=torch.from_numpy(z["Sq"]), Sk=torch.from_numpy(z["Sk"]), Sv=torch.from_numpy(z["Sv"]), uq=f16(z["uq"]))
    return z, NS, HV, L, R, S, ref


def check_quantized(S, got, ref, what):
    """`got` and `ref`: dicts Sq, Sk, Sv, uq of the same heads.  Products and dequantised state; then the deterministic stage."""
    mag = float(S.abs().max())
    prod = lambda uq: torch.einsum("...rv,...rc->...vc", uq.float()[..., K:], uq.float()[..., :K])
    deq = lambda d: d["Sq"].float() / 127.0 * d["Sk"][..., None, :] * d["Sv"][..., :, None] + prod(d["uq"])
    close(prod(got["uq"]), prod(ref["uq"]), 1e-3, 2e-3 * mag, what + ": Q U^T")
    # Dequantised state.  The two sets of factors differ at fp32 rounding level, so a residual that sits on a rounding
    # boundary may become the neighbouring code: fewer than 0.1 % of the elements may be off by up to one code step.
    err = (deq(got) - deq(ref)).abs()
    lim = 2e-3 * mag + 1e-3 * deq(ref).abs()
    step = ref["Sk"][..., None, :] * ref["Sv"][..., :, None] / 127.0
    assert bool((err <= lim + 1.01 * step).all()), f"{what}: dequantised state off by more than one code step ({float(err.max()):.3e})"
    assert int((err > lim).sum()) <= 1e-3 * err.numel(), f"{what}: {int((err > lim).sum())} elements beyond the tolerance"
    assert float((deq(ref) - S).abs().max()) <= 2e-2 * mag                  # (the reference's own checkpoint is that close)


@pytest.mark.parametrize("name", QUANT)
def test_oracle_quantize_against_reference_kernel(name):
    z, NS, HV, L, R, S, ref = quant_fixture(name)
    # window reset as the reference kernel left it
    assert float(np.abs(z["Wbuf"][[1, 2]]).max()) == 0.0 and float(np.abs(z["Pbuf"][[1, 2]] - 1).max()) == 0.0
    assert int(np.abs(z["hcnt"][[1, 2]]).max()) == 0 and int(z["hcnt"][0].min()) == 3
    code, sk, sv, uq, _ = O.quantize_heads(S.reshape(-1, V, K), O.make_q0(V, R), 1)
    got = dict(Sq=code.reshape(2, HV, V, K), Sk=sk.reshape(2, HV, K), Sv=sv.reshape(2, HV, V), uq=uq.reshape(2, HV, R, K + V))
    check_quantized(S, got, ref, name)
    # the deterministic stage: from the REFERENCE'S stored factors the oracle reproduces the reference's scales and codes
    uqr = ref["uq"].float()
    E = S.clone()
    for r in range(R):
        E = (E.double() - uqr[..., r, K:, None].double() * uqr[..., r, None, :K].double()).float()
    sk_o, sv_o, code_o = O.quantize_stage(E)
    close(sk_o, ref["Sk"], 1e-5, 0.0, name + ": Sk from the reference's factors")
    # fp32 evaluation noise of the residual (a few ulps of the magnitudes that cancel), in units of E / Sk
    mags = S.abs() + torch.einsum("...rv,...rc->...vc", uqr[..., K:].abs(), uqr[..., :K].abs())
    noise = 6e-7 * mags / ref["Sk"][..., None, :]
    assert bool(((sv_o - ref["Sv"]).abs() <= 1e-5 * ref["Sv"] + noise.amax(-1)).all()), name + ": Sv"
    x = E / (ref["Sk"][..., None, :] * ref["Sv"][..., :, None]) * 127.0
    codes_match(ref["Sq"], x, 1e-3 + noise / ref["Sv"][..., :, None] * 127.0, name + ": reference codes vs oracle stage")
    assert int(ref["Sq"].abs().max()) == 127


def deq_fixture(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    NS, HV, _, _, L, R = (int(x) for x in z["dims"])
    ck = dict(Sq=torch.from_numpy(z["Sq"]), Sk=torch.from_numpy(z["Sk"]), Sv=torch.from_numpy(z["Sv"]), uq=f16(z["uq"]))
    win = dict(Kbuf=bf16(z["Kbuf"]), Ubuf=bf16(z["Ubuf"]), Wbuf=torch.from_numpy(z["Wbuf_in"]), Pbuf=torch.from_numpy(z["Pbuf_in"]),
               hcnt=torch.from_numpy(z["hcnt_in"]))
    return z, HV, L, R, ck, win


@pytest.mark.parametrize("name", DEQ)
def test_oracle_dequantize_against_reference_kernel(name):
    z, HV, L, R, ck, win = deq_fixture(name)
    S = O.dequant_heads(ck["Sq"], ck["Sk"], ck["Sv"], ck["uq"], win["Pbuf"][..., 0], win["Kbuf"], win["Ubuf"], win["Wbuf"],
                        win["hcnt"].long())
    ref = torch.from_numpy(z["S_out"])
    close(S, ref, 1e-4, 1e-5 * float(ref.abs().max()), name + ": fp32 state")
    assert float(np.abs(z["Wbuf_out"]).max()) == 0.0 and float(np.abs(z["Pbuf_out"] - 1).max()) == 0.0 and int(np.abs(z["hcnt_out"]).max()) == 0


@pytest.mark.parametrize("name", LOWR)
def test_oracle_lowrank_against_reference_kernel(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    r, iters = (int(x) for x in z["r"])
    x = bf16(z["x"]).float()
    U, Q = O.lowrank_factor(x, r, iters)
    Ur, Qr = torch.from_numpy(z["U"]), torch.from_numpy(z["Q"])
    close(U @ Q.transpose(-1, -2), Ur @ Qr.transpose(-1, -2), 1e-3, 1e-3 * float(x.abs().max()), name + ": U Q^T")
    G = torch.einsum("nvr,nvs->nrs", Qr, Qr)
    assert torch.allclose(G, torch.eye(r).expand_as(G), atol=1e-4), "the reference's Q is orthonormal"


# ---------------------------------------------------------------------------------------------------------------------
# the CUDA library against the same fixtures (through the C ABI)
# ---------------------------------------------------------------------------------------------------------------------
def gpu_state(NS, HV, L, R):
    from leapquant_b200.state import LeapQuantState
    ssm = torch.zeros(NS, HV, V, K, device="cuda")
    return ssm, LeapQuantState(ssm, HV, L=L, R=R)


@pytest.mark.gpu
@pytest.mark.parametrize("name", QUANT)
def test_lq_quantize_against_reference_kernel(name):
    z, NS, HV, L, R, S, ref = quant_fixture(name)
    ssm, st = gpu_state(NS, HV, L, R)
    ssm[[1, 2]] = S.cuda()
    st.quantize(ssm, torch.tensor([2, 0, 1], dtype=torch.int32, device="cuda"))
    v = st.views(ssm)
    got = {k: v[k][[1, 2]].cpu() for k in ("Sq", "Sk", "Sv", "uq")}
    check_quantized(S, got, ref, name + " (lq_quantize)")


@pytest.mark.gpu
@pytest.mark.parametrize("name", DEQ)
def test_lq_dequant_against_reference_kernel(name):
    z, HV, L, R, ck, win = deq_fixture(name)
    ssm, st = gpu_state(3, HV, L, R)
    v = st.views(ssm)
    for k in ("Sq", "Sk", "Sv", "uq"):
        v[k][[1, 2]] = ck[k].cuda()
    for k in ("Kbuf", "Ubuf", "Wbuf", "Pbuf", "hcnt"):
        getattr(st, k)[[1, 2]] = win[k].cuda()
    st.dequantize(ssm, torch.tensor([2, 0, 1], dtype=torch.int32, device="cuda"))
    ref = torch.from_numpy(z["S_out"])
    close(ssm[[1, 2]].cpu(), ref, 1e-4, 1e-5 * float(ref.abs().max()), name + " (lq_dequant): fp32 state")
    assert int(st.hcnt[[1, 2]].abs().max()) == 0 and float(st.Wbuf[[1, 2]].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("name", LOWR)
def test_lq_lowrank_against_reference_kernel(name):
    from leapquant_b200.kernels import lowrank_factor
    z = np.load(os.path.join(GOLD, name + ".npz"))
    r, iters = (int(x) for x in z["r"])
    x = bf16(z["x"]).float()
    U, Q = lowrank_factor(x.cuda(), r, iters)
    Ur, Qr = torch.from_numpy(z["U"]), torch.from_numpy(z["Q"])
    close(U.cpu() @ Q.cpu().transpose(-1, -2), Ur @ Qr.transpose(-1, -2), 1e-3, 1e-3 * float(x.abs().max()), name + " (lq_lowrank): U Q^T")
