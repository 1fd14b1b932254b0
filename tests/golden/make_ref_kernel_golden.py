"""Generates fixtures from the REFERENCE'S OWN TileLang kernels for quantize, dequant and lowrank (needs a CUDA device).

    LEAPQUANT_REFERENCE=/path/to/LeapQuant python tests/golden/make_ref_kernel_golden.py [out_dir]

Only the three plain-SIMT kernels are built and run: make_quantize (leapquant/kernels.py:2126-2242), make_dequant
(:2041-2123) and make_lowrank (:2246-2331).  They contain no mbarrier and no spin.  The persistent step and flush kernels
are NOT built here.  The reference pins tilelang 0.1.12; whatever tilelang the machine has is used, and a failure to
lower or compile is reported per kernel (the run still writes the fixtures of the kernels that worked and a log).

Inputs are seeded on the host and stored with the outputs, so the consuming tests (tests/test_ref_kernel_golden.py) need
neither the reference nor tilelang.  Input states are rounded to bf16 values so that the fixture stores them in two bytes.
"""
import json
import os
import sys
import traceback

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
K = V = 128


def bf16_exact(x):
    return x.to(torch.bfloat16).to(torch.float32)


def bits16(x):
    return x.contiguous().view(torch.int16).cpu().numpy()


def outlier_states(n, HV, seed, frac=0.01, gain=50.0):
    g = torch.Generator().manual_seed(seed)
    S = torch.randn(n, HV, V, K, generator=g)
    nr = max(1, int(round(frac * V)))
    for i in range(n):
        for h in range(HV):
            S[i, h, torch.randperm(V, generator=g)[:nr], :] *= gain
            S[i, h, :, torch.randperm(K, generator=g)[:nr]] *= gain
    return S


def packed(ssm, views, slots):
    """The checkpoint a kernel left in the listed slots: codes, scales, factors."""
    sl = torch.as_tensor(slots, device=ssm.device)
    return dict(Sq=views["Sq"][sl].cpu().numpy(), Sk=views["Sk"][sl].cpu().numpy(), Sv=views["Sv"][sl].cpu().numpy(),
                uq=bits16(views["uq"][sl]))


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_kernels")
    os.makedirs(out, exist_ok=True)
    # a checkout of the reference: LEAPQUANT_REFERENCE, or a directory `reference` beside this repository
    ref = os.environ.get("LEAPQUANT_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
    sys.path.insert(0, ref)
    log = {"reference": ref, "torch": torch.__version__, "device": torch.cuda.get_device_name(0), "kernels": {}}
    try:
        import tilelang
        log["tilelang"] = getattr(tilelang, "__version__", "?")
        from leapquant import kernels as RK
        from leapquant.state import state_views
    except Exception as e:                                      # nothing can be generated
        log["import_error"] = "".join(traceback.format_exception_only(type(e), e)).strip()
        json.dump(log, open(os.path.join(out, "log.json"), "w"), indent=1)
        print(json.dumps(log))
        return 1
    dev = torch.device("cuda", 0)
    NS, HV, L = 3, 2, 16
    SS = HV * V * K
    slots = [1, 2]
    idx = torch.tensor([2, 0, 1], dtype=torch.int32, device=dev)
    q0 = lambda R: torch.randn(V, R, generator=torch.Generator().manual_seed(0))

    # ---- quantize: seeded N(0, 0.1) states and x50-outlier states, R = 4 and 8 ----
    for R in (4, 8):
        for kind in ("normal", "outlier"):
            name = f"quantize_R{R}_{kind}"
            try:
                S = (torch.randn(NS, HV, V, K, generator=torch.Generator().manual_seed(10 + R)) * 0.1 if kind == "normal"
                     else outlier_states(NS, HV, 20 + R))
                S = bf16_exact(S)
                ssm = S.to(dev).clone()
                views = state_views(ssm, R)
                Wbuf = torch.full((NS, HV, L), 0.5, device=dev)
                Pbuf = torch.full((NS, HV, 1), 0.25, device=dev)
                hcnt = torch.full((NS, HV), 3, dtype=torch.int32, device=dev)
                kq = RK.make_quantize(NS, HV, K, V, L, SS, R=R, ITERS=1)
                kq(ssm, views["Sq"], views["Sk"], views["Sv"], views["uq"], Wbuf, Pbuf, hcnt, q0(R).to(dev), idx)
                torch.cuda.synchronize()
                np.savez(os.path.join(out, name + ".npz"), dims=np.array([NS, HV, V, K, L, R]), slots=np.array(slots),
                         S=bits16(S[slots].to(torch.bfloat16)), Wbuf=Wbuf.cpu().numpy(), Pbuf=Pbuf.cpu().numpy(),
                         hcnt=hcnt.cpu().numpy(), **packed(ssm, views, slots))
                log["kernels"][name] = "ok"
            except Exception as e:
                log["kernels"][name] = "".join(traceback.format_exception_only(type(e), e)).strip()[-600:]

    # ---- dequant: a reference-quantized checkpoint plus a hand-made live window of h entries ----
    for R, h in ((4, 5), (8, 16)):
        name = f"dequant_R{R}_h{h}"
        try:
            g = torch.Generator().manual_seed(30 + R)
            S = bf16_exact(torch.randn(NS, HV, V, K, generator=g) * 0.1)
            ssm = S.to(dev).clone()
            views = state_views(ssm, R)
            Wbuf = torch.zeros(NS, HV, L, device=dev)
            Pbuf = torch.ones(NS, HV, 1, device=dev)
            hcnt = torch.zeros(NS, HV, dtype=torch.int32, device=dev)
            kq = RK.make_quantize(NS, HV, K, V, L, SS, R=R, ITERS=1)
            kq(ssm, views["Sq"], views["Sk"], views["Sv"], views["uq"], Wbuf, Pbuf, hcnt, q0(R).to(dev), idx)
            Kb = (torch.randn(NS, HV, L, K, generator=g) * 0.09).to(torch.bfloat16)
            Ub = torch.randn(NS, HV, L, V, generator=g).to(torch.bfloat16)
            Wb = torch.rand(NS, HV, L, generator=g)
            Pb = 0.2 + 0.8 * torch.rand(NS, HV, 1, generator=g)
            hc = torch.full((NS, HV), h, dtype=torch.int32)
            hc[2, 1] = max(h - 3, 0)
            Kbuf, Ubuf, Wbuf, Pbuf, hcnt = Kb.to(dev), Ub.to(dev), Wb.to(dev), Pb.to(dev), hc.to(dev)
            Gbuf = torch.zeros(NS, HV, L, 1, device=dev)
            torch.cuda.synchronize()
            before = packed(ssm, views, slots)
            kd = RK.make_dequant(NS, HV, K, V, L, SS, buf_dtype=RK.BF16, R=R)
            kd(ssm, views["Sq"], views["Sk"], views["Sv"], Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, views["uq"], idx)
            torch.cuda.synchronize()
            np.savez(os.path.join(out, name + ".npz"), dims=np.array([NS, HV, V, K, L, R]), slots=np.array(slots),
                     Kbuf=bits16(Kb[slots]), Ubuf=bits16(Ub[slots]), Wbuf_in=Wb[slots].numpy(), Pbuf_in=Pb[slots].numpy(),
                     hcnt_in=hc[slots].numpy(), S_out=ssm[slots].cpu().numpy(), Wbuf_out=Wbuf[slots].cpu().numpy(),
                     Pbuf_out=Pbuf[slots].cpu().numpy(), hcnt_out=hcnt[slots].cpu().numpy(), **before)
            log["kernels"][name] = "ok"
        except Exception as e:
            log["kernels"][name] = "".join(traceback.format_exception_only(type(e), e)).strip()[-600:]

    # ---- lowrank_factor: rank-r structure plus noise ----
    for r, iters in ((4, 3), (8, 1)):
        name = f"lowrank_r{r}_it{iters}"
        try:
            g = torch.Generator().manual_seed(40 + r)
            x = torch.randn(3, K, r, generator=g) @ torch.randn(3, r, V, generator=g) + 0.05 * torch.randn(3, K, V, generator=g)
            x = bf16_exact(x)
            U, Q = RK.lowrank_factor(x.to(dev), r, iters)
            torch.cuda.synchronize()
            np.savez(os.path.join(out, name + ".npz"), r=np.array([r, iters]), x=bits16(x.to(torch.bfloat16)), U=U.cpu().numpy(),
                     Q=Q.cpu().numpy())
            log["kernels"][name] = "ok"
        except Exception as e:
            log["kernels"][name] = "".join(traceback.format_exception_only(type(e), e)).strip()[-600:]

    json.dump(log, open(os.path.join(out, "log.json"), "w"), indent=1)
    print(json.dumps(log))
    return 0


if __name__ == "__main__":
    sys.exit(main())
