"""Generates the golden fixtures of tests/golden/ by running the REFERENCE's own Python code on CPU tensors.

    python tests/golden/make_golden.py /path/to/reference_checkout

What the reference can execute without a GPU, and therefore what these fixtures pin:
  * `leapquant.state.state_views`            -> layout.json   (dtype / shape / stride / offset of every aliasing view)
  * `LeapQuantState._kda_rebuild`            -> kda_rebuild.npz   (pure torch; called unbound on a stand-in object)
  * `LeapQuantState._kda_checkpoint`         -> kda_checkpoint.npz (pure torch except `lowrank_factor`, a CUDA kernel,
                                                which is replaced here by the oracle's restatement; the fixture therefore
                                                pins the residual / scales / codes / factor packing GIVEN the factors)
The decode-step, flush, quantize and dequant kernels of the reference are CUDA-only and cannot produce fixtures here.
Inputs are seeded; bf16 / fp16 tensors are stored as int16 bit patterns.
"""
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def bits16(t):
    return t.contiguous().view(torch.int16).numpy()


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.path.insert(0, ROOT)
    import leapquant.state as RS              # the reference
    import leapquant.kernels as RK
    from oracle import lq_oracle as O

    # ---- 1. layout ----
    layout = []
    for (NS, HV, V, K, R, off, pad) in [(5, 3, 128, 128, 4, 0, 0), (4, 2, 128, 128, 8, 16, 0), (3, 2, 128, 128, 4, 32, 4096),
                                        (3, 2, 64, 128, 4, 0, 0), (2, 2, 32, 32, 2, 8, 0)]:
        SS = HV * V * K + pad
        store = torch.zeros(off + NS * SS)
        ssm = store[off:off + NS * SS].view(NS, SS)[:, :HV * V * K].view(NS, HV, V, K)
        views = RS.state_views(ssm, R)
        layout.append(dict(NS=NS, HV=HV, V=V, K=K, R=R, off=off, pad=pad,
                           views={k: dict(dtype=str(t.dtype), shape=list(t.shape), stride=list(t.stride()),
                                          offset=t.storage_offset()) for k, t in views.items()}))
    with open(os.path.join(HERE, "layout.json"), "w") as f:
        json.dump(layout, f, indent=1)

    # ---- 2. KDA rebuild ----
    NS, HV, V, K, L, R = 4, 2, 32, 32, 8, 2
    g = torch.Generator().manual_seed(1234)
    ssm = torch.zeros(NS, HV, V, K)
    v = RS.state_views(ssm, R)
    v["Sq"].copy_(torch.randint(-127, 128, (NS, HV, V, K), generator=g, dtype=torch.int32).to(torch.int8))
    v["Sk"].copy_(torch.rand(NS, HV, K, generator=g) + 0.1)
    v["Sv"].copy_(torch.rand(NS, HV, V, generator=g) + 0.1)
    v["uq"].copy_((torch.randn(NS, HV, R, K + V, generator=g) * 0.3).half())
    fake = types.SimpleNamespace(K=K, L=L, R=R,
                                 Kbuf=(torch.randn(NS, HV, L, K, generator=g) * 0.2).bfloat16(),
                                 Ubuf=torch.randn(NS, HV, L, V, generator=g).bfloat16(),
                                 Wbuf=torch.rand(NS, HV, L, generator=g),
                                 Pbuf=-torch.rand(NS, HV, K, generator=g) * 3.0,
                                 Gbuf=(0.5 + 0.5 * torch.rand(NS, HV, L, K, generator=g)).half(),
                                 hcnt=torch.tensor([[0, 3], [8, 5], [1, 7], [4, 2]], dtype=torch.int32))
    fake.views = lambda s: v
    for n in range(NS):                                   # entries at and after hcnt carry weight 0, as the kernels leave them
        for hh in range(HV):
            fake.Wbuf[n, hh, int(fake.hcnt[n, hh]):] = 0.0
    sl = torch.tensor([1, 3, 2])
    S = RS.LeapQuantState._kda_rebuild(fake, ssm, sl)
    np.savez_compressed(os.path.join(HERE, "kda_rebuild.npz"), ssm=ssm.numpy(), Kbuf=bits16(fake.Kbuf), Ubuf=bits16(fake.Ubuf),
                        Wbuf=fake.Wbuf.numpy(), Pbuf=fake.Pbuf.numpy(), Gbuf=bits16(fake.Gbuf), hcnt=fake.hcnt.numpy(),
                        sl=sl.numpy(), S=S.numpy(), dims=np.array([NS, HV, V, K, L, R]))

    # ---- 3. KDA checkpoint (lowrank_factor supplied by the oracle) ----
    RK.lowrank_factor = lambda x, r, iters=3: O.lowrank_factor(x, r, iters)
    ssm2 = torch.randn(NS, HV, V, K, generator=g)
    ssm2[1, 0, 3, :] *= 40.0
    ssm2[2, 1, :, 5] *= 25.0
    src = ssm2.clone()
    v2 = RS.state_views(ssm2, R)
    fake2 = types.SimpleNamespace(K=K, L=L, R=R, Wbuf=torch.ones(NS, HV, L), Pbuf=torch.ones(NS, HV, K),
                                  Gbuf=torch.zeros(NS, HV, L, K).half(), hcnt=torch.full((NS, HV), 3, dtype=torch.int32))
    fake2.views = lambda s: v2
    sl2 = torch.tensor([1, 2])
    RS.LeapQuantState._kda_checkpoint(fake2, ssm2, sl2)
    np.savez_compressed(os.path.join(HERE, "kda_checkpoint.npz"), src=src.numpy(), out=ssm2.numpy(), sl=sl2.numpy(),
                        Wbuf=fake2.Wbuf.numpy(), Pbuf=fake2.Pbuf.numpy(), Gbuf=bits16(fake2.Gbuf), hcnt=fake2.hcnt.numpy(),
                        dims=np.array([NS, HV, V, K, L, R]))
    print("wrote layout.json, kda_rebuild.npz, kda_checkpoint.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
