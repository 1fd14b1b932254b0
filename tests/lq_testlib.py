"""Shared helpers of the test-suite: build identical quantized states for the CPU oracle and for the CUDA library."""
import torch

from oracle import lq_oracle as O


class CpuSide:
    """State tensor + window buffers on the CPU, driven by the oracle."""

    def __init__(self, NS, HV, H, K, V, L, R, kda=False, glb=0.0, slot_pad=0):
        self.NS, self.HV, self.H, self.K, self.V, self.L, self.R, self.kda, self.glb = NS, HV, H, K, V, L, R, kda, glb
        SS = HV * V * K + slot_pad
        self.store = torch.zeros(NS * SS + 64)
        self.ssm = self.store[16:16 + NS * SS].view(NS, SS)[:, :HV * V * K].view(NS, HV, V, K)
        self.bufs = O.Buffers(NS, HV, K, V, L, R, kda)
        self.v = O.state_views(self.ssm, R)

    def quantize(self, idx):
        b, v = self.bufs, self.v
        if self.kda:
            O.kda_checkpoint(self.ssm, v["Sq"], v["Sk"], v["Sv"], v["uq"], b.Wbuf, b.Pbuf, b.Gbuf, b.hcnt,
                             idx[idx > 0].long(), self.R)
        else:
            O.quantize(self.ssm, v["Sq"], v["Sk"], v["Sv"], v["uq"], b.Wbuf, b.Pbuf, b.hcnt, b.Q0, idx)

    def dequantize(self, idx):
        b, v = self.bufs, self.v
        if self.kda:
            sl = idx[idx > 0].long()
            self.ssm[sl] = O.kda_rebuild(v["Sq"], v["Sk"], v["Sv"], v["uq"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.Gbuf, b.hcnt, sl)
        else:
            O.dequantize(self.ssm, v["Sq"], v["Sk"], v["Sv"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.hcnt, v["uq"], idx)

    def step(self, mixed, a, b_, A_log, dt_bias, idx, o):
        b, v = self.bufs, self.v
        if self.kda:
            O.kda_step(v["Sq"], v["Sk"], v["Sv"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.Gbuf, b.hcnt, mixed, a, b_, A_log,
                       dt_bias, v["uq"], idx, o, self.H, glb=self.glb)
        else:
            O.gdn_step(v["Sq"], v["Sk"], v["Sv"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.hcnt, mixed, a, b_, A_log, dt_bias,
                       v["uq"], idx, o, self.H)

    def flush(self, idx):
        b, v = self.bufs, self.v
        return O.flush(v["Sq"], v["Sk"], v["Sv"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.Gbuf if self.kda else None, b.hcnt,
                       v["uq"], b.Q0, idx, kda=self.kda)

    def decode(self, mixed, a, b_, A_log, dt_bias, idx, o):
        self.step(mixed, a, b_, A_log, dt_bias, idx, o)
        return self.flush(idx)

    def full_state(self, slots):
        b, v = self.bufs, self.v
        return O.full_state(v["Sq"], v["Sk"], v["Sv"], v["uq"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.Gbuf, b.hcnt,
                            torch.as_tensor(slots), self.kda)


class GpuSide:
    """The same state on a CUDA device, driven through leapquant_b200.state.LeapQuantState (C ABI underneath)."""

    def __init__(self, cpu, device="cuda"):
        from leapquant_b200.state import LeapQuantState
        self.cpu_shape = cpu
        self.store = cpu.store.to(device)
        NS, HV, V, K = cpu.ssm.shape
        SS = cpu.ssm.stride(0)
        self.ssm = self.store[16:16 + NS * SS].view(NS, SS)[:, :HV * V * K].view(NS, HV, V, K)
        self.st = LeapQuantState(self.ssm, cpu.H, kda=cpu.kda, gate_lower_bound=cpu.glb, L=cpu.L, R=cpu.R)
        self.device = device
        self.sync_from(cpu)

    def sync_from(self, cpu):
        """Overwrite the device state with the oracle's: checkpoint bytes and every window buffer."""
        self.store.copy_(cpu.store)
        st, b = self.st, cpu.bufs
        for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf", "hcnt"):
            getattr(st, name).copy_(getattr(b, name))
        if cpu.kda:
            st.Gbuf.copy_(b.Gbuf)

    def views_cpu(self):
        """CPU copies of the checkpoint views and the window buffers."""
        ssm = torch.zeros_like(self.cpu_shape.store)
        ssm.copy_(self.store)
        NS, HV, V, K = self.ssm.shape
        SS = self.ssm.stride(0)
        s4 = ssm[16:16 + NS * SS].view(NS, SS)[:, :HV * V * K].view(NS, HV, V, K)
        v = O.state_views(s4, self.st.R)
        st = self.st
        bufs = dict(Kbuf=st.Kbuf.cpu(), Ubuf=st.Ubuf.cpu(), Wbuf=st.Wbuf.cpu(), Pbuf=st.Pbuf.cpu(), Gbuf=st.Gbuf.cpu(),
                    hcnt=st.hcnt.cpu())
        return s4, v, bufs

    def full_state(self, slots):
        s4, v, b = self.views_cpu()
        return O.full_state(v["Sq"], v["Sk"], v["Sv"], v["uq"], b["Kbuf"], b["Ubuf"], b["Wbuf"], b["Pbuf"], b["Gbuf"],
                            b["hcnt"], torch.as_tensor(slots), self.st.kda)


def random_states(NS, HV, V, K, seed, scale=0.1):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(NS, HV, V, K, generator=g) * scale


def assert_close(a, b, rtol, atol, what):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    bad = err > lim
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {bad.numel()} elements off; max err {float(err.max()):.3e} "
                                 f"(limit there {float(lim.flatten()[err.argmax()]):.3e}); ref max {float(b.abs().max()):.3e}")
