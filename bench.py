"""Benchmark of the quantized-state decode path (step + window flush) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload gdn|kda] [--batch B] [--only-main]

Workload (default): the batched GDN decode of a Qwen3-Next-like layer -- 16 key / 32 value heads, d_k = d_v = 128,
B = 256 independent sequences per GPU, window L = 64, R = 4 Compensator Tokens, bf16 q/k/v, INT8 state with fp32
scales.  One bench "step" is one decode step of the whole batch: ONE launch of the fused decode kernel (the step of every
head plus the flush of the heads whose window fills).  Inputs are seeded synthetic tensors.

Fill levels are STAGGERED, as on a serving engine whose sequences arrive at different times: sequence n starts with
n mod L live window entries, so every step reads the window-average number of bytes and flushes B * HV / L heads, and any
run of steps is representative whatever --steps is.  The timed region is a CUDA graph of L steps replayed until at least
--steps steps and 0.5 s have been timed; `steps` in the output is the number actually timed.

Prints ONE JSON line.  `value`: (sequence, value-head) decode steps per second, inputs resident in HBM.  `e2e`: the same
through LeapQuantState.decode with each step's inputs copied from pinned host memory and the output copied back inside
the timed region.  `roofline`: the decode kernel over the timed region (algorithmic bytes of the fill levels that were
timed / CUDA-event time).  Further keys: `parity_check` (a decode step of the whole batch after the timed region against
the CPU oracle), `step_kernel` and `flush` (the two halves alone, lock-step windows), `lockstep` (all heads flush on the
same step), `prefill_round_trip`, `kda` (the KDA layer: 32 heads, B = 128, L = 32, R = 8, and the isolated quantize on
outlier states), `batch_sweep` (B = 1 ... 256), `config3` (48 layers x 32 heads, 1 024 sequences split over the GPUs),
`cpu_baseline` (the CPU oracle on the host cores).
With N > 1 (torchrun) every rank runs its own B sequences on its own GPU (weak scaling, no communication on the state
path) and the time is the maximum over ranks.
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K = V = 128
WORKLOADS = {
    "gdn": dict(name="gdn_decode_H16_HV32_d128_L64_R4", H=16, HV=32, L=64, R=4, B=256, kda=False),
    "kda": dict(name="kda_decode_H32_HV32_d128_L32_R8", H=32, HV=32, L=32, R=8, B=128, kda=True),
}
# DRAM bytes (read + write) per algorithmic byte of the fused decode kernel on the staggered batch, from the ncu captures
# summarised under profiles/ (decode_gdn_B256_ncu.md: 302.1 MB + 10.0 MB against 313.5 MB algorithmic;
# decode_kda_B128_ncu.md: 145.5 MB + 6.5 MB against 159.6 MB).  `roofline.traffic` scales the live algorithmic bytes per
# launch by this ratio.
NCU_TRAFFIC_RATIO = {"gdn": 1.00, "kda": 0.95}
MIN_TIMED_S = 0.5


def step_bytes(h, L, R, gqa, kda):
    """Algorithmic bytes of one (sequence, value head) decode step with h live window entries."""
    ck = V * K + 4 * (K + V) + 2 * R * (K + V)
    win = h * (2 * K + 2 * V + 4 + (2 * K if kda else 0))
    tok = 2 * V + 4 * K // gqa + 2 * V + (2 * K + 2 * V)            # v, q + k, out, appended rows
    if kda:
        tok += 2 * K + 2 + 2 * K + 8 * K + 8                         # gate row a, b, appended Gbuf row, Pbuf r/w, hcnt
    else:
        tok += 4 + 4 * (h + 1) + 8 + 8                               # gates, W rewrite, Pbuf r/w, hcnt
    return ck + win + tok


def flush_bytes(L, R, kda):
    ck = V * K + 4 * (K + V) + 2 * R * (K + V)
    rd = ck + L * (2 * K + 2 * V + 4 + (2 * K if kda else 0)) + (4 * K if kda else 4)
    wr = ck + 4 * L + (4 * K + 2 * K * L if kda else 4) + 4
    return rd + wr


def window_bytes_per_head_step(L, R, gqa, kda):
    """Mean over one window: the steps at h = 0 .. L-1 plus one flush, per step."""
    return (sum(step_bytes(h, L, R, gqa, kda) for h in range(L)) + flush_bytes(L, R, kda)) / L


def roundtrip_bytes(R):
    return 4 * V * K + K * V + 4 * (K + V) + 2 * R * (K + V)


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU every 100 ms through NVML (read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._halt = index, [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = get(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._halt.wait(0.1)

    def finish(self):
        self._halt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def visible_to_nvml_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ---------------------------------------------------------------------------------------------------------------------
# reference arm / cpu baseline: the CPU oracle (the reference has no CPU implementation of this path)
# ---------------------------------------------------------------------------------------------------------------------
def cpu_oracle_rate(wl, steps, warmup, nseq=8):
    """Head-steps/s of the CPU oracle on `nseq` sequences of the workload's layer, all host threads."""
    from oracle import lq_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    H, HV, L, R, kda = wl["H"], wl["HV"], wl["L"], wl["R"], wl["kda"]
    NS = nseq + 1
    g = torch.Generator().manual_seed(0)
    ssm = torch.randn(NS, HV, V, K, generator=g) * 0.1
    v = O.state_views(ssm, R)
    b = O.Buffers(NS, HV, K, V, L, R, kda)
    idx = torch.arange(1, nseq + 1, dtype=torch.int32)
    if kda:
        O.kda_checkpoint(ssm, v["Sq"], v["Sk"], v["Sv"], v["uq"], b.Wbuf, b.Pbuf, b.Gbuf, b.hcnt, idx.long(), R)
    else:
        O.quantize(ssm, v["Sq"], v["Sk"], v["Sv"], v["uq"], b.Wbuf, b.Pbuf, b.hcnt, b.Q0, idx)
    per = min(steps + warmup, L)
    mixed, a, bb, A_log, dtb = O.synth_inputs(nseq, H, HV, K, V, per, 1, kda=kda)
    o = torch.zeros(nseq, HV, V, dtype=torch.bfloat16)

    def one(t):
        i = t % per
        if kda:
            O.kda_step(v["Sq"], v["Sk"], v["Sv"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.Gbuf, b.hcnt, mixed[i], a[i], bb[i],
                       A_log, dtb, v["uq"], idx, o, H)
        else:
            O.gdn_step(v["Sq"], v["Sk"], v["Sv"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.hcnt, mixed[i], a[i], bb[i], A_log, dtb,
                       v["uq"], idx, o, H)
        O.flush(v["Sq"], v["Sk"], v["Sv"], b.Kbuf, b.Ubuf, b.Wbuf, b.Pbuf, b.Gbuf if kda else None, b.hcnt, v["uq"], b.Q0,
                idx, kda=kda)

    for t in range(warmup):
        one(t)
    t0 = time.perf_counter()
    for t in range(warmup, warmup + steps):
        one(t)
    dt = time.perf_counter() - t0
    return nseq * HV * steps / dt, dt, (f"{nseq} sequences x {HV} heads, {steps} decode steps (step + flush, one whole window "
                                        f"from empty), torch CPU oracle")


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    L = wl["L"]
    steps = L * max(1, min(-(-args.steps // L), 2))            # whole windows, so that the flush is inside the sample
    warm = max(3, min(args.warmup, 8))
    rate, dt, sample = cpu_oracle_rate(wl, steps, warm)
    cores = os.cpu_count() or 1
    line = {"impl": "reference", "metric": "int8_state_decode_head_steps_per_s", "value": rate, "unit": "head-steps/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": 1e3 * dt / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"], "note": "the reference has no CPU implementation of this path; this is the "
                       "CPU restatement (oracle) of its kernel arithmetic on the host cores, on a bounded sample"},
            "cpu_baseline": {"value": rate, "unit": "head-steps/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": rate, "unit": "head-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------------------------------------------------
def synth_inputs(N, H, HV, steps, seed, kda):
    """Seeded per-step inputs: q, k ~ N(0,1) l2-normalised per head, v ~ N(0,1), b ~ N(0,1), raw gate a ~ N(0,1) with
    A_log = 0 and dt_bias = 0 (alpha = exp(-softplus a)); bf16, stacked on dim 0."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(steps, N, H, K, generator=g)
    k = torch.randn(steps, N, H, K, generator=g)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(steps, N, HV, V, generator=g)
    mixed = torch.cat([q.reshape(steps, N, -1), k.reshape(steps, N, -1), v.reshape(steps, N, -1)], -1).to(torch.bfloat16)
    a = torch.randn(steps, N, HV, K if kda else 1, generator=g).to(torch.bfloat16)
    a = a if kda else a[..., 0].contiguous()
    b = torch.randn(steps, N, HV, generator=g).to(torch.bfloat16)
    return mixed, a, b, torch.zeros(HV), (torch.zeros(HV, K) if kda else torch.zeros(HV))


def device_inputs(N, H, HV, steps, seed, kda, device):
    """The same distributions generated on the device (for the large secondary workloads; values differ from the host
    generator's, distributions do not)."""
    g = torch.Generator(device=device).manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, device=device)
    q, k = r(steps, N, H, K), r(steps, N, H, K)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    mixed = torch.cat([q.reshape(steps, N, -1), k.reshape(steps, N, -1), r(steps, N, HV * V)], -1).to(torch.bfloat16)
    a = r(steps, N, HV, K).to(torch.bfloat16) if kda else r(steps, N, HV).to(torch.bfloat16)
    b = r(steps, N, HV).to(torch.bfloat16)
    z = lambda *s: torch.zeros(*s, device=device)
    return mixed, a, b, z(HV), (z(HV, K) if kda else z(HV))


class Layer:
    """One layer's quantized state for B sequences on the current device, plus one window period (L steps) of inputs."""

    def __init__(self, wl, B, device, seed, host_io=True, device_rng=False, inputs=None):
        from leapquant_b200.state import LeapQuantState
        self.wl, self.B, self.device = wl, B, device
        H, HV, L, R, kda = wl["H"], wl["HV"], wl["L"], wl["R"], wl["kda"]
        NS = B + 9
        self.ssm = torch.empty(NS, HV, V, K, device=device)
        if device_rng:
            gd = torch.Generator(device=device).manual_seed(seed)
            for s0 in range(0, NS, 256):
                n = min(256, NS - s0)
                self.ssm[s0:s0 + n] = torch.randn(n, HV, V, K, generator=gd, device=device) * 0.1
        else:
            g = torch.Generator(device="cpu").manual_seed(seed)
            for s0 in range(0, NS, 64):                         # seeded fp32 states, generated in chunks
                n = min(64, NS - s0)
                self.ssm[s0:s0 + n] = (torch.randn(n, HV, V, K, generator=g) * 0.1).to(device)
        self.st = LeapQuantState(self.ssm, H, kda=kda, L=L, R=R, nmax=B)
        self.idx = torch.arange(1, B + 1, dtype=torch.int32, device=device)
        self.st.quantize(self.ssm, self.idx)
        self.period = L
        if inputs is not None:                                  # inputs shared with other layers of a model
            self.mixed, self.a, self.b, self.A_log, self.dtb = inputs
        elif device_rng:
            self.mixed, self.a, self.b, self.A_log, self.dtb = device_inputs(B, H, HV, L, seed + 1, kda, device)
        else:
            mixed, a, b, A_log, dtb = synth_inputs(B, H, HV, L, seed + 1, kda)
            self.mixed, self.a, self.b = mixed.to(device), a.contiguous().to(device), b.to(device)
            self.A_log, self.dtb = A_log.to(device), dtb.to(device)
        self.out = torch.zeros(B, HV, V, dtype=torch.bfloat16, device=device)
        self.graph = None
        self.staged = None
        if host_io:
            # pinned host copies of the inputs, the three tensors of a step back to back so that one copy moves them
            from leapquant_b200.host_io import HostStagedDecoder
            self.h_slab, hv = HostStagedDecoder.host_slab(mixed[0], a[0].contiguous(), b[0], steps=L)
            for i in range(L):
                hv[i][0].copy_(mixed[i]); hv[i][1].copy_(a[i]); hv[i][2].copy_(b[i])
            self.h_mixed, self.h_a, self.h_b = [x[0] for x in hv], [x[1] for x in hv], [x[2] for x in hv]
            self.h_out = torch.zeros(B, HV, V, dtype=torch.bfloat16).pin_memory()
            self.staged = HostStagedDecoder(self.st, self.ssm, self.A_log, self.dtb, self.idx, self.h_mixed[0], self.h_a[0],
                                            self.h_b[0], self.h_out)

    def decode_resident(self, t, idx=None):
        i = t % self.period
        self.st.decode(self.ssm, self.mixed[i], self.a[i], self.b[i], self.A_log, self.dtb, self.idx if idx is None else idx,
                       self.out)

    def stagger(self):
        """From all windows empty to sequence n holding n mod L entries: L - 1 decode steps in which row n takes part only
        while t < n mod L (the other rows are padding rows of the call)."""
        L = self.period
        phase = (torch.arange(self.B, device=self.device) % L).to(torch.int32)
        for t in range(L - 1):
            self.decode_resident(t, torch.where(phase > t, self.idx, torch.zeros_like(self.idx)))

    def capture(self):
        """One window period (L decode steps, one launch each) as a CUDA graph."""
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            for t in range(self.period):
                self.decode_resident(t)
        return self.graph

    def to_lockstep(self):
        """All windows empty again (the prefill round trip: dequantize to fp32, quantize back); returns the two times."""
        deq = timed(lambda: self.st.dequantize(self.ssm, self.idx))
        qnt = timed(lambda: self.st.quantize(self.ssm, self.idx))
        return deq, qnt

    def decode_host(self, t):
        """One step with host-resident inputs and output: the three input tensors come from pinned host memory and the
        step's output goes back to pinned host memory, staged by HostStagedDecoder (copies of neighbouring steps overlap
        the kernels; every step still moves its own bytes both ways)."""
        i = t % self.period
        self.staged.submit(self.h_mixed[i], self.h_a[i], self.h_b[i], self.h_out)

    def step_only(self, t):
        i = t % self.period
        st, v = self.st, self.st.views(self.ssm)
        args = (self.mixed[i], self.a[i].reshape(self.B, st.HV, -1), self.b[i], self.A_log, self.dtb.reshape(st.HV, -1),
                v["uq"], self.idx, self.out)
        if st.kda:
            st.kstep(v["q32"], v["Sk"], v["Sv"], v["skv"], st.Kbuf, st.Ubuf, st.Wbuf, st.Pbuf, st.Gbuf, st.hcnt, *args)
        else:
            st.kstep(v["q32"], v["Sk"], v["Sv"], v["skv"], st.Kbuf, st.Ubuf, st.Wbuf, st.Pbuf, st.hcnt, *args)

    def flush_only(self):
        st, v = self.st, self.st.views(self.ssm)
        st.kflush(v["q32"], v["Sk"], v["Sv"], v["skv"], st.Kbuf, st.Ubuf, st.Wbuf, st.Pbuf, st.Gbuf if st.kda else st.Gd,
                  st.hcnt, v["sq16"], v["uq"], st.Q0, self.idx)

    def h2d_bytes(self):
        return sum(t[0].numel() * t[0].element_size() for t in (self.h_mixed, self.h_a, self.h_b))

    def d2h_bytes(self):
        return self.h_out.numel() * self.h_out.element_size()


def timed(fn, stream=None):
    stream = stream or torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    fn()
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e-3


def replay_timed(graph, min_windows, min_seconds, barrier=None):
    """Replays the window graph: a calibration replay, then `reps` replays timed as one region (>= min_windows, >= min_seconds)."""
    graph.replay()
    t1 = timed(graph.replay)
    reps = max(min_windows, int(math.ceil(min_seconds / max(t1, 1e-6))))
    if barrier:
        barrier()

    def body():
        for _ in range(reps):
            graph.replay()

    return timed(body), reps


def parity_check(layer, rows):
    """One more decode step of the WHOLE batch (the launch shape that was timed) from the state the timed region left behind,
    against the CPU oracle on a few rows whose device state is copied to the host bit for bit.  Returns (ok, detail)."""
    from oracle import lq_oracle as O
    st, wl = layer.st, layer.wl
    H, HV, L, R, kda = wl["H"], wl["HV"], wl["L"], wl["R"], wl["kda"]
    rows = [r for r in rows if r < layer.B]
    slots = layer.idx[rows].long()
    n = len(rows)
    # oracle-side copies: slot i + 1 of a small state tensor holds the device's slot of row rows[i]
    ssm_c = torch.zeros(n + 1, HV, V, K)
    ssm_c[1:] = layer.ssm[slots].cpu()
    bufs = O.Buffers(n + 1, HV, K, V, L, R, kda)
    for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf", "hcnt") + (("Gbuf",) if kda else ()):
        getattr(bufs, name)[1:] = getattr(st, name)[slots].cpu()
    vc = O.state_views(ssm_c, R)
    t = 7 % layer.period
    idx_c = torch.arange(1, n + 1, dtype=torch.int32)
    o_c = torch.zeros(n, HV, V, dtype=torch.bfloat16)
    mixed, a, b = layer.mixed[t][rows].cpu(), layer.a[t][rows].cpu(), layer.b[t][rows].cpu()
    A_log, dtb = layer.A_log.cpu(), layer.dtb.cpu()
    h_before = bufs.hcnt[1:].clone()
    if kda:
        O.kda_step(vc["Sq"], vc["Sk"], vc["Sv"], bufs.Kbuf, bufs.Ubuf, bufs.Wbuf, bufs.Pbuf, bufs.Gbuf, bufs.hcnt, mixed, a, b,
                   A_log, dtb, vc["uq"], idx_c, o_c, H)
    else:
        O.gdn_step(vc["Sq"], vc["Sk"], vc["Sv"], bufs.Kbuf, bufs.Ubuf, bufs.Wbuf, bufs.Pbuf, bufs.hcnt, mixed, a, b, A_log, dtb,
                   vc["uq"], idx_c, o_c, H)
    u_c = torch.stack([bufs.Ubuf[1 + i, torch.arange(HV), h_before[i].long().clamp(max=L - 1)] for i in range(n)]).float()
    O.flush(vc["Sq"], vc["Sk"], vc["Sv"], bufs.Kbuf, bufs.Ubuf, bufs.Wbuf, bufs.Pbuf, bufs.Gbuf if kda else None, bufs.hcnt,
            vc["uq"], bufs.Q0, idx_c, kda=kda)
    layer.decode_resident(t)
    torch.cuda.synchronize()
    o_g = layer.out[rows].cpu().float()
    u_g = torch.stack([st.Ubuf[slots[i], torch.arange(HV, device=layer.device), h_before[i].long().clamp(max=L - 1).to(layer.device)]
                       for i in range(n)]).cpu().float()
    oc = o_c.float()
    scale = float(oc.abs().max())
    err_o = float((o_g - oc).abs().max())
    err_u = float((u_g - u_c).abs().max())
    lim_o = 8e-3 * scale + 1e-4                                   # one bf16 ulp of the largest output
    lim_u = 8e-3 * float(u_c.abs().max()) + 2e-4
    hc_ok = bool(torch.equal(st.hcnt[slots].cpu(), bufs.hcnt[1:]))
    # the state after the step -- and, for the rows whose window filled, after the flush: the live fp32 state that checkpoint
    # and window stand for, device against oracle (a flush that lost or mangled a window shows here, not in this step's output)
    ssm_g = torch.zeros(n + 1, HV, V, K)
    ssm_g[1:] = layer.ssm[slots].cpu()
    bufs_g = O.Buffers(n + 1, HV, K, V, L, R, kda)
    for name in ("Kbuf", "Ubuf", "Wbuf", "Pbuf", "hcnt") + (("Gbuf",) if kda else ()):
        getattr(bufs_g, name)[1:] = getattr(st, name)[slots].cpu()
    vg = O.state_views(ssm_g, R)
    full = lambda v_, b_: O.full_state(v_["Sq"], v_["Sk"], v_["Sv"], v_["uq"], b_.Kbuf, b_.Ubuf, b_.Wbuf, b_.Pbuf,
                                       b_.Gbuf if kda else None, b_.hcnt, idx_c, kda)
    s_c, s_g = full(vc, bufs), full(vg, bufs_g)
    err_s = float((s_g - s_c).norm() / s_c.norm().clamp_min(1e-30))
    lim_s = 5e-4                                                 # (observed 6e-5 .. 8e-5; the 8-bit checkpoint itself is ~1e-2 from the fp32 state)
    ok = err_o <= lim_o and err_u <= lim_u and hc_ok and err_s <= lim_s
    return ok, {"rows": rows, "heads_flushed_in_check": int((h_before == L - 1).sum()), "max_abs_err_out": err_o,
                "limit_out": lim_o, "max_abs_err_appended_u": err_u, "limit_u": lim_u, "window_counters_equal": hc_ok,
                "state_rel_err_after_step_and_flush": err_s, "limit_state": lim_s}


def measure_staggered(layer, steps, min_seconds, barrier=None):
    """Staggered fill levels, graph of one window period replayed.  Returns (seconds, steps timed, reps)."""
    L = layer.period
    layer.stagger()
    layer.capture()
    nwin = max(1, -(-steps // L))
    dt, reps = replay_timed(layer.graph, nwin, min_seconds, barrier)
    return dt, reps * L, reps


def secondary_layer_numbers(layer, peak, reps_step=3):
    """The prefill round trip, the lock-step window, the step kernel alone and the flush alone, on a layer whose main
    measurement is done.  Leaves every window empty."""
    wl, B = layer.wl, layer.B
    L, HV, R, kda = wl["L"], wl["HV"], wl["R"], wl["kda"]
    gqa = HV // wl["H"]
    st = layer.st
    st.dequantize(layer.ssm, torch.zeros(1, dtype=torch.int32, device=layer.device))      # loads the kernel (null slot: no work)
    torch.cuda.synchronize()
    live_deq_s, _ = layer.to_lockstep()                          # windows as the main measurement left them (every fill level): live
    for t in range(3):
        layer.decode_resident(t)                                 # a few live entries for the dequantize to fold in
    deq_s, qnt_s = layer.to_lockstep()
    deq0_s, _ = layer.to_lockstep()                              # windows empty: a slot between two chunks of its prefill
    rt = B * HV * roundtrip_bytes(R)
    out = {"prefill_round_trip": {"dequantize_ms": 1e3 * deq_s, "quantize_ms": 1e3 * qnt_s,
                                  "dequantize_gbs": rt / deq_s / 1e9, "quantize_gbs": rt / qnt_s / 1e9,
                                  "dequantize_frac_of_measured_hbm": rt / deq_s / 1e9 / peak,
                                  "quantize_frac_of_measured_hbm": rt / qnt_s / 1e9 / peak,
                                  "bytes_per_head": roundtrip_bytes(R),
                                  "dequantize_live_windows_ms": 1e3 * live_deq_s,
                                  "dequantize_empty_windows_ms": 1e3 * deq0_s,
                                  "dequantize_empty_windows_frac_of_measured_hbm": rt / deq0_s / 1e9 / peak,
                                  "note": "dequantize_ms: windows with 3 entries; dequantize_empty_windows_ms: no live entry (a slot "
                                          "between two chunks of its prefill); dequantize_live_windows_ms: the staggered windows of "
                                          "the decode batch (a mixed prefill + decode step), first call"}}
    # lock-step: every head flushes on the same step (the graph is the one captured for the staggered run)
    dt_l, reps_l = replay_timed(layer.graph, 1, 0.1)
    amort = window_bytes_per_head_step(L, R, gqa, kda)
    out["lockstep"] = {"ms_per_step": 1e3 * dt_l / (reps_l * L), "value": B * HV * reps_l * L / dt_l, "steps": reps_l * L,
                       "frac_of_measured_hbm": B * HV * reps_l * L / dt_l * amort / 1e9 / peak,
                       "note": "all windows in phase: every head flushes on the same step, once per window"}
    # the step kernel alone over one lock-step window (h = 0 .. L-1), state restored between repetitions
    bufs = (layer.ssm, st.Kbuf, st.Ubuf, st.Wbuf, st.Pbuf, st.hcnt) + ((st.Gbuf,) if kda else ())
    snap = [t.clone() for t in bufs]
    tk = 0.0
    for r in range(reps_step + 1):
        for dst, src in zip(bufs, snap):
            dst.copy_(src)
        torch.cuda.synchronize()

        def body_k():
            for t in range(L):
                layer.step_only(t)

        x = timed(body_k)
        if r > 0:
            tk += x
    step_ms = 1e3 * tk / (reps_step * L)
    alg_step = B * HV * sum(step_bytes(h, L, R, gqa, kda) for h in range(L)) / L
    out["step_kernel"] = {"kernel": "step_pipelined_kernel (no flush tail)", "ms_per_launch": step_ms,
                          "alg_bytes_per_launch": alg_step, "achieved": alg_step / (step_ms * 1e-3) / 1e9, "unit": "GB/s",
                          "frac": alg_step / (step_ms * 1e-3) / 1e9 / peak, "frac_of_8tbs": alg_step / (step_ms * 1e-3) / 1e9 / 8000.0,
                          "note": "one lock-step window h = 0 .. L-1, %d repetitions" % reps_step}
    # the flush kernel alone: every head due (state left by the last pass above), then nothing due
    flush_all_s = timed(layer.flush_only)
    flush_idle_s = timed(lambda: [layer.flush_only() for _ in range(20)]) / 20
    out["flush"] = {"all_due_ms": 1e3 * flush_all_s, "none_due_ms": 1e3 * flush_idle_s, "heads": B * HV,
                    "all_due_gbs": B * HV * flush_bytes(L, R, kda) / flush_all_s / 1e9,
                    "all_due_frac_of_measured_hbm": B * HV * flush_bytes(L, R, kda) / flush_all_s / 1e9 / peak}
    for dst, src in zip(bufs, snap):
        dst.copy_(src)
    del snap
    return out


def conv_and_fp32_baseline(wl, B, device, peak, graph_steps=16):
    """Two figures for the Gated DeltaNet layer, staggered fill levels, CUDA graphs of `graph_steps` steps:
    (a) the decode step with the conv1d update fused in (one launch) against the standalone conv kernel followed by decode;
    (b) the serving engine's own path on an fp32 state -- vLLM's causal_conv1d_update + packed-decode kernels, the path the
        reference plugin replaces -- when that vLLM is importable: the kernel-level speed-up the reference publishes is
        measured against this."""
    from leapquant_b200.kernels import make_conv1d_update
    H, HV, L = wl["H"], wl["HV"], wl["L"]
    C = 2 * H * K + HV * V
    ly = Layer(wl, B, device, seed=500, host_io=False)
    NS = ly.ssm.shape[0]
    g = torch.Generator(device=device).manual_seed(9)
    x = (torch.randn(L, B, C, generator=g, device=device) * 0.7).to(torch.bfloat16)
    conv_store = torch.randn(NS, 3, C, generator=g, device=device).to(torch.bfloat16)       # (slot, tap, channel)
    conv_state = conv_store.transpose(-1, -2)
    w = (torch.randn(C, 4, generator=g, device=device) * 0.5).to(torch.bfloat16)
    bias = torch.zeros(C, dtype=torch.bfloat16, device=device)
    for t in range(3):
        ly.decode_resident(t)
    ly.to_lockstep()
    ly.stagger()
    conv = make_conv1d_update(NS, C)
    mixed = torch.zeros(B, C, dtype=torch.bfloat16, device=device)

    def fused(t):
        ly.st.conv_one_launch = True
        ly.st.decode_conv(ly.ssm, x[t % L], conv_state, w, bias, ly.a[t % L], ly.b[t % L], ly.A_log, ly.dtb, ly.idx, ly.out)
        ly.st.conv_one_launch = False

    def unfused(t):
        conv(x[t % L], conv_state, w, bias, ly.idx, mixed)
        ly.st.decode(ly.ssm, mixed, ly.a[t % L], ly.b[t % L], ly.A_log, ly.dtb, ly.idx, ly.out)

    def time_graph(fn, nsteps):
        for t in range(2):
            fn(t)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for t in range(nsteps):
                fn(t)
        dt, reps = replay_timed(gr, 1, 0.1)
        return dt / (reps * nsteps)

    out = {"batch": B}
    tf, tu = time_graph(fused, L), time_graph(unfused, L)
    out["conv_and_decode"] = {"ms_per_step_one_launch": 1e3 * tf, "ms_per_step_two_launches": 1e3 * tu,
                              "default": "two launches (conv1d update kernel, then decode)",
                              "note": "replayed from a CUDA graph; the single launch pays where launches are issued one by one"}
    try:
        from vllm.model_executor.layers.fla.ops.fused_recurrent import fused_recurrent_gated_delta_rule_packed_decode as eng_decode
        from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update as eng_conv
        ssm32 = torch.randn(NS, HV, V, K, generator=g, device=device) * 0.1
        o32 = torch.zeros(B, 1, HV, V, dtype=torch.bfloat16, device=device)
        a16, b16 = ly.a.contiguous(), ly.b.contiguous()

        def engine(t):
            m = eng_conv(x[t % L], conv_state, w, bias, "silu", conv_state_indices=ly.idx)
            eng_decode(mixed_qkv=m, a=a16[t % L], b=b16[t % L], A_log=ly.A_log, dt_bias=ly.dtb, scale=K ** -0.5, initial_state=ssm32,
                       out=o32, ssm_state_indices=ly.idx, use_qk_l2norm_in_kernel=True)

        te = time_graph(engine, graph_steps)
        out["fp32_state_engine_kernels"] = {"ms_per_step": 1e3 * te, "head_steps_per_s": B * HV / te,
                                            "gbs": B * HV * 2 * 4 * V * K / te / 1e9, "frac_of_measured_hbm": B * HV * 2 * 4 * V * K / te / 1e9 / peak,
                                            "kernels": "vllm causal_conv1d_update + fused_recurrent_gated_delta_rule_packed_decode (Triton), fp32 state",
                                            "speedup_of_int8_conv_and_decode": te / min(tf, tu)}
    except Exception as e:                                       # the engine is not importable here: no fp32-state figure
        out["fp32_state_engine_kernels"] = {"unavailable": str(e).splitlines()[0][:160] if str(e) else type(e).__name__}
    return out


def outlier_quantize(layer, peak):
    """The isolated quantize on fp32 states drawn as N(0,1) with 1 % of the rows and of the columns scaled by 50."""
    wl, B = layer.wl, layer.B
    HV, R = wl["HV"], wl["R"]
    g = torch.Generator(device=layer.device).manual_seed(77)
    S = layer.ssm
    for s0 in range(0, S.shape[0], 64):
        n = min(64, S.shape[0] - s0)
        x = torch.randn(n, HV, V, K, generator=g, device=layer.device)
        rsel = torch.rand(n, HV, V, 1, generator=g, device=layer.device) < 0.01
        csel = torch.rand(n, HV, 1, K, generator=g, device=layer.device) < 0.01
        S[s0:s0 + n] = x * torch.where(rsel, 50.0, 1.0) * torch.where(csel, 50.0, 1.0)
    q_s = timed(lambda: layer.st.quantize(layer.ssm, layer.idx))
    by = B * HV * roundtrip_bytes(R)
    return {"heads": B * HV, "quantize_ms": 1e3 * q_s, "gbs": by / q_s / 1e9, "frac_of_measured_hbm": by / q_s / 1e9 / peak,
            "states": "N(0,1), 1 % of rows and of columns x 50", "iters": 3 if wl["kda"] else 1}


def run_config3(world, rank, device, peak, barrier):
    """48 GDN layers x 32 value heads, 1 024 sequences split over the ranks (strong scaling), staggered fill levels, one
    window period of decode steps per layer group.  On one GPU the 48 layer states (3.3 GB each at 1 024 sequences) do not
    fit next to each other, so the layers are timed in groups and the group times are added."""
    from leapquant_b200.sharding import job_times, shard_rows
    wl = WORKLOADS["gdn"]
    L, HV, R = wl["L"], wl["HV"], wl["R"]
    NL, BT = 48, 1024
    r0, r1 = shard_rows(BT, world, rank)
    Bl = r1 - r0
    # every layer has its own state; the per-step inputs (1 GB per window period at 1 024 sequences) come from four sets
    # that the layers take in turn, so that consecutive layers never read the same rows
    inputs = [device_inputs(Bl, wl["H"], HV, L, 900 + 13 * rank + i, False, device) for i in range(4)]
    per_layer = (Bl + 9) * HV * (4 * V * K + L * (2 * K + 2 * V + 4) + 8)
    free, _ = torch.cuda.mem_get_info(device)
    ngroups = -(-NL // max(1, min(NL, int((free * 0.85) // per_layer))))
    group = -(-NL // ngroups)
    total_s = 0.0
    done = 0
    for gi in range(ngroups):
        nl = min(group, NL - gi * group)
        layers = [Layer(wl, Bl, device, seed=1000 + 97 * rank + gi * group + i, host_io=False, device_rng=True,
                        inputs=inputs[(gi * group + i) % 4]) for i in range(nl)]
        for ly in layers:
            ly.stagger()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for t in range(L):
                for ly in layers:                                # a decode step of the model: every layer once
                    ly.decode_resident(t)
        graph.replay()
        barrier()
        dt = timed(graph.replay)
        total_s += dt
        done += nl
        del graph, layers
        torch.cuda.empty_cache()
    total_s = job_times([total_s], device)[0]
    amort = window_bytes_per_head_step(L, R, HV // wl["H"], False)
    units = BT * HV * NL * L
    return {"layers": NL, "sequences": BT, "sequences_per_gpu": Bl, "steps": L, "layer_groups": ngroups, "layers_per_group": group,
            "ms_per_model_step": 1e3 * total_s / L, "value": units / total_s, "unit": "head-steps/s",
            "model_decode_steps_per_s": L / total_s, "gbs_per_gpu": units / total_s * amort / 1e9 / world,
            "frac_of_measured_hbm_per_gpu": units / total_s * amort / 1e9 / world / peak, "scaling": "strong",
            "note": "all 48 layers per step; group times added when the states of all layers do not fit at once"}


def run_b200(args, wl):
    import torch.distributed as dist
    from leapquant_b200.sharding import job_times
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback (use --impl reference for the CPU oracle)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    B = args.batch or wl["B"]
    L, HV, R, kda = wl["L"], wl["HV"], wl["R"], wl["kda"]
    gqa = HV // wl["H"]
    steps, warm = args.steps, max(args.warmup, 3)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    layer = Layer(wl, B, device, seed=100 + rank)
    for t in range(max(warm, 3)):                               # eager warm-up steps (module load, first-launch set-up)
        layer.decode_resident(t)
    layer.to_lockstep()
    sampler = ClockSampler(visible_to_nvml_index(local)) if rank == 0 else None
    layer.stagger()
    layer.capture()
    nwin_w = max(1, -(-warm // L))
    for _ in range(nwin_w):
        layer.graph.replay()
    if sampler:
        sampler.start()
    nwin = max(1, -(-steps // L))
    dt, reps = replay_timed(layer.graph, nwin, MIN_TIMED_S, barrier)
    done = reps * L
    barrier()
    ok, pdetail = parity_check(layer, [0, 1, B // 2, B - 1])

    # ---- end to end through the public API with host buffers (same staggered state) ----
    per_e2e = max(dt / done, 1e-6) * 2.2                       # a host-fed step costs about twice a resident one
    e2e_steps = L * max(1, int(math.ceil(0.3 / per_e2e / L)))
    for t in range(L):                                          # warm-up: one whole window through the host path
        layer.decode_host(t)
    layer.staged.drain()
    barrier()

    def body_e2e():
        for t in range(e2e_steps):
            layer.decode_host(t)
        layer.staged.join()                                     # the timed stream waits for the last output copy

    dt_e2e = timed(body_e2e)
    barrier()
    clocks = sampler.finish() if sampler else None
    dt, dt_e2e = job_times([dt, dt_e2e], device)               # max over ranks
    units = world * B * HV * done
    value = units / dt
    e2e_value = world * B * HV * e2e_steps / dt_e2e

    extras = {}
    if not args.only_main:
        extras.update(secondary_layer_numbers(layer, peak))
        if world == 1 and not args.batch:
            other = WORKLOADS["kda" if not kda else "gdn"]
            key = "kda" if not kda else "gdn"
            layer.graph = None
            ly2 = Layer(other, other["B"], device, seed=300, host_io=False)
            for t in range(3):
                ly2.decode_resident(t)
            ly2.to_lockstep()
            dt2, done2, reps2 = measure_staggered(ly2, other["L"], 0.25)
            ok2, pd2 = parity_check(ly2, [0, other["B"] - 1])
            am2 = window_bytes_per_head_step(other["L"], other["R"], other["HV"] // other["H"], other["kda"])
            v2 = other["B"] * other["HV"] * done2 / dt2
            sec2 = secondary_layer_numbers(ly2, peak)
            extras[key] = {"workload": other["name"], "batch": other["B"], "value": v2, "unit": "head-steps/s", "steps": done2,
                           "ms_per_step": 1e3 * dt2 / done2, "alg_bytes_per_head_step": am2,
                           "roofline": {"bound": "hbm", "kernel": "step_pipelined_kernel<FUSE> (decode)", "achieved": v2 * am2 / 1e9,
                                        "peak": peak, "unit": "GB/s", "frac": v2 * am2 / 1e9 / peak, "frac_of_8tbs": v2 * am2 / 1e9 / 8000.0,
                                        "ms_per_launch": 1e3 * dt2 / done2},
                           "parity_check": "ok" if ok2 else "fail", "parity_detail": pd2, **sec2,
                           "isolated_quantize_outlier_states": outlier_quantize(ly2, peak)}
            del ly2
            torch.cuda.empty_cache()
            # the same layer at twice the batch: the launch is twice as long, filling and draining its pipeline weigh half as much
            B3 = 2 * other["B"]
            ly3 = Layer(other, B3, device, seed=310, host_io=False)
            for t in range(3):
                ly3.decode_resident(t)
            ly3.to_lockstep()
            dt3, done3, _ = measure_staggered(ly3, other["L"], 0.15)
            v3 = B3 * other["HV"] * done3 / dt3
            extras[key]["at_twice_the_batch"] = {"batch": B3, "ms_per_step": 1e3 * dt3 / done3, "value": v3,
                                                 "frac_of_measured_hbm": v3 * am2 / 1e9 / peak}
            del ly3
            torch.cuda.empty_cache()
            sweep = []
            for Bs in (1, 8, 32, 128, 256):
                lys = Layer(wl, Bs, device, seed=400 + Bs, host_io=False)
                for t in range(3):
                    lys.decode_resident(t)
                lys.to_lockstep()
                dts, dones, _ = measure_staggered(lys, L, 0.1)
                am = window_bytes_per_head_step(L, R, gqa, kda)
                vs = Bs * HV * dones / dts
                sweep.append({"batch": Bs, "ms_per_step": 1e3 * dts / dones, "value": vs, "decode_steps_per_s": dones / dts,
                              "gbs": vs * am / 1e9, "frac_of_measured_hbm": vs * am / 1e9 / peak, "steps": dones})
                del lys
                torch.cuda.empty_cache()
            extras["batch_sweep"] = sweep
            if not kda:
                extras["conv_and_fp32_state"] = [conv_and_fp32_baseline(wl, Bs, device, peak) for Bs in (32, 128, 256)]
        if not args.batch:
            layer.graph = None
            del layer
            torch.cuda.empty_cache()
            extras["config3"] = run_config3(world, rank, device, peak, barrier)

    if rank == 0:
        cpu_rate, cpu_dt, cpu_sample = cpu_oracle_rate(wl, L, 3, nseq=32) if world == 1 else (None, None, None)
        amort = window_bytes_per_head_step(L, R, gqa, kda)
        alg_launch = B * HV * amort                              # every staggered step sees each fill level B * HV / L times
        ms_step = 1e3 * dt / done
        achieved = alg_launch / (ms_step * 1e-3) / 1e9
        traffic = NCU_TRAFFIC_RATIO["kda" if kda else "gdn"]
        h2d, d2h = layer_h2d_d2h(wl, B)
        line = {"metric": "int8_state_decode_head_steps_per_s", "value": value, "unit": "head-steps/s", "n_gpus": world,
                "steps": done, "warmup": nwin_w * L + max(warm, 3), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": wl["name"], "batch_per_gpu": B, "value_heads": HV, "key_heads": wl["H"], "window": L,
                           "rank": R, "decode_steps_per_s_per_gpu": value / world / (B * HV),
                           "fill_levels": "staggered: sequence n starts with n mod %d live entries, so every step reads the "
                                          "window-average bytes and flushes %d heads" % (L, B * HV // L),
                           "alg_bytes_per_head_step": amort, "whole_path_gbs_per_gpu": value / world * amort / 1e9,
                           "whole_path_frac_of_measured_hbm": value / world * amort / 1e9 / peak,
                           "whole_path_frac_of_8tbs": value / world * amort / 1e9 / 8000.0,
                           "l2": "per-step working set %.0f MB exceeds the 126 MB L2" % (B * HV * amort / 1e6),
                           "timing": "CUDA graph of %d decode steps (one launch each) replayed %d times as one timed region of "
                                     "%.2f s; --steps %d rounded up to whole windows and to >= %.1f s" % (L, reps, dt, steps, MIN_TIMED_S),
                           "reps": reps},
                "e2e": {"value": e2e_value, "unit": "head-steps/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "steps": e2e_steps, "h2d_gbs_per_gpu": h2d * e2e_steps / dt_e2e / 1e9,
                        "d2h_gbs_per_gpu": d2h * e2e_steps / dt_e2e / 1e9,
                        "bound": "PCIe: every step moves its own inputs host->device and its output device->host; the "
                                 "state stays on the device"},
                "gpu_launches": done,
                "roofline": {"bound": "hbm", "kernel": "step_pipelined_kernel<FUSE> (decode: step + flush tail, one launch per step)",
                             "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "frac_of_8tbs": achieved / 8000.0, "traffic": (traffic * alg_launch) if traffic else None,
                             "alg_bytes_per_launch": alg_launch, "ms_per_launch": ms_step,
                             "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback"},
                "parity_check": "ok" if ok else "fail", "parity_detail": pdetail,
                "clocks": clocks}
        line.update(extras)
        if cpu_rate is not None:
            line["cpu_baseline"] = {"value": cpu_rate, "unit": "head-steps/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": cpu_sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_config4(args):
    """End-to-end tensor-parallel decode of the hybrid model (leapquant_b200/harness.py), 8-bit state against fp32 state, on the
    GPUs of this launch (TP = world size).  `--c4 small` runs a reduced model for a quick check."""
    import torch.distributed as dist
    from leapquant_b200.harness import HybridConfig, run_generation
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.c4 == "small":
        cfg = HybridConfig(hidden=1024, layers=8, gdn_key_heads=8, gdn_value_heads=16, attn_q_heads=16, attn_kv_heads=8, mlp=2048, vocab=8192)
        batch, prompt, new = 16, 256, 64
    else:
        cfg = HybridConfig()
        batch, prompt, new = 64, 4096, args.c4_new_tokens
    res = {}
    for state in ("fp32", "int8"):
        res[state] = run_generation(cfg, state, batch, prompt, new, seed=5)
        torch.cuda.empty_cache()
    if rank == 0:
        a, b = res["int8"], res["fp32"]
        line = {"metric": "tp_decode_tokens_per_s", "value": a["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                "steps": a["decode_steps_timed"], "warmup": 2, "ms_per_step": a["ms_per_decode_step"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "hybrid_tp_decode_hidden%d_L%d_gdn%d_attn%d_mlp%d_vocab%d" % (
                    cfg.hidden, cfg.layers, cfg.layers - cfg.layers // cfg.full_attention_every, cfg.layers // cfg.full_attention_every,
                    cfg.mlp, cfg.vocab), "tensor_parallel": world, "batch": batch, "prompt_len": prompt, "new_tokens": new,
                    "weights": "random init bf16", "prompts": "uniformly random token ids"},
                "int8_state": a, "fp32_state": b,
                "decode_speedup_int8_over_fp32": (b["ms_per_decode_step"] / a["ms_per_decode_step"]) if a["ms_per_decode_step"] else None,
                "first_tokens_equal": a["first_tokens"] == b["first_tokens"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def layer_h2d_d2h(wl, B):
    H, HV, kda = wl["H"], wl["HV"], wl["kda"]
    mixed = B * (2 * H * K + HV * V) * 2
    a = B * HV * (K if kda else 1) * 2
    b = B * HV * 2
    return mixed + a + b, B * HV * V * 2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gdn", choices=sorted(WORKLOADS) + ["config4"])
    ap.add_argument("--c4", default="full", choices=["full", "small"], help="config4: the full hybrid model or a reduced one")
    ap.add_argument("--c4-new-tokens", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--only-main", action="store_true", help="skip the secondary keys (kda, batch_sweep, config3, ...)")
    ap.add_argument("--step-impl", type=int, default=-1, help="debug: step kernel driver (see lq_set_option)")
    ap.add_argument("--profile-case", action="store_true",
                    help="for a profiler: quantize, stagger the fill levels (L - 1 decode launches), 4 more decode launches, "
                         "the prefill round trip once, L launches of the step kernel alone, one flush of every head, exit; "
                         "prints nothing")
    args = ap.parse_args()
    if args.workload == "config4":
        return run_config4(args)
    wl = WORKLOADS[args.workload]
    if args.step_impl >= 0:
        from leapquant_b200 import _lib
        _lib.set_option("step_impl", args.step_impl)
    if args.profile_case:
        torch.cuda.set_device(0)
        layer = Layer(wl, args.batch or wl["B"], torch.device("cuda", 0), seed=100, host_io=False)
        layer.stagger()
        for t in range(4):
            layer.decode_resident(t)
        layer.to_lockstep()
        for t in range(layer.period):                  # one window of the step kernel alone, then the flush kernel with every head due
            layer.step_only(t)
        layer.flush_only()
        torch.cuda.synchronize()
    elif args.impl == "reference":
        run_reference(args, wl)
    else:
        run_b200(args, wl)


if __name__ == "__main__":
    main()
