"""Benchmark of the quantized-state decode path (step + window flush) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload gdn|kda] [--batch B]

Workload (default): the batched GDN decode of a Qwen3-Next-like layer -- 16 key / 32 value heads, d_k = d_v = 128,
B = 256 independent sequences per GPU, window L = 64, R = 4 Compensator Tokens, bf16 q/k/v, INT8 state with fp32
scales; every head flushes every 64 steps.  One bench "step" is one decode step of the whole batch (step kernel + flush
kernel).  `--workload kda` runs the KDA layer (32 heads, B = 128, L = 32, R = 8).  Inputs are seeded synthetic tensors.

Prints ONE JSON line.  `value` is the whole-job rate in (sequence, value-head) decode steps per second with inputs
resident in HBM (one window of 64 steps captured in a CUDA graph and replayed); `e2e` is the same rate through
LeapQuantState.decode with the step's inputs copied from pinned host memory and the output copied back inside the
timed region; `roofline` times the step kernel alone over one window; `cpu_baseline` times the CPU oracle.
With N > 1 (torchrun) every rank runs its own B sequences on its own GPU (weak scaling, no communication on the state
path) and the time is the maximum over ranks.
"""
import argparse
import json
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
# DRAM bytes (read + write) of the step kernel relative to its algorithmic bytes, from the ncu capture summarised in
# profiles/step_pipelined_gdn_B128_ncu.md (150.05 MB + 5.40 MB for 4 096 programs at h = 33 vs 37 928 B algorithmic per
# program).  `roofline.traffic` scales the live algorithmic bytes per launch by this ratio.  None = not captured.
NCU_TRAFFIC_RATIO = {"gdn": 1.01, "kda": None}


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
    return (sum(step_bytes(h, L, R, gqa, kda) for h in range(L)) + flush_bytes(L, R, kda)) / L


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
    return nseq * HV * steps / dt, dt, f"{nseq} sequences x {HV} heads, {steps} decode steps (step + flush), torch CPU oracle"


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 2 * wl["L"]))
    warm = max(3, min(args.warmup, 8))
    rate, dt, sample = cpu_oracle_rate(wl, steps, warm)
    cores = os.cpu_count() or 1
    line = {"impl": "reference", "metric": "int8_state_decode_head_steps_per_s", "value": rate, "unit": "head-steps/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": 1e3 * dt / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"], "note": "the reference has no CPU implementation of this path; this is the "
                       "CPU restatement (oracle) of its kernel arithmetic on the host cores"},
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


class Layer:
    """One layer's quantized state for B sequences on the current device, plus 64 steps of device-resident inputs."""

    def __init__(self, wl, B, device, seed):
        from leapquant_b200.state import LeapQuantState
        self.wl, self.B, self.device = wl, B, device
        H, HV, L, R, kda = wl["H"], wl["HV"], wl["L"], wl["R"], wl["kda"]
        NS = B + 9
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.ssm = torch.empty(NS, HV, V, K, device=device)
        for s0 in range(0, NS, 64):                             # seeded fp32 states, generated in chunks
            n = min(64, NS - s0)
            self.ssm[s0:s0 + n] = (torch.randn(n, HV, V, K, generator=g) * 0.1).to(device)
        self.st = LeapQuantState(self.ssm, H, kda=kda, L=L, R=R, nmax=B)
        self.idx = torch.arange(1, B + 1, dtype=torch.int32, device=device)
        self.st.quantize(self.ssm, self.idx)
        self.period = L
        mixed, a, b, A_log, dtb = synth_inputs(B, H, HV, self.period, seed + 1, kda)
        # pinned host copies of the inputs, the three tensors of a step back to back so that one copy moves them
        from leapquant_b200.host_io import HostStagedDecoder
        self.h_slab, hv = HostStagedDecoder.host_slab(mixed[0], a[0].contiguous(), b[0], steps=self.period)
        for i in range(self.period):
            hv[i][0].copy_(mixed[i]); hv[i][1].copy_(a[i]); hv[i][2].copy_(b[i])
        self.h_mixed, self.h_a, self.h_b = [v[0] for v in hv], [v[1] for v in hv], [v[2] for v in hv]
        self.mixed, self.a, self.b = mixed.to(device), a.contiguous().to(device), b.to(device)
        self.A_log, self.dtb = A_log.to(device), dtb.to(device)
        self.out = torch.zeros(B, HV, V, dtype=torch.bfloat16, device=device)
        self.h_out = torch.zeros(B, HV, V, dtype=torch.bfloat16).pin_memory()
        self.staged = HostStagedDecoder(self.st, self.ssm, self.A_log, self.dtb, self.idx, self.h_mixed[0], self.h_a[0],
                                        self.h_b[0], self.h_out)

    def decode_resident(self, t):
        i = t % self.period
        self.st.decode(self.ssm, self.mixed[i], self.a[i], self.b[i], self.A_log, self.dtb, self.idx, self.out)

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


def timed(fn, stream):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    fn()
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e-3


def run_b200(args, wl):
    import torch.distributed as dist
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
    layer = Layer(wl, B, device, seed=100 + rank)
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (eager), then capture one window of L steps in a CUDA graph ----
    for t in range(L):                                          # a whole window: every head flushes once, hcnt returns to 0
        layer.decode_resident(t)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for t in range(L):
            layer.decode_resident(t)
    nwin_w, nwin = -(-warm // L), max(1, steps // L)
    rem = steps - nwin * L if steps >= L else 0
    if steps < L:                                               # fewer steps than a window: run them eagerly
        nwin, rem = 0, steps
    for _ in range(nwin_w):
        graph.replay()
    sampler = ClockSampler(visible_to_nvml_index(local)) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()

    def body():
        for _ in range(nwin):
            graph.replay()
        for t in range(rem):
            layer.decode_resident(t)

    dt = timed(body, torch.cuda.current_stream())
    barrier()
    if rem:                                                     # finish the partial window so that hcnt returns to 0
        for t in range(rem, L):
            layer.decode_resident(t)
    # ---- end to end through the public API with host buffers ----
    e2e_steps = min(steps, 4 * L)
    e2e_steps -= e2e_steps % L if e2e_steps >= L else 0
    for t in range(L):                                          # warm-up: one whole window through the host path
        layer.decode_host(t)
    layer.staged.drain()
    barrier()

    def body_e2e():
        for t in range(e2e_steps):
            layer.decode_host(t)
        layer.staged.join()                                     # the timed stream waits for the last output copy

    dt_e2e = timed(body_e2e, torch.cuda.current_stream())
    barrier()
    if e2e_steps % L:
        for t in range(e2e_steps % L, L):
            layer.decode_resident(t)
    clocks = sampler.finish() if sampler else None

    # ---- the step kernel alone over one window (roofline) ----
    snap = [t.clone() for t in (layer.ssm, layer.st.Kbuf, layer.st.Ubuf, layer.st.Wbuf, layer.st.Pbuf, layer.st.hcnt)]
    reps, tk = 3, 0.0
    for r in range(reps + 1):
        for dst, src in zip((layer.ssm, layer.st.Kbuf, layer.st.Ubuf, layer.st.Wbuf, layer.st.Pbuf, layer.st.hcnt), snap):
            dst.copy_(src)
        if kda:
            layer.st.Gbuf.fill_(1.0)
        torch.cuda.synchronize()

        def body_k():
            for t in range(L):
                layer.step_only(t)

        x = timed(body_k, torch.cuda.current_stream())
        if r > 0:
            tk += x
    step_ms = 1e3 * tk / (reps * L)
    # ---- the flush kernel alone: every head due (state left by the last pass above), then nothing due ----
    flush_all_ms = 1e3 * timed(lambda: layer.flush_only(), torch.cuda.current_stream())

    def body_f():
        for _ in range(20):
            layer.flush_only()

    flush_idle_ms = 1e3 * timed(body_f, torch.cuda.current_stream()) / 20
    # ---- the prefill round trip: dequantize every slot to fp32, quantize it again (65 536 B fp32 + the checkpoint per head) ----
    layer.st.dequantize(layer.ssm, layer.idx)
    layer.st.quantize(layer.ssm, layer.idx)
    deq_ms = 1e3 * timed(lambda: layer.st.dequantize(layer.ssm, layer.idx), torch.cuda.current_stream())
    quant_ms = 1e3 * timed(lambda: layer.st.quantize(layer.ssm, layer.idx), torch.cuda.current_stream())
    rt_bytes = B * HV * (4 * V * K + K * V + 4 * (K + V) + 2 * R * (K + V))
    alg_launch = B * HV * sum(step_bytes(h, L, R, gqa, kda) for h in range(L)) / L
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = alg_launch / (step_ms * 1e-3) / 1e9
    traffic = NCU_TRAFFIC_RATIO["kda" if kda else "gdn"]

    from leapquant_b200.sharding import job_times
    dt, dt_e2e = job_times([dt, dt_e2e], device)               # max over ranks
    done = nwin * L + rem
    units = world * B * HV * done
    value = units / dt
    e2e_value = world * B * HV * e2e_steps / dt_e2e if e2e_steps else None
    if rank == 0:
        cpu_rate, cpu_dt, cpu_sample = cpu_oracle_rate(wl, L, 3, nseq=8) if world == 1 else (None, None, None)
        amort = window_bytes_per_head_step(L, R, gqa, kda)
        line = {"metric": "int8_state_decode_head_steps_per_s", "value": value, "unit": "head-steps/s", "n_gpus": world,
                "steps": done, "warmup": nwin_w * L, "ms_per_step": 1e3 * dt / done, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": wl["name"], "batch_per_gpu": B, "value_heads": HV, "key_heads": wl["H"], "window": L,
                           "rank": R, "decode_steps_per_s_per_gpu": value / world / (B * HV),
                           "alg_bytes_per_head_step": amort, "whole_path_gbs_per_gpu": value / world * amort / 1e9,
                           "whole_path_frac_of_measured_hbm": value / world * amort / 1e9 / peak,
                           "whole_path_frac_of_8tbs": value / world * amort / 1e9 / 8000.0,
                           "l2": "per-step working set %.0f MB exceeds the 126 MB L2" % (B * HV * amort / 1e6),
                           "timing": "one window of %d steps captured in a CUDA graph, replayed" % L},
                "e2e": {"value": e2e_value, "unit": "head-steps/s", "h2d_bytes_per_step": layer.h2d_bytes(),
                        "d2h_bytes_per_step": layer.d2h_bytes(), "steps": e2e_steps},
                "gpu_launches": (1 if layer.st.fused else 2) * done,
                "roofline": {"bound": "hbm", "kernel": "step_pipelined_kernel", "achieved": achieved, "peak": peak,
                             "unit": "GB/s", "frac": achieved / peak, "frac_of_8tbs": achieved / 8000.0,
                             "traffic": (traffic * alg_launch) if traffic else None, "alg_bytes_per_launch": alg_launch,
                             "ms_per_launch": step_ms, "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback"},
                "flush": {"all_due_ms": flush_all_ms, "none_due_ms": flush_idle_ms,
                          "all_due_gbs": B * HV * flush_bytes(L, R, kda) / (flush_all_ms * 1e-3) / 1e9},
                "prefill_round_trip": {"dequantize_ms": deq_ms, "quantize_ms": quant_ms,
                                       "dequantize_gbs": rt_bytes / (deq_ms * 1e-3) / 1e9,
                                       "quantize_gbs": rt_bytes / (quant_ms * 1e-3) / 1e9},
                "clocks": clocks}
        if cpu_rate is not None:
            line["cpu_baseline"] = {"value": cpu_rate, "unit": "head-steps/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": cpu_sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gdn", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--step-impl", type=int, default=-1, help="debug: step kernel driver (see lq_set_option)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.step_impl >= 0:
        from leapquant_b200 import _lib
        _lib.set_option("step_impl", args.step_impl)
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_b200(args, wl)


if __name__ == "__main__":
    main()
