"""The N > 1 path on CPU: two gloo ranks shard one workload (whole sequences, then value heads on key-head boundaries),
each drives the oracle on its shard with no data-path communication, and rank 0 checks that the gathered outputs and
states equal the unsharded run bit for bit; the timing aggregation (max over ranks) goes through the same helper the
benchmark uses."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lq_testlib import CpuSide, random_states
from oracle import lq_oracle as O

K = V = 128
NS, HV, H, L, R, N, T = 5, 4, 2, 4, 4, 4, 6


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_rows(states, lo, hi, mixed, a, b, A_log, dtb):
    """Oracle decode of the sequences lo .. hi-1 (slots lo+1 .. hi) in their own state object."""
    n = hi - lo
    cpu = CpuSide(n + 1, HV, H, K, V, L, R)
    cpu.ssm[1:].copy_(states[lo + 1:hi + 1])
    idx = torch.arange(1, n + 1, dtype=torch.int32)
    cpu.quantize(idx)
    outs = []
    for t in range(T):
        o = torch.zeros(n, HV, V, dtype=torch.bfloat16)
        cpu.decode(mixed[t, lo:hi], a[t, lo:hi], b[t, lo:hi], A_log, dtb, idx, o)
        outs.append(o)
    return torch.stack(outs), cpu.ssm[1:].clone(), cpu.bufs.hcnt[1:].clone()


def _run_heads(states, k0, k1, v0, v1, world, rank, mixed, a, b, A_log, dtb):
    from leapquant_b200.sharding import slice_mixed_heads
    hv, hk = v1 - v0, k1 - k0
    cpu = CpuSide(N + 1, hv, hk, K, V, L, R)
    cpu.ssm[1:].copy_(states[1:N + 1, v0:v1])
    idx = torch.arange(1, N + 1, dtype=torch.int32)
    cpu.quantize(idx)
    outs = []
    for t in range(T):
        o = torch.zeros(N, hv, V, dtype=torch.bfloat16)
        cpu.decode(slice_mixed_heads(mixed[t], H, HV, K, V, world, rank), a[t][:, v0:v1].contiguous(), b[t][:, v0:v1].contiguous(),
                   A_log[v0:v1], dtb[v0:v1], idx, o)
        outs.append(o)
    return torch.stack(outs), cpu.ssm[1:].clone()


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from leapquant_b200.sharding import job_times, shard_heads, shard_rows
        torch.set_num_threads(1)
        states = random_states(NS, HV, V, K, 11, 0.1)
        mixed, a, b, A_log, dtb = O.synth_inputs(N, H, HV, K, V, T, 12)
        # ---- whole sequences per rank ----
        lo, hi = shard_rows(N, world, rank)
        o_loc, s_loc, h_loc = _run_rows(states, lo, hi, mixed, a, b, A_log, dtb)
        # (gloo gathers neither bf16 nor int16: send the bit patterns widened to int32)
        ob = o_loc.view(torch.int16).to(torch.int32)
        go = [torch.zeros_like(ob) for _ in range(world)] if rank == 0 else None
        dist.gather(ob, go, dst=0)
        gs = [torch.zeros_like(s_loc) for _ in range(world)] if rank == 0 else None
        dist.gather(s_loc, gs, dst=0)
        # ---- value heads per rank ----
        (k0, k1), (v0, v1) = shard_heads(H, HV, world, rank)
        oh_loc, sh_loc = _run_heads(states, k0, k1, v0, v1, world, rank, mixed, a, b, A_log, dtb)
        ohb = oh_loc.view(torch.int16).to(torch.int32)
        goh = [torch.zeros_like(ohb) for _ in range(world)] if rank == 0 else None
        dist.gather(ohb, goh, dst=0)
        gsh = [torch.zeros_like(sh_loc) for _ in range(world)] if rank == 0 else None
        dist.gather(sh_loc, gsh, dst=0)
        # ---- timing aggregation: the slowest rank defines the job ----
        agg = job_times([1.0 + rank, 5.0 - rank])
        assert agg == [float(world), 5.0], agg
        if rank == 0:
            o_all, s_all, _ = _run_rows(states, 0, N, mixed, a, b, A_log, dtb)
            bits = lambda x: x.view(torch.int32)
            ok_rows = torch.equal(torch.cat(go, dim=1), o_all.view(torch.int16).to(torch.int32)) and \
                torch.equal(bits(torch.cat(gs, dim=0)), bits(s_all))
            ok_heads = torch.equal(torch.cat(goh, dim=2), o_all.view(torch.int16).to(torch.int32)) and \
                torch.equal(bits(torch.cat(gsh, dim=1)), bits(s_all))
            ret.put((ok_rows, ok_heads))
        dist.barrier()
    except Exception as e:                                     # report instead of leaving the parent to wait
        ret.put(("error", f"rank {rank}: {e!r}"))
        raise
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_without_communication():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    got = ret.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
    assert got[0] != "error", got[1]
    assert all(p.exitcode == 0 for p in procs)
    ok_rows, ok_heads = got
    assert ok_rows, "sequences sharded over two ranks differ from the unsharded run"
    assert ok_heads, "value heads sharded over two ranks differ from the unsharded run"
