"""Sharding of the state path over the GPUs of one box: none of it communicates.

Every (sequence slot, value head) is an independent unit, so the decode path scales by giving each process (one per
GPU) its own rows and its own state tensor.  Two partitions are provided: whole sequences (keeps each row of `mixed`
intact; what a data-parallel engine does) and value heads on key-head boundaries (what tensor parallelism does: the
reference reads the local head counts vLLM already sharded, reference leapquant/vllm/gdn.py:23).
"""


def shard_rows(n_rows, world, rank):
    """Contiguous, balanced [start, stop) of `n_rows` sequences for `rank` of `world` (sizes differ by at most one)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    base, extra = divmod(int(n_rows), int(world))
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_heads(H, HV, world, rank):
    """Key heads [k0, k1) and value heads [v0, v1) of `rank`: value heads follow their key head (GQA groups stay whole)."""
    if HV % H != 0:
        raise ValueError("HV must be a multiple of H")
    if H % world != 0:
        raise ValueError(f"{H} key heads do not split evenly over {world} ranks")
    gqa = HV // H
    k0, k1 = shard_rows(H, world, rank)
    return (k0, k1), (k0 * gqa, k1 * gqa)


def slice_mixed_heads(mixed, H, HV, K, V, world, rank):
    """Columns of a [N, 2HK + HV*V] q|k|v row block that belong to `rank` under shard_heads, as one tensor."""
    import torch
    (k0, k1), (v0, v1) = shard_heads(H, HV, world, rank)
    q = mixed[:, k0 * K:k1 * K]
    k = mixed[:, H * K + k0 * K:H * K + k1 * K]
    v = mixed[:, 2 * H * K + v0 * V:2 * H * K + v1 * V]
    return torch.cat([q, k, v], dim=1).contiguous()


def job_times(local_seconds, device=None):
    """Whole-job time of a weakly scaled run: the MAXIMUM over the ranks of each entry of `local_seconds` (a list of floats
    timed on this rank's device).  The only communication of the multi-GPU path: one all-reduce of a few doubles after the
    timed region (NCCL on GPUs, gloo in the CPU tests).  Without an initialised process group it returns the input."""
    import torch
    import torch.distributed as dist
    vals = [float(x) for x in local_seconds]
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return vals
    t = torch.tensor(vals, dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]
