"""Multi-GPU scaling as independent replicas.

A 0.6B-parameter model does not shard: every GPU holds the full weights and
its own KV cache and serves its own sequences.  Nothing crosses GPUs on the
data path; the only communication is the control plane below (a start barrier
and a max-reduce of the per-rank timings), which runs over gloo on CPU tensors.
"""
from __future__ import annotations

import os


def dist_env():
    """(rank, world_size, local_rank) from the torchrun environment."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def init_control_plane(world: int):
    """Initialise the gloo process group when there is more than one rank."""
    if world <= 1:
        return None
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not dist.is_initialized():
        dist.init_process_group("gloo")
    return dist


def barrier(dist) -> None:
    if dist is not None:
        dist.barrier()


def max_over_ranks(dist, values):
    """Element-wise maximum of a list of floats over all ranks."""
    if dist is None:
        return list(values)
    import torch
    t = torch.tensor(list(values), dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def aggregate_throughput(units_per_rank: float, world: int, slowest_seconds: float) -> float:
    """Whole-job throughput of `world` replicas that each processed
    `units_per_rank` units, the slowest in `slowest_seconds`."""
    return units_per_rank * world / slowest_seconds


def replica_seed(base_seq_idx: int, rank: int) -> int:
    """Every replica decodes its own prompt: the sequence index of the synthetic
    prompt generator is offset by the rank."""
    return base_seq_idx + rank
