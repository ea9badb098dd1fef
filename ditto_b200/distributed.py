"""Multi-GPU plumbing: the chains shard over independent units (slices or row blocks), one
process per GPU, with no collective on the data path.  torch.distributed is used for the barrier,
the max-over-ranks timing reduction and an optional gather of the per-rank outputs."""
import os

import torch
import torch.distributed as dist


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def init(backend=None, device=None):
    """Join the process group described by the torchrun environment (no-op for one process).
    `device` (a CUDA device) binds the NCCL communicator to this rank's GPU."""
    rank, world = env_rank_world()
    if world > 1 and not dist.is_initialized():
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {"device_id": device} if (backend == "nccl" and device is not None) else {}
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, world


def barrier():
    if dist.is_initialized():
        dist.barrier()


def shard_range(units, rank, world):
    """Contiguous [lo, hi) of `units` independent work items for `rank`; covers every unit once."""
    per = -(-units // world)
    lo = min(rank * per, units)
    return lo, min(lo + per, units)


def max_over_ranks(value, device="cpu"):
    """Largest `value` (a float, e.g. milliseconds) seen by any rank."""
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, device="cpu"):
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_outputs(local, units_total):
    """Optional all-gather of the per-rank output shards along dim 0 (NCCL over NVLink on GPUs), in unit
    order.  Shards follow `shard_range`, so the last ranks may hold fewer rows than the first, or none:
    every rank pads its shard to the common size ceil(units_total / world) before the collective (equal
    counts on every rank, which is what all_gather requires) and the padding is cut off afterwards.
    Not part of any timed region."""
    if not dist.is_initialized():
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    per = -(-units_total // world)
    lo, hi = shard_range(units_total, rank, world)
    if local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} holds {local.shape[0]} units, its shard of {units_total} has {hi - lo}")
    padded = local.new_zeros((per,) + tuple(local.shape[1:]))
    padded[:hi - lo] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat(parts, dim=0)[:units_total]
