"""world_size-2 CPU (gloo) test of the multi-GPU plumbing: shard ownership, the max-over-ranks
timing reduction and the optional output gather."""
import os
import socket
import sys

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from ditto_b200 import distributed as D
    from ditto_b200 import workloads as W
    r, w = D.init(backend="gloo")
    assert (r, w) == (rank, world)
    wl = W.WORKLOADS["cfg2"]
    lo, hi = D.shard_range(wl.units, rank, world)
    assert (lo, hi) == wl.shard(rank, world)
    q, k, v = W.attention_inputs(wl, lo, hi)
    # stand-in for the per-rank kernel: one row-sum per slice, enough to check who owns what
    local = torch.from_numpy(q.sum(axis=(1, 2), dtype="float64")).reshape(-1, 1)
    D.barrier()
    slowest = D.max_over_ranks(1.0 + rank)
    units = D.sum_over_ranks(hi - lo)
    full = D.gather_outputs(local, wl.units)
    # shards of unequal size (5 units over 2 ranks: 3 + 2; 1 unit over 2 ranks: 1 + 0)
    uneven = {}
    for total in (5, 1):
        ulo, uhi = D.shard_range(total, rank, world)
        mine = torch.arange(ulo, uhi, dtype=torch.float64).reshape(-1, 1) * 10
        uneven[total] = D.gather_outputs(mine, total)
    if rank == 0:
        torch.save({"slowest": slowest, "units": units, "full": full, "uneven": uneven}, out)
    D.barrier()
    torch.distributed.destroy_process_group()


def test_two_rank_sharding_and_reductions(tmp_path):
    from ditto_b200 import workloads as W
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    wl = W.WORKLOADS["cfg2"]
    assert res["slowest"] == 2.0           # the max over ranks, not rank 0's own time
    assert res["units"] == wl.units        # every slice owned exactly once
    q, _, _ = W.attention_inputs(wl, 0, wl.units)
    want = torch.from_numpy(q.sum(axis=(1, 2), dtype="float64")).reshape(-1, 1)
    assert torch.equal(res["full"], want)  # gather restores slice order
    for total, got in res["uneven"].items():
        assert torch.equal(got, torch.arange(total, dtype=torch.float64).reshape(-1, 1) * 10)
