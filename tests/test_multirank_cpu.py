"""CPU, world_size 2 over gloo: the aggregation bench.py applies when it runs one process per GPU (replicas:
the path has no data-path collective, so the only cross-rank step is max-of-times / sum-of-units)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ms = 10.0 + 5.0 * rank          # rank 1 is slower
        tokens = 80 + rank              # and emitted one more token
        (ms_all, e2e_all), (tok_all, _) = bench.reduce_over_ranks([ms, 2.0 * ms], [tokens, 0])
        out[rank] = (ms_all, e2e_all, tok_all)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_replica_aggregation_world_size_2():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert out[0] == out[1] == (15.0, 30.0, 161.0)
    # whole-job throughput = all units / slowest rank's time
    assert abs(out[0][2] / (out[0][0] * 1e-3) - 161.0 / 0.015) < 1e-6


def test_single_process_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.reduce_over_ranks([1.5], [7]) == ([1.5], [7])
