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


# ---------------------------------------------------------------------------------------------- N-split shard
def _tp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import numpy as np
    import oracle
    from conftest import synth_linear
    from xinfer_b200.tp import ColumnShardedLinear
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N = 3, 256, 64
        X, W, S, _ = synth_linear(M, K, N, seed=5)        # every rank builds the same full projection
        bias = np.linspace(-1.0, 1.0, N, dtype=np.float32)

        def cpu_linear(Y, Xt, Wt, St, bt, m, n, k, group_size=128):  # the shard's linear, on the CPU oracle
            y = oracle.linear_int4_grouped_f32(Xt.numpy(), Wt.numpy(), St.numpy(), None if bt is None else bt.numpy())
            Y.copy_(torch.from_numpy(y.astype(np.float16)))

        lin = ColumnShardedLinear(torch.from_numpy(W), torch.from_numpy(S), torch.from_numpy(bias), N, K,
                                  compute=cpu_linear, max_rows=4)
        y = lin.forward(torch.from_numpy(X), M)
        full = oracle.linear_int4_grouped_f32(X, W, S, bias).astype(np.float16)
        out[rank] = (lin.n0, lin.n1, bool(np.array_equal(y.numpy(), full)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_column_sharded_linear_world_size_2():
    world = 2
    port = 31500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_tp_worker, args=(world, port, out), nprocs=world, join=True)
    assert out[0] == (0, 32, True)
    assert out[1] == (32, 64, True)


def test_shard_rows_rules():
    sys.path.insert(0, ROOT)
    from xinfer_b200.tp import can_shard, shard_rows
    assert shard_rows(17408, 8, 3) == (6528, 8704)
    assert shard_rows(151936, 8, 7) == (132944, 151936)
    assert can_shard(48, 8) and not can_shard(48, 5) and not can_shard(1023, 2)
    with pytest.raises(ValueError):
        shard_rows(1023, 2, 0)
