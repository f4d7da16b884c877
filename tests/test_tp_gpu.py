"""N-split tensor-parallel linear over NCCL on two GPUs of one node (skipped with fewer): the gathered result
of the sharded call must equal the unsharded call on the same GPU (same kernel per output row; only the
split-K summation order may differ, hence the GEMM tolerance) and match the oracle."""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, synth_linear

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import xinfer_b200.ops as ops
    from xinfer_b200 import lib
    from xinfer_b200.tp import ColumnShardedLinear
    torch.cuda.set_device(rank)
    assert lib().xinfer_b200_init(rank) == 0
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        worst = 0.0
        for (M, K, N) in [(1, 5120, 6144), (8, 5120, 17408), (32, 6144, 5120)]:
            X, W, S, _ = synth_linear(M, K, N, seed=11)
            Xd, Wd, Sd = torch.from_numpy(X).cuda(), torch.from_numpy(W).cuda(), torch.from_numpy(S).cuda()
            lin = ColumnShardedLinear(Wd, Sd, None, N, K)
            y_tp = lin.forward(Xd, M)
            y_full = torch.empty((M, N), dtype=torch.float16, device="cuda")
            ops.linear_int4(y_full, Xd, Wd, Sd, None, M, N, K)
            torch.cuda.synchronize()
            a, b = y_tp.float().cpu().numpy(), y_full.float().cpu().numpy()
            worst = max(worst, float(np.max(np.abs(a - b) / (np.abs(b) + 1e-2))))
        out[rank] = (worst, ops.device_status(rank))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_column_sharded_linear_two_gpus(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    port = 33500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for r in range(world):
        worst, status = out[r]
        assert status == 0
        assert worst <= 2e-3, worst   # one fp16 rounding of the output apart at most
