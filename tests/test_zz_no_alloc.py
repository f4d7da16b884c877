"""GPU: the allocation-free linear entry point against the ordinary one.

Some callers of the library cannot allocate device memory when they call it (all HBM already pledged to a
cache pool, a fixed container quota, an ongoing graph capture), so `xinfer_linear_int4_f16f16_noalloc`
keeps its scratch in a fixed in-library array.  It runs the same kernel as `xinfer_linear_int4_f16f16`, so
the two must agree bit for bit; the second call in a row checks that what the first call left in the shared
array (partials, counters) does no harm.  This file is collected last on purpose."""
import numpy as np
import pytest
import torch

from conftest import synth_linear

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# (M, K, N): a cluster split-K shape, and one with more tiles than SMs, whose straddling tiles go through the
# scratch partials and counters
@pytest.mark.parametrize("M,K,N", [(4, 1024, 1000), (32, 512, 40000)])
def test_noalloc_matches_allocating_entry_point_twice(cuda, M, K, N):
    X, W, S, _ = synth_linear(M, K, N, seed=N)
    bias = np.linspace(-1, 1, N).astype(np.float32)
    Xd, Wd, Sd, Bd = dev(X), dev(W), dev(S), dev(bias)
    ref = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    assert cuda.linear_int4(ref, Xd, Wd, Sd, Bd, M, N, K) == 0
    assert cuda.last_linear_path() == 1
    torch.cuda.synchronize()
    ref_h = ref.cpu().numpy()
    assert not np.isnan(ref_h.astype(np.float32)).any()
    for call in range(2):
        got = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        assert cuda.linear_int4_noalloc(got, Xd, Wd, Sd, Bd, M, N, K) == 0
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint16), ref_h.view(np.uint16)), call
    # a different problem right after, through the same array
    X2, W2, S2, _ = synth_linear(2, 256, 600, seed=1)
    a = torch.empty((2, 600), dtype=torch.float16, device="cuda")
    b = torch.empty((2, 600), dtype=torch.float16, device="cuda")
    assert cuda.linear_int4(a, dev(X2), dev(W2), dev(S2), None, 2, 600, 256) == 0
    assert cuda.linear_int4_noalloc(b, dev(X2), dev(W2), dev(S2), None, 2, 600, 256) == 0
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_noalloc_takes_no_device_memory(cuda):
    """The property the entry point exists for: after the first call on the device (which resolves the array's
    address and configures all three row-count variants of the kernel), further calls change the device's free
    memory by nothing - measured with the driver's own figure, which sees every cudaMalloc of the process, not
    only torch's allocator."""
    shapes = [(4, 1024, 1000), (16, 512, 3000), (32, 512, 40000)]
    bufs = []
    for M, K, N in shapes:
        X, W, S, _ = synth_linear(M, K, N, seed=M)
        bufs.append((M, K, N, dev(X), dev(W), dev(S), torch.empty((M, N), dtype=torch.float16, device="cuda")))
    M, K, N, Xd, Wd, Sd, Y = bufs[0]
    assert cuda.linear_int4_noalloc(Y, Xd, Wd, Sd, None, M, N, K) == 0      # first call: set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        for M, K, N, Xd, Wd, Sd, Y in bufs:
            assert cuda.linear_int4_noalloc(Y, Xd, Wd, Sd, None, M, N, K) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert cuda.device_status(0) == 0


def test_noalloc_timeout_is_reported_through_device_status(cuda):
    """A bounded wait that gives up inside this entry point is reported by xinfer_device_status like any other
    launch's, and stays on record across a later call until it is read."""
    from xinfer_b200 import _lib
    M, K, N = 4, 256, 256
    X, W, S, _ = synth_linear(M, K, N, seed=9)
    Xd, Wd, Sd = dev(X), dev(W), dev(S)
    Y = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    ref = torch.empty_like(Y)
    assert cuda.linear_int4(ref, Xd, Wd, Sd, None, M, N, K) == 0
    cuda.set_wait_hooks(8_000_000, 0)           # the loader withholds the activations; waits give up after ~4 ms
    try:
        assert cuda.linear_int4_noalloc(Y, Xd, Wd, Sd, None, M, N, K) == 0
        torch.cuda.synchronize()
    finally:
        cuda.set_wait_hooks(0, -1)
    assert cuda.linear_int4_noalloc(Y, Xd, Wd, Sd, None, M, N, K) == 0   # a good call does not wipe the record
    torch.cuda.synchronize()
    assert torch.equal(Y, ref)
    assert cuda.device_status(0) == _lib.ERR_DEVICE_TIMEOUT
    assert cuda.device_status(0) == 0


def test_noalloc_refuses_what_it_cannot_do(cuda):
    from xinfer_b200 import _lib
    X, W, S, _ = synth_linear(40, 256, 64, seed=0)
    Y = torch.empty((40, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(_lib.XInferError) as e:
        cuda.linear_int4_noalloc(Y, dev(X), dev(W), dev(S), None, 40, 64, 256)       # M > 32
    assert e.value.code == _lib.ERR_INVALID_ARGUMENT
    with pytest.raises(_lib.XInferError):
        cuda.linear_int4_noalloc(Y, dev(X), dev(W), dev(S), None, 4, 64, 256, 64)    # group size 64
    assert cuda.linear_int4_noalloc(Y, dev(X), dev(W), dev(S), None, 0, 64, 256) == 1  # empty shape: no-op
