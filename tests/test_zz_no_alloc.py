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
        before = torch.cuda.memory_allocated()
        assert cuda.linear_int4_noalloc(got, Xd, Wd, Sd, Bd, M, N, K) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert np.array_equal(got.cpu().numpy().view(np.uint16), ref_h.view(np.uint16)), call
    # a different problem right after, through the same array
    X2, W2, S2, _ = synth_linear(2, 256, 600, seed=1)
    a = torch.empty((2, 600), dtype=torch.float16, device="cuda")
    b = torch.empty((2, 600), dtype=torch.float16, device="cuda")
    assert cuda.linear_int4(a, dev(X2), dev(W2), dev(S2), None, 2, 600, 256) == 0
    assert cuda.linear_int4_noalloc(b, dev(X2), dev(W2), dev(S2), None, 2, 600, 256) == 0
    torch.cuda.synchronize()
    assert torch.equal(a, b)


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
