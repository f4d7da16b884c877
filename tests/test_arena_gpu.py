"""GPU: the cudaMalloc-backed arena keeps the DeviceArena contract (src/core/arena.h:14-66,
src/core/arena.cpp:84-139; exercised by the reference in tests/test_core_device.cpp)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bump_alignment_reset_and_overflow(cuda):
    a = cuda.DeviceArena(1 << 20)
    assert a.capacity() == 1 << 20 and a.allocated_bytes() == 0
    p0 = a.allocate(100)
    p1 = a.allocate(100)
    assert p0 == a.base_ptr() and p0 % 64 == 0 and p1 % 64 == 0 and p1 - p0 == 128
    p2 = a.allocate(8, 4096)
    assert p2 % 4096 == 0
    assert a.allocate(0) is None
    used = a.allocated_bytes()
    assert used == (p2 - p0) + 8 and a.remaining_bytes() == (1 << 20) - used
    with pytest.raises(MemoryError):
        a.allocate(1 << 20)
    assert a.allocated_bytes() == used  # a failed allocation changes nothing
    a.reset()
    assert a.allocated_bytes() == 0 and a.peak_allocated_bytes() == used
    # address reuse over many steps, as the reference's 500-step loop checks
    first = a.allocate(4096)
    for _ in range(500):
        a.reset()
        assert a.allocate(4096) == first
    a.close()


def test_persistent_allocations_survive_reset(cuda):
    a = cuda.DeviceArena(1 << 16)
    p = a.allocate_persistent(1 << 12)
    base = a.base_ptr()
    assert p is not None and not (base <= p < base + (1 << 16))
    with pytest.raises(ValueError):
        a.persistent_buffer(0)  # the first call must give a size
    b = a.persistent_buffer(1 << 14)
    a.reset()
    assert a.persistent_buffer() == b and a.persistent_buffer(1 << 10) == b
    with pytest.raises(ValueError):
        a.persistent_buffer(1 << 15)  # refuses to grow
    # the memory is usable from kernels: fill it on the device, reduce it on the device
    import numpy as np
    import oracle
    from xinfer_b200 import lib
    n = 3000
    s = torch.cuda.current_stream().cuda_stream
    assert lib().xinfer_philox_uniform(s, p, n, 5, 0) == 0
    assert lib().xinfer_argmax(s, p, n, None, None) == oracle.argmax(oracle.philox_uniform(n, 5, 0))
    a.close()
