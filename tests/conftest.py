import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    arrays = dict(np.load(os.path.join(GOLDEN_DIR, "ref_vectors.npz")))
    with open(os.path.join(GOLDEN_DIR, "ref_vectors.json")) as f:
        meta = json.load(f)
    return arrays, meta


def fill_weights(n_bytes, a, b):
    """W[i] = ((i+a)&0xF) | (((i+b)&0xF)<<4): the reference tests' weight pattern."""
    i = np.arange(n_bytes, dtype=np.int64)
    return (((i + a) & 0xF) | (((i + b) & 0xF) << 4)).astype(np.uint8)


def fill_scales(n, base=0.015, shift=0):
    i = np.arange(n, dtype=np.int64)
    f = np.float32(base) + ((i + shift) % 10).astype(np.float32) * np.float32(0.001)
    return f.astype(np.float16)


def synth_linear(M, K, N, seed=0):
    """Synthetic inputs with the benchmark configuration's distributions: int4 uniform in [-8, 7]
    packed two per byte along K (low nibble = even k), fp16 scales |N(0, 0.02)| / 7, fp16 N(0, 1)
    activations."""
    rng = np.random.default_rng(seed)
    q = rng.integers(-8, 8, size=(N, K), dtype=np.int8)
    W = ((q[:, 0::2] & 0xF) | ((q[:, 1::2] & 0xF) << 4)).astype(np.uint8)
    S = (np.abs(rng.normal(0.0, 0.02, size=(N, K // 128))) / 7.0).astype(np.float16)
    X = rng.normal(0.0, 1.0, size=(M, K)).astype(np.float16)
    return X, W, S, q


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import xinfer_b200.ops as ops
    from xinfer_b200 import lib
    assert lib().xinfer_b200_init(0) == 0, lib().xinfer_last_cuda_error()
    return ops
