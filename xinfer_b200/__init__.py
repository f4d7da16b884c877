"""xinfer_b200: the speculative-decode hot path of xInfer, rebuilt for NVIDIA B200 (sm_100a).

The product is ``libxinfer_b200.so`` (hand-written CUDA behind a C-ABI, see ``include/xinfer_b200.h``).
This package is the thin host-side mirror of the reference's ops interface used by the tests and the
benchmark: it loads the shared library with ctypes and passes raw device pointers of torch tensors.
There is no CPU fallback: importing ``xinfer_b200.ops`` without the built library raises.
"""
from ._lib import lib, library_path, XInferError  # noqa: F401

__all__ = ["lib", "library_path", "XInferError"]
