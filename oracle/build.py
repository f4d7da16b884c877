"""Build recipe for the CPU oracle (test infrastructure, never part of the product).

Two artefacts:
  oracle/liboracle.so            this repository's C++ restatement (xinfer_oracle.cpp, mixers_oracle.cpp)
  oracle/_ref/libxinfer_artifact_c.so
                                 the reference's own CPU-only C-ABI library, compiled from the
                                 reference sources where they lie (only when the reference tree is
                                 present; nothing is copied).
  oracle/_ref/libxinfer_artifact_ref.so
                                 the reference's artifact writer and reader behind a small C wrapper
                                 (oracle/refwrap), same rule.  The reference's compute path is SYCL and
                                 cannot be built with gcc/nvcc, so the artifact code is the only reference
                                 code that runs here.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_LIB = os.path.join(REF_DIR, "libxinfer_artifact_c.so")
REF_ARTIFACT_LIB = os.path.join(REF_DIR, "libxinfer_artifact_ref.so")


def reference_root():
    """The reference tree: $XINFER_REFERENCE_ROOT, else a checkout named `reference` beside this repository."""
    env = os.environ.get("XINFER_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _sources():
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cpp"))


def _stale(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force: bool = False) -> str:
    srcs = _sources()
    if force or _stale(LIB, srcs):
        cmd = ["g++", "-O3", "-march=x86-64-v3", "-fopenmp", "-std=c++20", "-shared", "-fPIC",
               "-fno-fast-math", "-ffp-contract=off", "-o", LIB] + srcs
        subprocess.check_call(cmd)
    return LIB


def build_reference_crc(force: bool = False):
    """Compile the reference's xinfer_artifact_c (src/artifact/checksum.cpp + c_api.cpp)."""
    src_dir = os.path.join(reference_root(), "src", "artifact")
    srcs = [os.path.join(src_dir, "checksum.cpp"), os.path.join(src_dir, "c_api.cpp")]
    if not all(os.path.exists(s) for s in srcs):
        return REF_LIB if os.path.exists(REF_LIB) else None
    os.makedirs(REF_DIR, exist_ok=True)
    if force or _stale(REF_LIB, srcs):
        cmd = ["g++", "-O2", "-std=c++20", "-shared", "-fPIC", "-include", "cstdint",
               "-I", src_dir, "-o", REF_LIB] + srcs
        subprocess.check_call(cmd)
    return REF_LIB


def build_reference_artifact(force: bool = False):
    """Compile the reference's artifact writer and reader (src/artifact/{checksum,metadata,reader,writer}.cpp)
    behind the small C wrapper of oracle/refwrap, for cross-checks of this repository's reader and writer."""
    src_dir = os.path.join(reference_root(), "src", "artifact")
    srcs = [os.path.join(src_dir, f) for f in ("checksum.cpp", "metadata.cpp", "reader.cpp", "writer.cpp")]
    if not all(os.path.exists(s) for s in srcs):
        return REF_ARTIFACT_LIB if os.path.exists(REF_ARTIFACT_LIB) else None
    wrap = os.path.join(HERE, "refwrap", "ref_artifact_wrap.cpp")
    os.makedirs(REF_DIR, exist_ok=True)
    if force or _stale(REF_ARTIFACT_LIB, srcs + [wrap]):
        cmd = ["g++", "-O2", "-std=c++20", "-shared", "-fPIC", "-include", "cstdint", "-I", src_dir, "-o",
               REF_ARTIFACT_LIB, wrap] + srcs
        subprocess.check_call(cmd)
    return REF_ARTIFACT_LIB


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference_crc(force="--force" in sys.argv))
    print(build_reference_artifact(force="--force" in sys.argv))
