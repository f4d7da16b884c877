"""The C++ shim include/xinfer_b200_ops.hpp, compiled: tests/shim/shim_check.cpp is a host program written against
the reference's own names (xinfer::ops::linear_int4, linear_int4_fused, mlp_gate_up_swiglu_int4, argmax,
speculative_accept_reject, xinfer::core::DeviceContext, DeviceArena), built with plain g++ -std=c++17 and linked
to libxinfer_b200.so.  On CPU the test builds it and checks that it loads; on the GPU it runs the reference
tests' own cases through it."""
import os
import subprocess

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def shim_exe(tmp_path_factory):
    from xinfer_b200 import _lib
    libdir = os.path.dirname(_lib.library_path())
    assert os.path.exists(_lib.library_path()), "build the library first (python -m xinfer_b200.build)"
    exe = str(tmp_path_factory.mktemp("shim") / "shim_check")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "shim", "shim_check.cpp"), "-L", libdir, "-l:libxinfer_b200.so",
           f"-Wl,-rpath,{libdir}", "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_shim_program_builds_links_and_loads(shim_exe):
    r = subprocess.run([shim_exe, "--list"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    for name in ("linear_int4", "linear_int4_fused", "mlp_gate_up_swiglu_int4", "argmax", "speculative_accept_reject",
                 "DeviceArena"):
        assert name in r.stdout


@pytest.mark.gpu
def test_shim_program_passes_the_reference_cases(shim_exe, cuda):
    r = subprocess.run([shim_exe], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "shim check passed" in r.stdout and "FAILED" not in r.stdout
