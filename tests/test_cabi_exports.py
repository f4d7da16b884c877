"""CPU suite: the C-ABI library loads and exports every symbol include/xinfer_b200.h declares.
No compute entry point is called here (there is no GPU); the CRC functions are host code in the
reference as well and are checked against the oracle and the reference's own build."""
import ctypes
import os
import re

import numpy as np
import pytest

import oracle
from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "xinfer_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"XINFER_EXPORT[^;(]*?\b(xinfer_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from xinfer_b200 import _lib
    names = _declared()
    assert len(names) >= 30
    handle = ctypes.CDLL(_lib.library_path())
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, missing
    # the ctypes signature table covers exactly the header
    assert sorted(_lib.SIGNATURES) == names


def test_missing_library_fails_loudly(monkeypatch):
    from xinfer_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_PATH", "/nonexistent/libxinfer_b200.so")
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_crc64_drop_in(tmp_path, golden):
    import xinfer_b200.ops as ops
    _, meta = golden
    assert f"{ops.crc64(b'123456789'):016x}" == meta["crc64"]["123456789"]
    assert ops.crc64(b"") == 0
    rng = np.random.default_rng(2)
    data = rng.integers(0, 256, size=5_000_003, dtype=np.uint8).tobytes()
    assert ops.crc64(data) == oracle.crc64(data)
    f = tmp_path / "a.bin"
    f.write_bytes(data)
    ref = oracle.reference_crc_lib()
    whole = ops.crc64_file(str(f))
    assert whole == ops.crc64(data)
    assert ops.crc64_file(str(f), 4096) == ops.crc64(data[:4096])
    assert ops.crc64_file(str(tmp_path / "missing.bin")) == 0
    if ref is not None:
        assert ref.xinfer_crc64_file(str(f).encode(), 0) == whole
        assert ref.xinfer_crc64_file(str(f).encode(), 4096) == ops.crc64_file(str(f), 4096)


def test_status_codes_match_header():
    from xinfer_b200 import _lib
    text = open(os.path.join(ROOT, "include", "xinfer_b200.h")).read()
    for name, val in (("XINFER_OK", _lib.OK), ("XINFER_NOOP_INVALID_SHAPE", _lib.NOOP_INVALID_SHAPE),
                      ("XINFER_ERR_CUDA", _lib.ERR_CUDA), ("XINFER_ERR_INVALID_ARGUMENT", _lib.ERR_INVALID_ARGUMENT),
                      ("XINFER_ERR_OUT_OF_MEMORY", _lib.ERR_OUT_OF_MEMORY), ("XINFER_ERR_CONTRACT", _lib.ERR_CONTRACT),
                      ("XINFER_ERR_DEVICE_TIMEOUT", _lib.ERR_DEVICE_TIMEOUT), ("XINFER_ERR_NO_DEVICE", _lib.ERR_NO_DEVICE)):
        m = re.search(rf"{name}\s*=\s*(-?\d+)", text)
        assert m and int(m.group(1)) == val, name
