"""`.xinfer` artifacts: a writer of the reference's container format and a handle on the C-ABI reader / loader.

Format (docs/artifact-format.md and src/artifact/container.h:20-63 of the reference): 64-byte header, metadata JSON,
section payloads on 64-byte boundaries, a table of 128-byte section entries, a 16-byte footer with the CRC-64 of
everything before it.  The writer lays a file out exactly as the reference's ArtifactWriter::write_to_file does
(src/artifact/writer.cpp:62-190), so its files are byte-identical for the same sections.
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import Iterable, Optional, Tuple

import numpy as np

from . import _lib
from ._lib import check, lib

RAW_BLOB, METADATA_JSON, TOKENIZER_DATA, TENSOR_WEIGHTS, TENSOR_SCALES, CHAT_TEMPLATE, CUSTOM = 0, 1, 2, 3, 4, 5, 0xFF
_ALIGN = 64


def _crc(data: bytes) -> int:
    if not data:
        return 0
    buf = C.create_string_buffer(data, len(data))
    return int(lib().xinfer_crc64(C.cast(buf, C.c_void_p), len(data)))


def write_artifact(path: str, metadata_json: str, sections: Iterable[Tuple[str, int, bytes]]) -> None:
    """Writes `sections` = (name, type tag, payload bytes) in order."""
    sections = [(n, t, bytes(d)) for n, t, d in sections]
    meta = metadata_json.encode()
    body = bytearray(64)                      # header placeholder
    meta_off = len(body)
    body += meta
    entries = []
    for name, tag, data in sections:
        body += b"\0" * ((-len(body)) % _ALIGN)
        nm = name.encode()[:95]
        entries.append(struct.pack("<96sIIQQQ", nm, tag, 0, len(body), len(data), _crc(data)))
        body += data
    body += b"\0" * ((-len(body)) % _ALIGN)
    table_off = len(body)
    for e in entries:
        body += e
    total = len(body) + 16
    body[0:64] = struct.pack("<8sIIIIQQQQQ", b"XINFER\0\0", 1, 64, 0, len(sections), meta_off, len(meta), table_off,
                             len(entries) * 128, total)
    with open(path, "wb") as f:
        f.write(body)
        f.write(struct.pack("<Q8s", _crc(bytes(body)), b"XINFFOOT"))


class ArtifactReader:
    """Handle on an open artifact (xinfer_artifact_* in the C-ABI)."""

    def __init__(self, path: str, verify_file_checksum: bool = True):
        h = C.c_void_p()
        check(lib().xinfer_artifact_open(path.encode(), 1 if verify_file_checksum else 0, C.byref(h)), "artifact_open")
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib().xinfer_artifact_close(self._h)
            self._h = None

    __del__ = close

    def error(self) -> str:
        return lib().xinfer_artifact_error(self._h).decode()

    def metadata_json(self) -> str:
        n = C.c_uint64()
        p = lib().xinfer_artifact_metadata(self._h, C.byref(n))
        return (p or b"")[: n.value].decode()

    def sections(self):
        out = []
        for i in range(lib().xinfer_artifact_section_count(self._h)):
            name, tag, off, size, crc = C.c_char_p(), C.c_uint32(), C.c_uint64(), C.c_uint64(), C.c_uint64()
            check(lib().xinfer_artifact_section_info(self._h, i, C.byref(name), C.byref(tag), C.byref(off), C.byref(size),
                                                     C.byref(crc)), "section_info")
            out.append({"name": name.value.decode(), "type": tag.value, "offset": off.value, "size": size.value,
                        "checksum": crc.value})
        return out

    def has_section(self, name: str) -> bool:
        return lib().xinfer_artifact_find(self._h, name.encode()) >= 0

    def read_section(self, name: str) -> bytes:
        i = lib().xinfer_artifact_find(self._h, name.encode())
        if i < 0:
            raise KeyError(name)
        size = self.sections()[i]["size"]
        buf = np.empty(max(size, 1), np.uint8)
        check(lib().xinfer_artifact_read_section(self._h, name.encode(), buf.ctypes.data_as(C.c_void_p), size), "read_section")
        return buf[:size].tobytes()

    def load_linear(self, weight_name: str, out_features: int, in_features: int, dst_weights, dst_scales,
                    row0: int = 0, rows: Optional[int] = None, group_size: int = 128, verify: bool = True) -> int:
        """Rows [row0, row0 + rows) of an INT4 projection and its scales into CUDA tensors (torch) or raw device pointers."""
        rows = out_features - row0 if rows is None else rows
        pw = dst_weights.data_ptr() if hasattr(dst_weights, "data_ptr") else dst_weights
        ps = dst_scales.data_ptr() if hasattr(dst_scales, "data_ptr") else dst_scales
        return check(lib().xinfer_artifact_load_linear(self._h, weight_name.encode(), out_features, in_features, group_size,
                                                       row0, rows, pw, ps, 1 if verify else 0), "load_linear")

    def load_bf16_as_f32(self, name: str, num_elements: int, dst, add_unit_offset: bool = False) -> int:
        p = dst.data_ptr() if hasattr(dst, "data_ptr") else dst
        return check(lib().xinfer_artifact_load_bf16_as_f32(self._h, name.encode(), num_elements, 1 if add_unit_offset else 0, p),
                     "load_bf16_as_f32")
