"""The native file reader: byte ranges of a weights file straight into device memory.

`csrc/weight_reader.cu` does the work (host threads, page-locked staging, asynchronous copies);
this module builds and loads that small library and gives it a Python signature.  The reference
reads its weights file once, tensors in offset order (src/model_loader/gguf_types.rs:200-241).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p, create_string_buffer
from typing import Sequence

_lib = None


class ReadError(OSError):
    """The file could not be read as asked (missing, short, a failed read or a failed copy)."""


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        from ..csrc import build
        lib = build.load_library("iert_io", build.IO_SOURCES)
        lib.iert_read_file_ranges.argtypes = [c_char_p, c_int, POINTER(c_longlong), POINTER(c_longlong),
                                              POINTER(c_void_p), c_int, c_int, c_longlong, c_char_p, c_int]
        lib.iert_read_file_ranges.restype = c_int
        _lib = lib
    return _lib


def read_file_ranges(path: str, offsets: Sequence[int], sizes: Sequence[int], destinations: Sequence[int],
                     device_index: int, threads: int = 0, chunk_bytes: int = 0) -> None:
    """Range i = `sizes[i]` bytes at `offsets[i]` of the file, to the address `destinations[i]`:
    device memory of CUDA device `device_index`, or host memory when `device_index` is negative.
    Returns when all bytes have arrived.  The caller keeps the destinations alive and makes sure
    that nothing queued on the device still uses them."""
    n = len(offsets)
    if not (len(sizes) == n and len(destinations) == n):
        raise ValueError("offsets, sizes and destinations must have one entry per range")
    err = create_string_buffer(512)
    rc = library().iert_read_file_ranges(
        path.encode("utf-8"), n, (c_longlong * n)(*offsets), (c_longlong * n)(*sizes),
        (c_void_p * n)(*destinations), device_index, threads, chunk_bytes, err, len(err))
    if rc != 0:
        raise ReadError(f"{path}: {err.value.decode('utf-8', 'replace')}")
