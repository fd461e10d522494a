"""Reading and writing the safetensors container: an 8-byte little-endian header length,
a JSON header `{name: {dtype, shape, data_offsets}}`, then the raw little-endian data.

This takes the place of the reference's GGUF reader (src/model_loader/file_loader.rs:26-65,
src/model_loader/gguf_types.rs:200-272): metadata first, tensors fetched by name, nothing
read that is not asked for.  Files are memory-mapped; a tensor's bytes are touched only
when it is fetched.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import torch


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors container."""


_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One mapped file.  `entries[name] = (dtype_name, shape, begin, end)`."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        data_len = size - self._base
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            n = 1
            for s in shape:
                n *= s
            if not (0 <= b <= e <= data_len) or e - b != n * _DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} ({dt}, shape {list(shape)}) has bad data_offsets [{b}, {e}] "
                    f"for {data_len} data bytes")
            self.entries[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def get(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor sharing the mapping (read-only: copy before writing)."""
        dt, shape, b, e = self.entries[name]
        tdt, _ = _DTYPES[dt]
        n = 1
        for s in shape:
            n *= s
        if n == 0:
            return torch.empty(shape, dtype=tdt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # torch warns that the buffer is not writable
            flat = torch.frombuffer(self._mm, dtype=tdt, count=n, offset=self._base + b)
        return flat.reshape(shape)


    def byte_range(self, name: str) -> Tuple[int, int]:
        """(offset in the file, size in bytes) of the tensor's data."""
        _, _, b, e = self.entries[name]
        return self._base + b, e - b


class TensorSource:
    """All tensors of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(single):
            f = SafetensorsFile(single)
            self._files[single] = f
            for n in f.names():
                self._where[n] = single
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as fh:
                try:
                    wm = json.load(fh)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: no 'weight_map' object") from None
            for name, shard in wm.items():
                p = os.path.join(model_dir, shard)
                if p not in self._files:
                    self._files[p] = SafetensorsFile(p)
                if name not in self._files[p].entries:
                    raise SafetensorsError(f"{index}: maps {name!r} to {shard}, which does not hold it")
                self._where[name] = p
        else:
            raise SafetensorsError(
                f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")

    def names(self) -> List[str]:
        return list(self._where)

    def describe(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        dt, shape, _, _ = self._files[self._where[name]].entries[name]
        return dt, shape

    def get(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].get(name)

    def stored_dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.describe(name)[0]][0]

    def read_into(self, targets: Mapping[str, torch.Tensor], threads: int = 0, chunk_bytes: int = 0) -> None:
        """Fill `targets[name]` (contiguous, of the stored dtype and shape; on a CUDA device or on
        the host) with the named tensors' data, through the native reader: one call per file,
        every tensor straight to its destination."""
        from .native_reader import read_file_ranges
        by_file: Dict[str, List[str]] = {}
        device = None
        for name, t in targets.items():
            dt, shape = self.describe(name)
            if t.dtype != _DTYPES[dt][0] or tuple(t.shape) != tuple(shape) or not t.is_contiguous():
                raise SafetensorsError(f"{name}: the destination must be contiguous {dt} of shape {list(shape)}")
            if device is None:
                device = t.device
            elif t.device != device:
                raise SafetensorsError("all destinations of one read must be on the same device")
            by_file.setdefault(self._where[name], []).append(name)
        if device is None:
            return
        if device.type == "cuda":
            index = device.index if device.index is not None else torch.cuda.current_device()
            torch.cuda.synchronize(device)      # memory the allocator hands out again may still be in use
        else:
            index = -1
        for path, names in by_file.items():
            f = self._files[path]
            ranges = [f.byte_range(n) for n in names]
            read_file_ranges(path, [r[0] for r in ranges], [r[1] for r in ranges],
                             [targets[n].data_ptr() for n in names], index, threads, chunk_bytes)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write `tensors` (CPU, contiguous or not) in name order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b"")
