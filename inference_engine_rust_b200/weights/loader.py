"""Weights by tensor name: checking a model folder against what the built model expects,
the stored-dtype policy, and the seeded random-weights mode.

The reference resolves roles to names, loads exactly those, and fails on a missing name
(src/model_weights/names.rs:52-222,295-297; src/model_weights/view.rs:152-155).  Here the
parts themselves say which tensors they expect (`TensorSpec`), and one error reports
every missing name, every unexpected name and every wrong shape together.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Tuple

import torch

from .safetensors_io import TensorSource, write_safetensors


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects under one name.  `init` tells the random-weights mode how to
    fill it: "normal" = N(0, std); "ones_plus_normal" = 1 + N(0, std) (norm scales);
    "int_table" = integers (kept as int32)."""

    shape: Tuple[int, ...]
    init: str = "normal"

    @property
    def is_int(self) -> bool:
        return self.init == "int_table"


class WeightError(ValueError):
    """Tensors of a model folder do not match the model.  Carries the three lists."""

    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_kind = sorted(wrong_kind)
        lines = [f"{where}: tensors do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file {list(got)}, model {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong dtype ({len(self.wrong_kind)}): " + "; ".join(
                f"{n}: file {dt}, model wants {kind}" for n, dt, kind in self.wrong_kind))
        super().__init__("\n".join(lines))


_FLOAT_NAMES = {"F32", "BF16", "F16", "F64"}
_INT_NAMES = {"I64", "I32", "I16", "I8", "U8"}


def check_source(expected: Mapping[str, TensorSpec], source: TensorSource, where: str,
                 strict: bool = True):
    """Compare what the model expects with what `source` holds; everything that is wrong comes
    in ONE `WeightError`.  `strict` (the default): a tensor the model does not know is an
    error.  Not strict: such tensors are left alone, as the reference loads only the names it
    resolves (src/model_weights/names.rs:224-276), and their names are returned."""
    have = set(source.names())
    want = set(expected)
    missing = want - have
    extra = have - want
    unexpected = extra if strict else set()
    wrong_shape, wrong_kind = [], []
    for name in want & have:
        dt, shape = source.describe(name)
        if tuple(shape) != tuple(expected[name].shape):
            wrong_shape.append((name, tuple(shape), tuple(expected[name].shape)))
        if expected[name].is_int and dt not in _INT_NAMES:
            wrong_kind.append((name, dt, "an integer table"))
        if not expected[name].is_int and dt not in _FLOAT_NAMES:
            wrong_kind.append((name, dt, "floating point"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_kind)
    return sorted(extra)


def stored_dtype_policy(t: torch.Tensor, run_dtype: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor keeps in memory.

    float32 run: every floating tensor is widened to float32 (the reference widens bf16 at
    load, src/model_loader/tensor_loader.rs:41-56).  bfloat16 run: bf16 stays bf16, a tensor
    stored in 32-bit stays 32-bit, f16/f64 go to 32-bit (exact for f16).  Integer tables
    become int32."""
    if not t.dtype.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    return torch.bfloat16 if t.dtype == torch.bfloat16 else torch.float32


def fetch(source, name: str, run_dtype: torch.dtype, device) -> torch.Tensor:
    t = source.get(name)
    return t.to(device=device, dtype=stored_dtype_policy(t, run_dtype)).contiguous()


def fetch_many(source, names, run_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """The named tensors on `device`, each in the dtype that `stored_dtype_policy` gives it.

    From files to a CUDA device, every tensor that keeps its stored dtype (bf16 weights in a
    bfloat16 run, 32-bit tensors always) is read by the native reader straight into its device
    tensor, all of them in one pass over each file; what needs a conversion, and every other kind
    of source, goes tensor by tensor through `fetch`."""
    device = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    direct: Dict[str, torch.Tensor] = {}
    can_read = hasattr(source, "read_into") and device.type == "cuda"
    for name in names:
        if can_read:
            stored = source.stored_dtype(name)
            if stored_dtype_policy(torch.empty(0, dtype=stored), run_dtype) == stored:
                _, shape = source.describe(name)
                direct[name] = torch.empty(tuple(shape), dtype=stored, device=device)
                continue
        out[name] = fetch(source, name, run_dtype, device)
    if direct:
        source.read_into(direct)
        out.update(direct)
    return out


# ---------------------------------------------------------------------------------------
# random weights


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, std: float,
                  dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """One tensor of the random model.  Its values depend on (seed, name) only, so any
    tensor can be made again alone.  (CPU and CUDA generators give different streams.)"""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.is_int:
        return torch.randint(0, 2 ** 15, spec.shape, generator=g, device=device, dtype=torch.int32)
    t = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * std
    if spec.init == "ones_plus_normal":
        t += 1.0
    elif spec.init != "normal":
        raise ValueError(f"tensor {name!r}: unknown init {spec.init!r}")
    return t.to(dtype)


class RandomSource:
    """Stands where a `TensorSource` stands, but makes each tensor when it is fetched."""

    def __init__(self, expected: Mapping[str, TensorSpec], seed: int, std: float = 0.02,
                 dtype: torch.dtype = torch.bfloat16, device="cpu"):
        self.expected, self.seed, self.std, self.dtype, self.device = dict(expected), seed, std, dtype, device

    def names(self):
        return list(self.expected)

    def describe(self, name):
        spec = self.expected[name]
        dt = "I32" if spec.is_int else {torch.bfloat16: "BF16", torch.float32: "F32"}[self.dtype]
        return dt, spec.shape

    def get(self, name):
        return random_tensor(name, self.expected[name], self.seed, self.std, self.dtype, self.device)


def write_model_folder(model_dir: str, config, tensors: Mapping[str, torch.Tensor]) -> None:
    """config.json + model.safetensors."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors, {"format": "pt"})
