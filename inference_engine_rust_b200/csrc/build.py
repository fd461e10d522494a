"""Compiles the CUDA sources of this package for sm_100a with nvcc and loads the result.

The shared objects are built into `csrc/_build/` inside the package when that folder can
be written, else into a per-user folder under the system temporary directory.  A library's
file name carries a hash of its sources and flags, so an edited source is never served by a
stale binary.  Nothing here falls back to another implementation: without nvcc, or when a
compile fails, the import of the kernels fails with the compiler's message.
"""
from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Sequence, Tuple

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]

# name -> (sources, extra defines).  `core` holds every kernel whose code does not depend on
# the model's sizes; kernels specialised on a size are separate libraries made on demand.
CORE_SOURCES = [
    "runtime.cu", "elementwise.cu", "gemm_plain.cu", "attention_plain.cu", "sampling.cu",
    "gemm_tc.cu", "gemm_rows.cu", "attention_decode.cu",
]
# the native reader of weight files (host code), loaded by the weights package
IO_SOURCES = ["weight_reader.cu"]
HEADERS = ["common.cuh"]
# Extra -D definitions for experiments (space separated), e.g. IERT_EXTRA_DEFINES="FOO=1 BAR".
EXTRA_DEFINES = os.environ.get("IERT_EXTRA_DEFINES", "").split()


class BuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    print(f"[inference_engine_rust_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("IERT_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $IERT_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of this package cannot be built")


def build_dir() -> str:
    d = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"inference_engine_rust_b200-build-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _digest(sources: Sequence[str], defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    for name in list(sources) + HEADERS + _extra_headers(sources):
        with open(os.path.join(CSRC_DIR, name), "rb") as f:
            h.update(name.encode() + b"\0" + f.read())
    h.update(" ".join(NVCC_FLAGS + list(defines) + EXTRA_DEFINES).encode())
    return h.hexdigest()[:12]


def _extra_headers(sources: Sequence[str]) -> List[str]:
    out = []
    for name in sorted(os.listdir(CSRC_DIR)):
        if name.endswith((".cuh", ".h")) and name not in HEADERS:
            out.append(name)
    return out


def library_path(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> str:
    return os.path.join(build_dir(), f"lib{name}-{_digest(sources, defines)}.so")


def _compile_one(nvcc: str, src: str, obj: str, defines: Sequence[str]) -> None:
    defines = list(defines) + EXTRA_DEFINES
    cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-I", CSRC_DIR, "-c",
           os.path.join(CSRC_DIR, src), "-o", obj]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{p.stdout}")


def build_library(name: str, sources: Sequence[str], defines: Sequence[str] = (),
                  verbose: bool = True) -> str:
    """Compile (if its file is not there yet) and return the path of the shared object."""
    out = library_path(name, sources, defines)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    bdir = os.path.dirname(out)
    tag = os.path.basename(out)[:-3]
    t0 = time.time()
    if verbose:
        _say(f"building {os.path.basename(out)} from {len(sources)} CUDA source(s) for sm_100a ...")
    objs = [os.path.join(bdir, f"{tag}.{os.path.splitext(s)[0]}.{os.getpid()}.o") for s in sources]
    done = 0
    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            futs = {pool.submit(_compile_one, nvcc, s, o, defines): s for s, o in zip(sources, objs)}
            for fut in concurrent.futures.as_completed(futs):
                fut.result()
                done += 1
                if verbose:
                    _say(f"  compiled {futs[fut]} ({done}/{len(sources)}, {time.time() - t0:.0f}s)")
        tmp = out + f".{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-o", tmp, *objs, "-lcudart"]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise BuildError(f"link failed:\n{' '.join(cmd)}\n{p.stdout}")
        os.replace(tmp, out)            # atomic: concurrent builders agree on the result
    finally:
        for o in objs:
            try:
                os.unlink(o)
            except OSError:
                pass
    # drop binaries of older source versions of the same library
    prefix = f"lib{name}-"
    for f in os.listdir(bdir):
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(bdir, f) != out:
            try:
                os.unlink(os.path.join(bdir, f))
            except OSError:
                pass
    if verbose:
        _say(f"built {os.path.basename(out)} in {time.time() - t0:.0f}s")
    return out


def load_library(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = f"{name}:{','.join(defines)}"
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = build_library(name, sources, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
        return lib


# Head sizes whose prompt-attention library is built ahead of time by build_all(); any other
# multiple of 16 up to 256 is compiled the first time a model with that head size runs.
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 128)


def attention_library(head_dim: int):
    """(name, sources, defines) of the tensor-core attention library (prompt and decode
    kernels) for one head size."""
    return (f"iert_attn_hd{head_dim}", ["runtime.cu", "attention_prefill.cu", "attention_prefill_tc.cu", "attention_decode_tc.cu"],
            [f"HEAD_DIM={head_dim}"])


def build_all(verbose: bool = True) -> List[str]:
    """Every library the package can need that does not depend on a model's sizes, plus the
    size-specialised ones for the head sizes in `PREBUILT_HEAD_DIMS`."""
    paths = [build_library("iert_core", CORE_SOURCES, verbose=verbose),
             build_library("iert_io", IO_SOURCES, verbose=verbose)]
    for hd in PREBUILT_HEAD_DIMS:
        paths.append(build_library(*attention_library(hd), verbose=verbose))
    return paths
