"""ctypes bindings of the CUDA launchers.  Every function here launches hand-written
kernels on the current CUDA stream; there is no other implementation behind them, so a
machine without the built library (or without a GPU) gets an error, not a fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
PAIR_HALF, PAIR_INTERLEAVED = 0, 1
GEMM_STORE, GEMM_ADD_RESIDUAL = 0, 1

ERR_TOKEN_RANGE, ERR_NONFINITE_LOGIT, ERR_PAGE_RANGE, ERR_WAIT_EXPIRED = 1, 2, 4, 8
_ERR_TEXT = {
    ERR_TOKEN_RANGE: "a token id outside [0, vocab) reached the embedding kernel",
    ERR_NONFINITE_LOGIT: "sampling saw a NaN or infinite logit",
    ERR_PAGE_RANGE: "a page-table entry outside the page pool was read",
    ERR_WAIT_EXPIRED: "a bounded wait inside a kernel expired",
}


class KernelError(RuntimeError):
    pass


class KvView(Structure):
    """Mirror of `IertKvView` (common.cuh)."""
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("page_table", c_void_p),
                ("table_width", c_int), ("ring_pages", c_int), ("page_tokens", c_int),
                ("n_pages", c_int), ("kv_heads", c_int), ("head_dim", c_int),
                ("dtype", c_int), ("window", c_int)]


class BatchView(Structure):
    """Mirror of `IertBatchView` (common.cuh)."""
    _fields_ = [("cu_q", c_void_p), ("slot_ids", c_void_p), ("tok_seq", c_void_p),
                ("pos0", c_void_p), ("n_seqs", c_int), ("n_tokens", c_int)]


class NormAhead(Structure):
    """Mirror of `IertNormAhead` (common.cuh): the first half of an RMSNorm, written by the kernel that
    writes the rows."""
    _fields_ = [("weight", c_void_p), ("weight_dtype", c_int), ("scaled_out", c_void_p), ("ld", c_longlong),
                ("sumsq_out", c_void_p), ("parts", c_int)]


class RowScale(Structure):
    """Mirror of `IertRowScale`: the second half, applied by the projection that reads the scaled rows."""
    _fields_ = [("sumsq", c_void_p), ("parts", c_int), ("hidden", c_int), ("eps", c_float)]


def norm_ahead(weight, scaled_out, sumsq_out) -> NormAhead:
    return NormAhead(weight=weight.data_ptr(), weight_dtype=dtype_code(weight.dtype), scaled_out=scaled_out.data_ptr(),
                     ld=scaled_out.stride(0), sumsq_out=sumsq_out.data_ptr(), parts=0)


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dt}")


_core = None


def core() -> ctypes.CDLL:
    """The core library, built on first use."""
    global _core
    if _core is None:
        lib = build.load_library("iert_core", build.CORE_SOURCES)
        _declare(lib)
        if os.environ.get("IERT_PDL", "1") == "0":      # programmatic dependent launch off (for measurements)
            lib.iert_set_pdl(0)
        _core = lib
    return _core


def _declare(lib) -> None:
    S = c_void_p  # cudaStream_t
    P = c_void_p
    lib.iert_last_cuda_error.restype = c_char_p
    lib.iert_device_arch.restype = c_int
    lib.iert_sm_count.restype = c_int
    sigs = {
        "iert_embed_gather": [P, c_int, P, P, c_int, c_int, c_int, c_float, P, POINTER(NormAhead), S],
        "iert_rmsnorm": [P, P, c_int, P, c_int, P, c_int, c_int, c_float, S],
        "iert_rope_kv_store": [P, c_int, POINTER(BatchView), POINTER(KvView), P, c_int, c_int, c_int, c_int, P, S],
        "iert_silu_mul": [P, P, c_int, c_int, c_int, S],
        "iert_add_into": [P, P, c_int, c_longlong, S],
        "iert_advance_positions": [P, P, P, c_int, S],
        "iert_gemm_plain": [P, c_int, P, c_int, P, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, S],
        "iert_attention_plain": [P, P, c_int, POINTER(BatchView), POINTER(KvView), c_int, c_float, c_int, P, S],
        "iert_sample_greedy": [P, c_int, c_int, c_longlong, P, P, S],
        "iert_sample_temperature": [P, c_int, c_int, c_longlong, c_float, c_ulonglong, P, P, P, P, S],
        "iert_uniform_draws": [c_ulonglong, P, P, P, c_int, S],
        "iert_gemm_tc": [P, c_longlong, P, c_longlong, P, c_int, c_longlong, c_int, c_int, c_int, c_int,
                         P, c_longlong, P, c_int, c_int, c_int, c_int, P, S],
    }
    lib.iert_attention_decode.argtypes = [P, P, POINTER(BatchView), POINTER(KvView), c_int, c_float, c_int, P, P, S]
    lib.iert_attention_decode.restype = c_int
    lib.iert_attention_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.iert_attention_decode_scratch_floats.restype = c_longlong
    lib.iert_gemm_tc_gated.argtypes = [P, c_longlong, P, c_longlong, P, c_longlong, c_int, c_int, c_int, c_int,
                                       c_int, P, S]
    lib.iert_gemm_tc_gated.restype = c_int
    lib.iert_gemm_rows.argtypes = [P, c_longlong, P, c_longlong, P, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                   POINTER(RowScale), POINTER(NormAhead), c_int, P, S]
    lib.iert_gemm_rows.restype = c_int
    lib.iert_gemm_tc_scaled.argtypes = [P, c_longlong, P, c_longlong, P, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                        P, c_longlong, P, c_int, POINTER(RowScale), POINTER(NormAhead), c_int, c_int, P, S]
    lib.iert_gemm_tc_scaled.restype = c_int
    lib.iert_gemm_tc_gated_scaled.argtypes = [P, c_longlong, P, c_longlong, P, c_longlong, c_int, c_int, c_int,
                                              POINTER(RowScale), c_int, P, S]
    lib.iert_gemm_tc_gated_scaled.restype = c_int
    lib.iert_gemm_tc_workspace_bytes.restype = c_longlong
    lib.iert_gemm_tc_counter_count.restype = c_int
    lib.iert_gemm_tc_set_poll_limit.argtypes = [ctypes.c_uint]
    lib.iert_gemm_tc_set_poll_limit.restype = None
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


launch_count = 0        # launcher calls that returned success since import (one kernel each)


def check(status: int, what: str) -> None:
    global launch_count
    if status == 0:
        launch_count += 1
        return
    if status == 1:
        raise KernelError(f"{what}: the kernel does not take these sizes or options")
    msg = core().iert_last_cuda_error().decode("utf-8", "replace")
    raise KernelError(f"{what}: CUDA error: {msg}")


def require_device() -> None:
    """Refuse to run anywhere but on an sm_100 GPU with the built library."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this package runs its hand-written sm_100a kernels only")
    arch = core().iert_device_arch()
    if arch < 0:
        raise KernelError("device query failed: " + core().iert_last_cuda_error().decode())
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a; this device is sm_{arch}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def describe_error_bits(bits: int) -> str:
    return "; ".join(t for b, t in _ERR_TEXT.items() if bits & b) or f"unknown error bits {bits}"


# ---------------------------------------------------------------------------------------
# thin wrappers: tensors in, launch, nothing returned


def embed_gather(table, ids, x, scale: float, err, stream, ahead: Optional[NormAhead] = None) -> int:
    """x[t] = table[ids[t]] * scale.  `ahead`: also the first half of the norm that follows
    (`norm_ahead`); returns the partial sums of squares per row it wrote (0 without `ahead`)."""
    vocab, hidden = table.shape
    check(core().iert_embed_gather(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(),
                                   x.data_ptr(), ids.numel(), hidden, vocab, scale,
                                   err.data_ptr(), byref(ahead) if ahead is not None else None, stream), "embed_gather")
    return int(ahead.parts) if ahead is not None else 0


def rmsnorm(x, w, out, eps: float, stream, rows_idx=None, rows: Optional[int] = None) -> None:
    hidden = x.shape[-1]
    n = rows if rows is not None else (rows_idx.numel() if rows_idx is not None else x.shape[0])
    check(core().iert_rmsnorm(x.data_ptr(), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(),
                              dtype_code(out.dtype),
                              rows_idx.data_ptr() if rows_idx is not None else None,
                              n, hidden, eps, stream), "rmsnorm")


_SM_COUNT = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device."""
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = int(core().iert_sm_count())
    return _SM_COUNT


def rope_kv_store(qkv, batch: BatchView, kv: KvView, inv_freq, heads: int, rotary_dim: int,
                  pairing: int, write_cache: bool, err, stream) -> None:
    check(core().iert_rope_kv_store(qkv.data_ptr(), dtype_code(qkv.dtype), byref(batch), byref(kv),
                                    inv_freq.data_ptr(), heads, rotary_dim, pairing,
                                    1 if write_cache else 0, err.data_ptr(), stream), "rope_kv_store")


_no_rotation = {}


def _zero_freq(device):
    key = str(device)
    if key not in _no_rotation:
        _no_rotation[key] = torch.zeros(1, dtype=torch.float32, device=device)
    return _no_rotation[key]


def kv_store(qkv, batch: BatchView, kv: KvView, heads: int, err, stream) -> None:
    """Write the step's keys and values (as they stand in the packed projection) into the cache."""
    rope_kv_store(qkv, batch, kv, _zero_freq(qkv.device), heads, 0, PAIR_HALF, True, err, stream)


def rotate_qk(qkv, batch: BatchView, inv_freq, heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
              pairing: int, err, stream) -> None:
    """Rotate the step's queries and keys in place; nothing is stored."""
    geometry = KvView(k=None, v=None, page_table=None, table_width=0, ring_pages=1, page_tokens=1, n_pages=0,
                      kv_heads=kv_heads, head_dim=head_dim, dtype=dtype_code(qkv.dtype), window=0)
    rope_kv_store(qkv, batch, geometry, inv_freq, heads, rotary_dim, pairing, False, err, stream)


def silu_mul(gu, out, n_tokens: int, inter: int, stream) -> None:
    check(core().iert_silu_mul(gu.data_ptr(), out.data_ptr(), dtype_code(gu.dtype), n_tokens, inter,
                               stream), "silu_mul")


def add_into(residual, y, n: int, stream) -> None:
    check(core().iert_add_into(residual.data_ptr(), y.data_ptr(), dtype_code(y.dtype), n, stream),
          "add_into")


def advance_positions(batch: "BatchView", stream) -> None:
    check(core().iert_advance_positions(batch.pos0, batch.cu_q, batch.slot_ids, batch.n_seqs, stream),
          "advance_positions")


def gemm_plain(x, w, out, M: int, mode: int, stream) -> None:
    """out[:M] (=|+=) x[:M] @ w.T with x [*, K], w [N, K], out [*, N]; row strides taken
    from the tensors."""
    N, K = w.shape
    check(core().iert_gemm_plain(x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype),
                                 out.data_ptr(), dtype_code(out.dtype), M, N, K,
                                 x.stride(0), w.stride(0), out.stride(0), mode, stream), "gemm_plain")


def attention_plain(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, paged: bool,
                    err, stream) -> None:
    check(core().iert_attention_plain(qkv.data_ptr(), out.data_ptr(), dtype_code(qkv.dtype),
                                      byref(batch), byref(kv), heads, scale, 1 if paged else 0,
                                      err.data_ptr(), stream), "attention_plain")


def sample_greedy(logits, out, err, stream) -> None:
    rows, vocab = logits.shape
    check(core().iert_sample_greedy(logits.data_ptr(), rows, vocab, logits.stride(0), out.data_ptr(),
                                    err.data_ptr(), stream), "sample_greedy")


def sample_temperature(logits, temperature: float, seed: int, request_ids, step_ids, out, err,
                       stream) -> None:
    rows, vocab = logits.shape
    check(core().iert_sample_temperature(logits.data_ptr(), rows, vocab, logits.stride(0),
                                         temperature, seed & 0xFFFFFFFFFFFFFFFF,
                                         request_ids.data_ptr(), step_ids.data_ptr(), out.data_ptr(),
                                         err.data_ptr(), stream), "sample_temperature")


def uniform_draws(seed: int, request_ids, step_ids, out, stream) -> None:
    check(core().iert_uniform_draws(seed & 0xFFFFFFFFFFFFFFFF, request_ids.data_ptr(),
                                    step_ids.data_ptr(), out.data_ptr(), out.numel(), stream),
          "uniform_draws")


class GemmScratch:
    """Scratch memory and ticket counters of the tensor-core projection's split-K path, shared
    by every launch on one stream of one device."""

    _by_device = {}

    def __init__(self, device):
        lib = core()
        self.ws = torch.empty(lib.iert_gemm_tc_workspace_bytes(), dtype=torch.uint8, device=device)
        self.counters = torch.zeros(lib.iert_gemm_tc_counter_count(), dtype=torch.int32, device=device)

    @classmethod
    def get(cls, device) -> "GemmScratch":
        key = str(torch.device(device))
        if key not in cls._by_device:
            cls._by_device[key] = cls(device)
        return cls._by_device[key]


def gemm_tc_set_poll_limit(polls: int) -> None:
    """Polls of a tile's counter before a CTA of the split-K projection gives up waiting for the tile's other
    CTAs (0: the default, about a second).  For tests of that bounded wait."""
    core().iert_gemm_tc_set_poll_limit(int(polls))


def gemm_tc(x, w, out, M: int, mode: int, err, stream, force_bt: int = 0, force_splits: int = 0,
            force_stages: int = 0) -> bool:
    """out[:M] (=|+=) x[:M] @ w.T on the tensor cores (bf16 operands).  Returns False, having
    launched nothing, when the operands do not meet the kernel's alignment rules."""
    N, K = w.shape
    sc = GemmScratch.get(x.device)
    status = core().iert_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                 dtype_code(out.dtype), out.stride(0), M, N, K, mode, sc.ws.data_ptr(),
                                 sc.ws.numel(), sc.counters.data_ptr(), sc.counters.numel(), force_bt,
                                 force_splits, force_stages, err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc")
    return True


def gemm_rows(x, w, out, M: int, mode: int, err, stream, scale: Optional[RowScale] = None,
              ahead: Optional[NormAhead] = None, force_stages: int = 0) -> bool:
    """out[:M] (=|+=) x[:M] @ w.T for one-token steps (M <= 32, bf16 operands): 16 weight rows per
    CTA over all of k, no split-K.  `scale`: x is the first half of an RMSNorm and the outputs
    are multiplied by the rows' 1 / rms; `ahead` (with a residual add): the first half of the
    next norm is written beside the new rows and `ahead.parts` is set.  Returns False, having
    launched nothing, when the operands do not meet the kernel's rules."""
    N, K = w.shape
    status = core().iert_gemm_rows(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                   dtype_code(out.dtype), out.stride(0), M, N, K, mode,
                                   byref(scale) if scale is not None else None,
                                   byref(ahead) if ahead is not None else None, force_stages,
                                   err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_rows")
    return True


def gemm_tc_scaled(x, w, out, M: int, mode: int, err, stream, scale: Optional[RowScale] = None,
                   ahead: Optional[NormAhead] = None, force_bt: int = 0, force_splits: int = 0) -> bool:
    """`gemm_tc` for one-token steps of 17 to 64 tokens with an RMSNorm split around the kernel: `scale`
    (x is a norm's first half: outputs times the rows' 1 / rms) and / or `ahead` (a residual add that
    also writes the next norm's first half; `ahead.parts` is set).  False, nothing launched, where
    the launch would not go through the split-K reduction."""
    N, K = w.shape
    sc = GemmScratch.get(x.device)
    status = core().iert_gemm_tc_scaled(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                        dtype_code(out.dtype), out.stride(0), M, N, K, mode, sc.ws.data_ptr(),
                                        sc.ws.numel(), sc.counters.data_ptr(), sc.counters.numel(),
                                        byref(scale) if scale is not None else None,
                                        byref(ahead) if ahead is not None else None, force_bt, force_splits,
                                        err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc_scaled")
    return True


def gemm_tc_gated_scaled(x, w, act, M: int, scale: RowScale, err, stream, force_bt: int = 0) -> bool:
    """`gemm_tc_gated` in its one-token form for an x that is the first half of an RMSNorm: gate and
    up are multiplied by the rows' 1 / rms before the activation."""
    two_i, K = w.shape
    status = core().iert_gemm_tc_gated_scaled(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), act.data_ptr(),
                                              act.stride(0), M, two_i // 2, K, byref(scale), force_bt,
                                              err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc_gated_scaled")
    return True


def attention_decode_scratch_floats(n_tokens: int, heads: int, head_dim: int, splits: int) -> int:
    return core().iert_attention_decode_scratch_floats(n_tokens, heads, head_dim, splits)


def attention_decode(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, splits: int,
                     scratch, err, stream) -> bool:
    """Split-KV decode attention (bf16 cache).  Returns False, having launched nothing, when
    the kernel does not take the cache's geometry."""
    status = core().iert_attention_decode(qkv.data_ptr(), out.data_ptr(), byref(batch), byref(kv), heads,
                                          scale, splits, scratch.data_ptr(), err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "attention_decode")
    global launch_count
    launch_count += 1          # the combine pass
    return True


_attn_libs = {}


def _attention_lib(head_dim: int):
    """The tensor-core attention library for one head size, compiled on first use."""
    lib = _attn_libs.get(head_dim)
    if lib is None:
        lib = build.load_library(*build.attention_library(head_dim))
        lib.iert_attention_prefill.argtypes = [c_void_p, c_void_p, POINTER(BatchView), c_int, c_int, c_int,
                                               c_float, c_int, c_void_p]
        lib.iert_attention_prefill.restype = c_int
        lib.iert_attention_decode_tc.argtypes = [c_void_p, c_void_p, POINTER(BatchView), POINTER(KvView), c_int,
                                                 c_float, c_int, c_int, c_void_p, c_void_p, c_void_p]
        lib.iert_attention_decode_tc.restype = c_int
        lib.iert_attention_decode_tc_rope.argtypes = [c_void_p, c_void_p, POINTER(BatchView), POINTER(KvView), c_int,
                                                      c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                      c_void_p, c_void_p]
        lib.iert_attention_decode_tc_rope.restype = c_int
        lib.iert_attention_prefill_tc.argtypes = [c_void_p, c_void_p, POINTER(BatchView), c_int, c_int, c_int,
                                                  c_float, c_int, c_void_p, c_void_p]
        lib.iert_attention_prefill_tc.restype = c_int
        lib.iert_attention_prefill_tc_available.restype = c_int
        lib.iert_attention_decode_tc_ctas_per_sm.restype = c_int
        if os.environ.get("IERT_PDL", "1") == "0":
            lib.iert_set_pdl(0)
        _attn_libs[head_dim] = lib
    return lib


def attention_prefill(qkv, out, batch: BatchView, heads: int, kv_heads: int, head_dim: int, window: int,
                      scale: float, max_q_len: int, stream, err=None, legacy: bool = False) -> bool:
    """Flash prompt attention (bf16) over the step's own keys and values.  Head sizes 64 and
    128 run on tcgen05 with the scores and the output in tensor memory (unless `legacy`); other
    multiples of 16 up to 256 run the mma.sync kernel.  The library is compiled per head size
    the first time it is needed; anything else returns False and nothing is launched."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        return False
    lib = _attention_lib(head_dim)
    global launch_count
    if not legacy and err is not None and lib.iert_attention_prefill_tc_available() \
            and os.environ.get("IERT_ATTN_TC", "1") != "0":
        status = lib.iert_attention_prefill_tc(qkv.data_ptr(), out.data_ptr(), byref(batch), heads, kv_heads,
                                               window, scale, max_q_len, err.data_ptr(), stream)
        if status == 0:
            launch_count += 1
            return True
        if status != 1:
            raise KernelError("attention_prefill_tc: the launch failed")
    status = lib.iert_attention_prefill(qkv.data_ptr(), out.data_ptr(), byref(batch), heads, kv_heads,
                                        window, scale, max_q_len, stream)
    if status == 1:
        return False
    if status != 0:
        raise KernelError("attention_prefill: the launch failed")
    launch_count += 1
    return True


def attention_decode_ctas_per_sm(head_dim: int) -> int:
    """CTAs of the tensor-core decode-attention kernels that one SM holds at once (a fact of those
    kernels, kept with them)."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"no tensor-core decode attention for head size {head_dim}")
    return int(_attention_lib(head_dim).iert_attention_decode_tc_ctas_per_sm())


def attention_decode_tc(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, splits: int,
                        scratch, err, stream, target_ctas: int = 0) -> bool:
    """Tensor-core split-KV decode attention (bf16 cache, 64-position pages, head sizes that
    are multiples of 16 up to 256).  Returns False, having launched nothing, otherwise."""
    hd = kv.head_dim
    if hd % 16 or not 16 <= hd <= 256:
        return False
    status = _attention_lib(hd).iert_attention_decode_tc(qkv.data_ptr(), out.data_ptr(), byref(batch), byref(kv),
                                                         heads, scale, splits, target_ctas, scratch.data_ptr(),
                                                         err.data_ptr(), stream)
    if status == 1:
        return False
    if status != 0:
        raise KernelError("attention_decode_tc: the launch failed")
    global launch_count
    launch_count += 1 if splits == 1 else 2        # a single split needs no merge kernel
    return True


def attention_decode_tc_rope(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, splits: int,
                             scratch, inv_freq, rotary_dim: int, pairing: int, store: bool, err, stream,
                             target_ctas: int = 0) -> bool:
    """`attention_decode_tc` with the rotary encoding and the step's cache write inside the
    kernel: `qkv` is the raw projection (one token per sequence) and stays as it is.  Returns
    False, having launched nothing, for anything the kernel does not take."""
    hd = kv.head_dim
    if hd % 16 or not 16 <= hd <= 256:
        return False
    status = _attention_lib(hd).iert_attention_decode_tc_rope(
        qkv.data_ptr(), out.data_ptr(), byref(batch), byref(kv), heads, scale, splits, target_ctas, scratch.data_ptr(),
        inv_freq.data_ptr(), rotary_dim, pairing, 1 if store else 0, err.data_ptr(), stream)
    if status == 1:
        return False
    if status != 0:
        raise KernelError("attention_decode_tc_rope: the launch failed")
    global launch_count
    launch_count += 1 if splits == 1 else 2        # a single split needs no merge kernel
    return True


def gemm_tc_gated(x, w, act, M: int, err, stream, force_bt: int = 0, force_stages: int = 0) -> bool:
    """act[:M] = silu(x @ w[:I].T) * (x @ w[I:].T) for w = [gate; up] with 2 I rows, on the tensor
    cores in one kernel.  Returns False, having launched nothing, when the operands do not meet
    the kernel's alignment rules."""
    two_i, K = w.shape
    status = core().iert_gemm_tc_gated(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), act.data_ptr(),
                                       act.stride(0), M, two_i // 2, K, force_bt, force_stages,
                                       err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc_gated")
    return True
