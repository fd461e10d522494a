"""The decode-attention entry point that allocates nothing (`iert_attention_decode_static`),
called through its exported C symbol, against the ordinary entry point.

Who needs it: hosts of the library that may not allocate device memory while they run: a
process whose GPU memory was handed out once at start-up, code that is called where a
cudaMalloc would stall or is forbidden, a loop with a fixed memory budget.  They cannot give
`iert_attention_decode` the scratch buffer it asks for, so this variant keeps the partial
results of the key splits in a fixed 8 MiB array inside the library image.

Checked here: two calls in a row give what the ordinary entry point gives (the array keeps
the first call's contents, and the second call must not be disturbed by them), a call that
would need more than the array holds is refused with its own status and launches nothing,
the messages name the limit, and, after one warm-up call (which may load the library's code
and its array onto the device), further calls leave the device's free memory as the driver
reports it (cudaMemGetInfo) exactly where it was: torch's own counter cannot see a
cudaMalloc made behind its back, the driver's can.  The file is collected last on purpose, and it passes alone
in a fresh process as well as after the other tests.
"""
import ctypes
import math
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_longlong, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def library():
    from inference_engine_rust_b200.csrc import bindings as B
    lib = B.core()
    fn = lib.iert_attention_decode_static
    fn.argtypes = [c_void_p, c_void_p, POINTER(B.BatchView), POINTER(B.KvView), c_int, c_float, c_int,
                   c_void_p, c_void_p]
    fn.restype = c_int
    lib.iert_attention_decode_static_capacity.restype = c_longlong
    lib.iert_attention_decode_static_message.argtypes = [c_int]
    lib.iert_attention_decode_static_message.restype = c_char_p
    return lib, B


def decoding_batch(B, heads, kvh, hd, window, lens, seed):
    """A cache filled with `lens[i] - 1` tokens per sequence and the packed projection of one
    more token each (keys and values already stored), as the attention kernel receives it."""
    from inference_engine_rust_b200.cache import Cache, KVRequest
    torch.manual_seed(seed)
    pages = sum(-(-n // 64) for n in lens)
    cache = Cache({0: KVRequest(kvh, hd, window)}, max_tokens=64 * pages, max_seq_len=1024,
                  max_sequences=len(lens), dtype=torch.bfloat16, device=DEV, poison=True)
    slots = [cache.open_sequence() for _ in lens]
    for s, n in zip(slots, lens):
        cache.reserve(s, n)
    cache.upload()
    kv = cache.layer_view(0).struct
    width = heads + 2 * kvh
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ident = torch.zeros(hd // 2, device=DEV)
    stream = B.stream_ptr()

    def batch_view(q_lens, pos0, which):
        n = len(q_lens)
        cu = np.zeros(n + 1, dtype=np.int32)
        cu[1:] = np.cumsum(q_lens)
        arrs = [torch.tensor(a, dtype=torch.int32, device=DEV) for a in
                (cu, which, np.repeat(np.arange(n, dtype=np.int32), q_lens), pos0)]
        return B.BatchView(cu_q=arrs[0].data_ptr(), slot_ids=arrs[1].data_ptr(), tok_seq=arrs[2].data_ptr(),
                           pos0=arrs[3].data_ptr(), n_seqs=n, n_tokens=int(cu[-1])), arrs

    filled = [(s, n - 1) for s, n in zip(slots, lens) if n > 1]
    if filled:
        view, keep = batch_view([n for _, n in filled], [0] * len(filled), [s for s, _ in filled])
        past = (torch.randn(sum(n for _, n in filled), width * hd, device=DEV) * 0.7).bfloat16()
        B.rope_kv_store(past, view, kv, ident, heads, hd, B.PAIR_HALF, True, err, stream)
    view1, keep1 = batch_view([1] * len(lens), [n - 1 for n in lens], slots)
    step = (torch.randn(len(lens), width * hd, device=DEV) * 0.7).bfloat16()
    B.rope_kv_store(step, view1, kv, ident, heads, hd, B.PAIR_HALF, True, err, stream)
    torch.cuda.synchronize()
    assert err.item() == 0
    return cache, kv, view1, keep1, step, err


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    lib, B = library()
    cases = [((32, 8, 128, 4096), [700, 33, 1, 64, 437], 5),      # Mistral's geometry
             ((6, 1, 32, 40), [5, 300, 90], 3)]                     # another one: contents of the array change shape
    for round_no, ((heads, kvh, hd, window), lens, splits) in enumerate(cases * 2):
        cache, kv, view, keep, step, err = decoding_batch(B, heads, kvh, hd, window, lens, seed=round_no)
        scale = 1.0 / math.sqrt(hd)
        n = B.attention_decode_scratch_floats(len(lens), heads, hd, splits)
        scratch = torch.empty(n, device=DEV)
        want = torch.full((len(lens), heads * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
        assert B.attention_decode(step, want, view, kv, heads, scale, splits, scratch, err, B.stream_ptr())
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        status = lib.iert_attention_decode_static(step.data_ptr(), got.data_ptr(), byref(view), byref(kv), heads,
                                                  scale, splits, err.data_ptr(), B.stream_ptr())
        assert status == 0, lib.iert_attention_decode_static_message(status).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert err.item() == 0 and torch.isfinite(got).all()
        # same kernels, same split order: the tolerance of the kernel tests holds with room to spare
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), f"call {round_no}"
        assert torch.equal(got, want), f"call {round_no}: the two entry points run the same arithmetic"


def test_calls_after_the_first_take_no_device_memory():
    """The free device memory that the driver reports does not move over a run of calls, once a
    first call has loaded what the runtime loads lazily.  torch allocates nothing in between
    either (its tensors are made before), so any change would be the library's."""
    lib, B = library()
    heads, kvh, hd, splits = 32, 8, 128, 4
    lens = [300, 64, 700, 1]
    cache, kv, view, keep, step, err = decoding_batch(B, heads, kvh, hd, None, lens, seed=21)
    scale = 1.0 / math.sqrt(hd)
    got = torch.zeros((len(lens), heads * hd), device=DEV, dtype=torch.bfloat16)
    call = lambda: lib.iert_attention_decode_static(step.data_ptr(), got.data_ptr(), byref(view), byref(kv), heads,
                                                    scale, splits, err.data_ptr(), B.stream_ptr())
    assert call() == 0                         # warm-up: address look-up, lazy loading of the kernels
    torch.cuda.synchronize()
    free_before, total = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    for _ in range(8):
        assert call() == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes over 8 calls"
    assert torch.cuda.memory_allocated() == torch_before
    assert err.item() == 0 and torch.isfinite(got).all()


def test_a_call_beyond_the_fixed_array_is_refused():
    lib, B = library()
    cap = lib.iert_attention_decode_static_capacity()
    assert cap == 2 * 1024 * 1024
    heads, kvh, hd = 32, 8, 128
    lens = [40] * 64
    cache, kv, view, keep, step, err = decoding_batch(B, heads, kvh, hd, None, lens, seed=9)
    out = torch.full((64, heads * hd), 7.0, device=DEV, dtype=torch.bfloat16)
    assert B.attention_decode_scratch_floats(64, heads, hd, 16) > cap
    status = lib.iert_attention_decode_static(step.data_ptr(), out.data_ptr(), byref(view), byref(kv), heads,
                                              0.1, 16, err.data_ptr(), B.stream_ptr())
    torch.cuda.synchronize()
    assert status == 3
    assert b"8 MiB" in lib.iert_attention_decode_static_message(status)
    assert float((out.float() - 7.0).abs().sum()) == 0.0            # nothing was launched
    # the same batch with fewer splits fits and runs
    assert B.attention_decode_scratch_floats(64, heads, hd, 4) <= cap
    status = lib.iert_attention_decode_static(step.data_ptr(), out.data_ptr(), byref(view), byref(kv), heads,
                                              0.1, 4, err.data_ptr(), B.stream_ptr())
    torch.cuda.synchronize()
    assert status == 0 and torch.isfinite(out).all() and err.item() == 0
