"""Weights from files to the device: the native reader against the tensors of the file, and the
loaded model's matrices against what the folder holds."""
import os

import pytest
import torch

from helpers import TINY_B, make_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_native_reader_fills_device_tensors(tmp_path):
    """Tensors of three dtypes and sizes from a few bytes to several chunks, with chunks that
    do not divide them and more threads than chunks: each arrives whole at its own address."""
    from inference_engine_rust_b200.weights import TensorSource, write_safetensors
    torch.manual_seed(1)
    tensors = {"big": torch.randn(3000, 1031).bfloat16(), "mid": torch.randn(257, 129), "small": torch.randn(3).bfloat16(),
               "table": torch.arange(1000, dtype=torch.int32), "empty": torch.empty(0, 8)}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    src = TensorSource(str(tmp_path))
    for threads, chunk in [(0, 0), (1, 1 << 20), (8, 100_003), (3, 4096)]:
        guard = torch.full((1 << 20,), 5, dtype=torch.uint8, device=DEV)     # neighbours must stay as they are
        targets = {n: torch.full(t.shape, 7, dtype=t.dtype, device=DEV) for n, t in tensors.items()}
        guard2 = torch.full((1 << 20,), 5, dtype=torch.uint8, device=DEV)
        src.read_into(targets, threads=threads, chunk_bytes=chunk)
        for n, t in tensors.items():
            assert torch.equal(targets[n].cpu(), t), (n, threads, chunk)
        assert bool((guard == 5).all()) and bool((guard2 == 5).all())


def test_fetch_many_keeps_the_dtype_policy(tmp_path):
    """bf16 stays bf16 and 32-bit stays 32-bit in a bfloat16 run (both read natively); f16 is
    widened, and a float32 run widens everything (both converted tensor by tensor)."""
    from inference_engine_rust_b200.weights import TensorSource, fetch_many, write_safetensors
    torch.manual_seed(2)
    tensors = {"w": torch.randn(40, 24).bfloat16(), "scale": torch.randn(24), "h": torch.randn(9, 5).half(),
               "ids": torch.arange(12, dtype=torch.int64)}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    src = TensorSource(str(tmp_path))
    got = fetch_many(src, list(tensors), torch.bfloat16, DEV)
    assert got["w"].dtype == torch.bfloat16 and got["scale"].dtype == torch.float32
    assert got["h"].dtype == torch.float32 and got["ids"].dtype == torch.int32
    for n, t in tensors.items():
        assert got[n].device.type == "cuda" and torch.equal(got[n].cpu().double(), t.double()), n
    got32 = fetch_many(src, ["w", "scale", "h"], torch.float32, DEV)
    assert all(v.dtype == torch.float32 for v in got32.values())
    assert torch.equal(got32["w"].cpu(), tensors["w"].float())


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_loaded_model_holds_the_folder_s_tensors(tmp_path, dtype):
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import TensorSource
    d = make_folder(tmp_path, TINY_B, seed=4, dtype="bfloat16")
    src = TensorSource(d)
    m = LoadedModel.load(d, dtype=dtype).model
    want_dt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    assert m.embedding.dtype == want_dt
    assert torch.equal(m.embedding.cpu(), src.get("model.embed_tokens.weight").to(want_dt))
    assert torch.equal(m.lm_head.weight.cpu(), src.get("lm_head.weight").to(want_dt))
    for i, (_, mixer, _, ffn) in enumerate(m._layer_parts):
        pre = f"model.layers.{i}."
        qkv = torch.cat([src.get(pre + f"self_attn.{p}_proj.weight") for p in "qkv"], dim=0).to(want_dt)
        assert torch.equal(mixer.qkv.weight.cpu(), qkv)
        assert torch.equal(mixer.o.weight.cpu(), src.get(pre + "self_attn.o_proj.weight").to(want_dt))


def test_a_folder_with_32_bit_scales_and_table_in_a_bfloat16_run(tmp_path):
    """Norm scales and the embedding table stored in 32-bit stay 32-bit in a bfloat16 run (the
    kernels read them as they are), matrices stay bfloat16; the model still agrees with the
    plain implementation run on exactly these values."""
    from helpers import TINY_A, compare, plain_weights, prompts_for
    from plain import mistral_plain as P
    from inference_engine_rust_b200 import LoadedModel
    from inference_engine_rust_b200.weights import TensorSource, write_safetensors
    d = make_folder(tmp_path, TINY_A, seed=9, dtype="bfloat16")
    src = TensorSource(d)
    torch.manual_seed(0)
    tensors = {}
    for n in src.names():
        t = src.get(n).clone()
        if n.endswith("norm.weight") or n == "model.embed_tokens.weight":
            t = t.float() + 1e-3 * torch.randn(t.shape)          # values that bfloat16 cannot hold
        tensors[n] = t
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    loaded = LoadedModel.load(d, dtype="bfloat16")
    m = loaded.model
    assert m.embedding.dtype == torch.float32 and torch.equal(m.embedding.cpu(), tensors["model.embed_tokens.weight"])
    assert m.final_norm.weight.dtype == torch.float32 and torch.equal(m.final_norm.weight.cpu(), tensors["model.norm.weight"])
    norm1, mixer, _, ffn = m._layer_parts[1]
    assert torch.equal(norm1.weight.cpu(), tensors["model.layers.1.input_layernorm.weight"])
    assert mixer.qkv.weight.dtype == torch.bfloat16 and ffn.down.weight.dtype == torch.bfloat16
    prompt = prompts_for(TINY_A, [37], seed=2)[0]
    eng = loaded.session(max_tokens=128, poison_cache=True).engine
    slot = eng.open_sequence()
    got = eng.step([(slot, prompt)], want="all")
    eng.check_device()
    compare(got, P.forward(TINY_A, plain_weights(d), prompt, P.bf16_rounding), "bfloat16", "32-bit scales and table")
