"""Weights by name: the container, the one error that lists everything wrong, the dtype
policy and the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_folder
from inference_engine_rust_b200 import Model, WeightError, config_from_dict, spec_of, write_random_model
from inference_engine_rust_b200.parts.base import Runtime
from inference_engine_rust_b200.weights import (RandomSource, SafetensorsError, TensorSource, TensorSpec,
                                                check_source, fetch, stored_dtype_policy, write_safetensors)


def cpu_model(cfg, dtype=torch.float32):
    return Model(spec_of(config_from_dict(cfg)), Runtime(dtype=dtype, device="cpu"))


def test_expected_names_and_shapes():
    exp = cpu_model(TINY_B).expected_tensors()
    assert exp["model.embed_tokens.weight"].shape == (384, 96)
    assert exp["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert exp["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert exp["model.layers.0.self_attn.o_proj.weight"].shape == (96, 192)
    assert exp["model.layers.1.mlp.gate_proj.weight"].shape == (160, 96)
    assert exp["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    assert exp["model.layers.0.input_layernorm.weight"].init == "ones_plus_normal"
    assert exp["lm_head.weight"].shape == (384, 96) and exp["model.norm.weight"].shape == (96,)
    assert len(exp) == 3 + 3 * 9
    assert "lm_head.weight" not in cpu_model(dict(TINY_B, tie_word_embeddings=True)).expected_tensors()


def test_folder_round_trip_matches_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file
    d = make_folder(tmp_path, TINY_A, seed=5, dtype="bfloat16")
    theirs = load_file(os.path.join(d, "model.safetensors"))
    ours = TensorSource(d)
    assert sorted(ours.names()) == sorted(theirs)
    for n in ours.names():
        assert theirs[n].dtype == torch.bfloat16 and torch.equal(ours.get(n), theirs[n])
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["MistralForCausalLM"]
    w = theirs["model.layers.0.input_layernorm.weight"].float()
    assert abs(w.mean().item() - 1) < 0.1                      # norm scales are 1 + N(0, std)
    assert abs(theirs["model.embed_tokens.weight"].float().std().item() - 0.1) < 0.01


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    exp = cpu_model(TINY_A).expected_tensors()
    a, b, c = RandomSource(exp, 1), RandomSource(exp, 1), RandomSource(exp, 2)
    n = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(a.get(n), b.get(n)) and not torch.equal(a.get(n), c.get(n))
    assert not torch.equal(a.get(n), a.get("model.layers.0.mlp.up_proj.weight"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_folder(tmp_path, TINY_A, seed=1)
    src = TensorSource(d)
    tensors = {n: src.get(n).clone() for n in src.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.7.extra.weight"] = torch.zeros(3)
    tensors["lm_head.weight"] = torch.zeros(256, 63)
    bad = tmp_path / "bad"
    bad.mkdir()
    write_safetensors(str(bad / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        cpu_model(TINY_A).load(TensorSource(str(bad)), where=str(bad))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("lm_head.weight", (256, 63), (256, 64))]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "model.norm.weight", "[256, 63]"):
        assert needle in text


def test_a_folder_of_another_size_is_refused(tmp_path):
    d = make_folder(tmp_path, TINY_A, seed=1)
    with pytest.raises(WeightError) as e:
        cpu_model(TINY_B).load(TensorSource(d), where=d)
    assert e.value.wrong_shape and e.value.missing


def test_dtype_policy():
    bf, f32, f16, i64 = (torch.zeros(2, dtype=t) for t in (torch.bfloat16, torch.float32, torch.float16, torch.int64))
    assert stored_dtype_policy(bf, torch.bfloat16) == torch.bfloat16
    assert stored_dtype_policy(f32, torch.bfloat16) == torch.float32       # stored in 32-bit stays so
    assert stored_dtype_policy(f16, torch.bfloat16) == torch.float32
    assert stored_dtype_policy(bf, torch.float32) == torch.float32         # widened for the 32-bit run
    assert stored_dtype_policy(i64, torch.bfloat16) == torch.int32


def test_mixed_storage_is_kept(tmp_path):
    d = make_folder(tmp_path, TINY_A, seed=2, dtype="bfloat16")
    src = TensorSource(d)
    tensors = {n: src.get(n).clone() for n in src.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    mixed = tmp_path / "mixed"
    mixed.mkdir()
    write_safetensors(str(mixed / "model.safetensors"), tensors)
    m = cpu_model(TINY_A, torch.bfloat16)
    m.load(TensorSource(str(mixed)))
    assert m.final_norm.weight.dtype == torch.float32
    assert m.blocks[0].norm1.weight.dtype == torch.bfloat16
    assert m.blocks[0].mixer.qkv.weight.dtype == torch.bfloat16 and m.blocks[0].mixer.qkv.weight.shape == (128, 64)
    m32 = cpu_model(TINY_A, torch.float32)
    m32.load(TensorSource(str(mixed)))
    assert m32.blocks[0].norm1.weight.dtype == torch.float32 and m32.embedding.dtype == torch.float32


def test_fused_rows_are_q_then_k_then_v(tmp_path):
    d = make_folder(tmp_path, TINY_B, seed=3)
    src = TensorSource(d)
    m = cpu_model(TINY_B)
    m.load(src)
    w = m.blocks[1].mixer.qkv.weight
    p = "model.layers.1.self_attn."
    assert torch.equal(w[:192], src.get(p + "q_proj.weight")) and torch.equal(w[192:224], src.get(p + "k_proj.weight"))
    assert torch.equal(w[224:], src.get(p + "v_proj.weight"))
    gu = m.blocks[1].ffn.gate_up.weight
    assert torch.equal(gu[:160], src.get("model.layers.1.mlp.gate_proj.weight"))
    assert torch.equal(gu[160:], src.get("model.layers.1.mlp.up_proj.weight"))


def test_malformed_containers(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError):
        TensorSource(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError):
        TensorSource(str(tmp_path))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError) as e:
        TensorSource(str(tmp_path))
    assert "data_offsets" in str(e.value)
    with pytest.raises(SafetensorsError):
        TensorSource(str(tmp_path / "empty_dir_that_is_not_there"))


def test_sharded_folder(tmp_path):
    t = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": torch.ones(4, dtype=torch.bfloat16)}
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": t["a"]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": t["b"]})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    src = TensorSource(str(tmp_path))
    assert torch.equal(src.get("a"), t["a"]) and torch.equal(src.get("b"), t["b"])
    assert src.describe("b") == ("BF16", (4,))
    # the native reader goes file by file
    into = {"b": torch.zeros(4, dtype=torch.bfloat16), "a": torch.zeros(2, 3)}
    src.read_into(into, threads=2, chunk_bytes=5)
    assert torch.equal(into["a"], t["a"]) and torch.equal(into["b"], t["b"])


def test_integer_tables_and_kind_check(tmp_path):
    write_safetensors(str(tmp_path / "model.safetensors"),
                      {"table": torch.arange(5, dtype=torch.int64), "w": torch.zeros(2, 2)})
    src = TensorSource(str(tmp_path))
    check_source({"table": TensorSpec((5,), "int_table"), "w": TensorSpec((2, 2))}, src, "x")
    assert fetch(src, "table", torch.bfloat16, "cpu").dtype == torch.int32
    with pytest.raises(WeightError) as e:
        check_source({"table": TensorSpec((5,)), "w": TensorSpec((2, 2), "int_table")}, src, "x")
    assert len(e.value.wrong_kind) == 2


# ---- the native reader (host destinations here; device destinations in the GPU tests) ----------

def test_native_reader_fills_host_tensors_in_any_chunking(tmp_path):
    """Every tensor of a file lands where it is sent, whatever the chunk size and the number of
    threads: chunks smaller than a row, chunks that do not divide a tensor, one thread or many."""
    torch.manual_seed(3)
    tensors = {"a": torch.randn(37, 53).bfloat16(), "b": torch.randn(1001), "c": torch.arange(77, dtype=torch.int32),
               "d": torch.randn(5, 3, 7).bfloat16(), "empty": torch.empty(0, 4)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors)
    src = TensorSource(str(tmp_path))
    for threads, chunk in [(1, 0), (3, 1000), (8, 13), (2, 1 << 20)]:
        targets = {n: torch.full_like(t, 7) for n, t in tensors.items()}
        src.read_into(targets, threads=threads, chunk_bytes=chunk)
        for n, t in tensors.items():
            assert torch.equal(targets[n], t), (n, threads, chunk)
    # a subset, in an order that is not the file's
    targets = {"d": torch.empty_like(tensors["d"]), "a": torch.empty_like(tensors["a"])}
    src.read_into(targets, threads=2, chunk_bytes=64)
    assert torch.equal(targets["a"], tensors["a"]) and torch.equal(targets["d"], tensors["d"])


def test_native_reader_refuses_wrong_destinations_and_reports_short_files(tmp_path):
    from inference_engine_rust_b200.weights.native_reader import ReadError, read_file_ranges
    t = torch.randn(64, 64)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {"w": t})
    src = TensorSource(str(tmp_path))
    with pytest.raises(SafetensorsError, match="destination"):
        src.read_into({"w": torch.empty(64, 64, dtype=torch.bfloat16)})
    with pytest.raises(SafetensorsError, match="destination"):
        src.read_into({"w": torch.empty(64, 65)[:, :64]})
    # the file loses its tail after it was opened: the reader says where it ends
    size = os.path.getsize(path)
    with open(path, "r+b") as f:
        f.truncate(size - 100)
    with pytest.raises(ReadError, match="the file ends at byte"):
        src.read_into({"w": torch.empty(64, 64)}, threads=2, chunk_bytes=4096)
    with pytest.raises(ReadError, match="cannot open"):
        read_file_ranges(str(tmp_path / "nothing"), [0], [4], [torch.empty(1).data_ptr()], -1)
    with pytest.raises(ReadError, match="negative"):
        read_file_ranges(path, [-1], [4], [torch.empty(1).data_ptr()], -1)


def test_fetch_many_without_a_device_goes_tensor_by_tensor(tmp_path):
    from inference_engine_rust_b200.weights import fetch_many
    d = make_folder(tmp_path, TINY_A, seed=2, dtype="bfloat16")
    src = TensorSource(d)
    names = src.names()[:5]
    got = fetch_many(src, names, torch.float32, "cpu")
    for n in names:
        assert got[n].dtype == torch.float32 and torch.equal(got[n], src.get(n).float())


def test_a_folder_without_the_output_head_ties_it_to_the_embedding(tmp_path):
    """src/model_weights/names.rs:300-310: no `output.weight` means the embedding table is the head,
    whatever the configuration's flag says."""
    d = make_folder(tmp_path, TINY_A, seed=4)
    src = TensorSource(d)
    tensors = {n: src.get(n).clone() for n in src.names() if n != "lm_head.weight"}
    bare = tmp_path / "no_head"
    bare.mkdir()
    write_safetensors(str(bare / "model.safetensors"), tensors)
    m = cpu_model(TINY_A)                                  # tie_word_embeddings is false in Tiny A
    m.load(TensorSource(str(bare)), where="no_head")
    assert m.lm_head.weight is m.embedding
    assert torch.equal(m.lm_head.weight, tensors["model.embed_tokens.weight"])
    assert any("tied" in n for n in m.notes)
    # the untouched folder keeps its own head
    m2 = cpu_model(TINY_A)
    m2.load(src)
    assert torch.equal(m2.lm_head.weight, src.get("lm_head.weight")) and m2.notes == []


def test_extra_tensors_are_an_error_unless_asked_otherwise(tmp_path):
    d = make_folder(tmp_path, TINY_B, seed=4)
    src = TensorSource(d)
    tensors = {n: src.get(n).clone() for n in src.names()}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["optimizer.step"] = torch.zeros(1)
    del tensors["model.norm.weight"]
    extra = tmp_path / "extra"
    extra.mkdir()
    write_safetensors(str(extra / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:                  # not strict: extras pass, what is missing does not
        cpu_model(TINY_B).load(TensorSource(str(extra)), strict=False)
    assert e.value.missing == ["model.norm.weight"] and e.value.unexpected == []
    tensors["model.norm.weight"] = src.get("model.norm.weight").clone()
    write_safetensors(str(extra / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        cpu_model(TINY_B).load(TensorSource(str(extra)))
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq", "optimizer.step"]
    m = cpu_model(TINY_B)
    m.load(TensorSource(str(extra)), strict=False)
    assert m.ignored_tensors == ["model.layers.0.self_attn.rotary_emb.inv_freq", "optimizer.step"]
    assert m.loaded and any("ignored" in n for n in m.notes)
