"""Weights: safetensors round trip, storage dtypes, one error listing every fault, random mode."""
import json
import os
import struct

import pytest
import torch

from qwen_decoder_b200.config import Qwen2Config, describe_model
from qwen_decoder_b200.parts import build_model
from qwen_decoder_b200.weights import (SafetensorsError, SafetensorsFile, TensorSource, WeightError,
                                       check_tensors, save_safetensors, storage_dtype, write_random_model)
from tiny_configs import TINY_A, TINY_B


def test_safetensors_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {"a": torch.randn(3, 5, generator=g).to(torch.bfloat16), "b": torch.randn(7, generator=g),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "d": torch.randn(2, 2, generator=g).half()}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, tensors, {"k": "v"})
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c", "d"] and f.metadata == {"k": "v"}
    for n, t in tensors.items():
        assert torch.equal(f.tensor(n), t) and f.tensor(n).dtype == t.dtype
    # the official reader agrees
    from safetensors import safe_open
    with safe_open(p, framework="pt") as sf:
        for n, t in tensors.items():
            assert torch.equal(sf.get_tensor(n), t)


def test_truncated_and_malformed_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, {"a": torch.zeros(100)})
    data = open(p, "rb").read()
    open(p, "wb").write(data[:-40])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        TensorSource.from_folder(str(tmp_path))


def test_storage_rule():
    assert storage_dtype(torch.bfloat16) == torch.bfloat16      # kept
    assert storage_dtype(torch.float32) == torch.float32        # a tensor stored in 32-bit stays so
    assert storage_dtype(torch.float16) == torch.float16        # kept exactly: bind rounds once, or not at all
    assert storage_dtype(torch.int64) == torch.int32            # integer tables
    src = TensorSource.from_dict({"a": torch.ones(2, dtype=torch.float16), "b": torch.ones(2),
                                  "i": torch.ones(2, dtype=torch.int64)})
    assert src.get("a").dtype == torch.float16 and src.get("b").dtype == torch.float32
    assert src.get("i").dtype == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_B)
    folder = write_random_model(cfg, str(tmp_path), seed=1)
    model = build_model(describe_model(cfg))
    check_tensors(model.tensor_specs(), TensorSource.from_folder(folder).shapes)      # fits
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n) for n in f.names()}
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["lm_head.weight"]
    tensors["model.layers.9.mlp.up_proj.weight"] = torch.zeros(2, 2)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(128, 351)
    with pytest.raises(WeightError) as ei:
        check_tensors(model.tensor_specs(), TensorSource.from_dict(tensors).shapes, "test")
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.k_proj.bias"]
    assert e.unexpected == ["model.layers.9.mlp.up_proj.weight"]
    assert e.wrong_shape == [("model.layers.0.mlp.down_proj.weight", (128, 352), (128, 351))]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shapes", "lm_head.weight", "expected [128, 352], found [128, 351]"):
        assert word in msg


def test_tied_model_has_no_output_matrix(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    names = [s.name for s in build_model(describe_model(cfg)).tensor_specs()]
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names
    assert "model.layers.1.self_attn.q_proj.bias" in names and "model.layers.0.self_attn.o_proj.bias" not in names


def test_tied_model_leaves_a_stored_output_matrix_aside(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    model = build_model(describe_model(cfg))
    shapes = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    shapes["lm_head.weight"] = (cfg.vocab_size, cfg.hidden_size)
    with pytest.warns(UserWarning, match="not used by this configuration: lm_head.weight"):
        check_tensors(model.tensor_specs(), shapes, "test", model.ignorable_tensors())
    shapes["model.extra.weight"] = (1,)
    with pytest.raises(WeightError) as ei, pytest.warns(UserWarning):
        check_tensors(model.tensor_specs(), shapes, "test", model.ignorable_tensors())
    assert ei.value.unexpected == ["model.extra.weight"]


def test_random_mode_is_seeded_and_order_free(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    a = write_random_model(cfg, str(tmp_path / "a"), seed=0)
    b = write_random_model(cfg, str(tmp_path / "b"), seed=0)
    c = write_random_model(cfg, str(tmp_path / "c"), seed=1)
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    assert not torch.equal(fa.tensor("model.embed_tokens.weight"), fc.tensor("model.embed_tokens.weight"))
    w = fa.tensor("model.layers.0.mlp.up_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 2e-3 and fa.tensor("model.norm.weight").dtype == torch.bfloat16
    nw = fa.tensor("model.layers.1.input_layernorm.weight").float()
    assert abs(float(nw.mean()) - 1.0) < 0.1
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen2ForCausalLM"]


def test_a_folder_of_shards_with_an_index(tmp_path):
    """model.safetensors.index.json + shards: every tensor is found in the shard the index names, the
    model binds from it as from a single file, and an index that names a wrong shard is an error."""
    cfg = Qwen2Config.from_dict(TINY_B)
    single = write_random_model(cfg, str(tmp_path / "single"), seed=1)
    f = SafetensorsFile(os.path.join(single, "model.safetensors"))
    names = sorted(f.names())
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    with open(os.path.join(single, "config.json")) as src, open(sharded / "config.json", "w") as dst:
        dst.write(src.read())
    cut = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:cut], "model-00002-of-00002.safetensors": names[cut:]}
    weight_map = {}
    for fname, ns in parts.items():
        save_safetensors(str(sharded / fname), {n: f.tensor(n) for n in ns})
        weight_map.update({n: fname for n in ns})
    with open(sharded / "model.safetensors.index.json", "w") as fh:
        json.dump({"metadata": {}, "weight_map": weight_map}, fh)
    src = TensorSource.from_folder(str(sharded))
    model = build_model(describe_model(cfg))
    check_tensors(model.tensor_specs(), src.shapes)
    for n in names:
        assert torch.equal(src.get(n), f.tensor(n))
    # an index entry that points at the other shard
    weight_map[names[0]] = "model-00002-of-00002.safetensors"
    with open(sharded / "model.safetensors.index.json", "w") as fh:
        json.dump({"weight_map": weight_map}, fh)
    with pytest.raises(SafetensorsError, match="is not in shard"):
        TensorSource.from_folder(str(sharded))
