"""Weights: the container, loading by name with one error for all faults, random models."""
import json
import os
import struct

import pytest
import torch

import plain_llama
from helpers import TINY, make_model
from llmplayer_b200.config import config_from_dict, load_config
from llmplayer_b200.engine.model import Model
from llmplayer_b200.errors import WeightError
from llmplayer_b200.weights import SafetensorsFile, load_tensors, random_tensors, write_safetensors


def specs_of(model_dir):
    return Model(load_config(model_dir).layout()).tensor_specs()


def test_container_round_trip(tmp_path):
    t = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": torch.randn(4, 2).to(torch.bfloat16),
         "c": torch.tensor([1, 2, 3], dtype=torch.int32)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, metadata={"k": "v"})
    f = SafetensorsFile(path)
    assert set(f.keys()) == set(t) and f.metadata == {"k": "v"}
    for name, ref in t.items():
        assert torch.equal(f.tensor(name), ref) and f.tensor(name).dtype == ref.dtype
    f.close()
    other = plain_llama.read_safetensors(path)             # an independent reader agrees
    assert all(torch.equal(other[k], t[k]) for k in t)


def test_random_model_is_seeded_and_complete(tmp_path):
    a = make_model(tmp_path / "1", "A")
    b = make_model(tmp_path / "2", "A")
    ta, tb = plain_llama.read_safetensors(a + "/model.safetensors"), plain_llama.read_safetensors(b + "/model.safetensors")
    assert ta.keys() == tb.keys() and all(torch.equal(ta[k], tb[k]) for k in ta)
    assert "lm_head.weight" not in ta                        # tied
    assert "lm_head.weight" in plain_llama.read_safetensors(make_model(tmp_path, "B") + "/model.safetensors")
    norm = ta["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.05 and ta["model.embed_tokens.weight"].dtype == torch.bfloat16
    loaded = load_tensors(a, specs_of(a))
    assert set(loaded) == set(ta) and all(v.dtype == torch.bfloat16 for v in loaded.values())


def test_dtypes_are_kept(tmp_path):
    d = make_model(tmp_path, "A", dtype="float32")
    loaded = load_tensors(d, specs_of(d))
    assert all(v.dtype == torch.float32 for v in loaded.values())        # stored in 32 bits: stays so
    different = random_tensors(specs_of(d), seed=0, dtype="float32")
    assert torch.equal(different["model.norm.weight"], loaded["model.norm.weight"])


def test_one_error_lists_everything(tmp_path):
    d = make_model(tmp_path, "B", dtype="float32")
    path = os.path.join(d, "model.safetensors")
    t = plain_llama.read_safetensors(path)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(7, 96)
    t["model.layers.9.extra.weight"] = torch.zeros(2)
    t["lm_head.weight"] = torch.zeros(384, 96, dtype=torch.int32)
    write_safetensors(path, t)
    with pytest.raises(WeightError) as err:
        load_tensors(d, specs_of(d))
    text = str(err.value)
    for needle in ("missing (2)", "model.layers.1.mlp.up_proj.weight", "model.norm.weight", "unexpected (1)",
                   "model.layers.9.extra.weight", "model.layers.0.self_attn.k_proj.weight", "[32, 96]", "[7, 96]",
                   "lm_head.weight", "I32"):
        assert needle in text, needle


def test_tied_model_with_a_head_tensor_is_refused(tmp_path):
    d = make_model(tmp_path, "A", dtype="float32")
    path = os.path.join(d, "model.safetensors")
    t = plain_llama.read_safetensors(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(path, t)
    with pytest.raises(WeightError, match="unexpected.*lm_head.weight"):
        load_tensors(d, specs_of(d))


def test_broken_files(tmp_path):
    d = make_model(tmp_path, "A", dtype="float32")
    path = os.path.join(d, "model.safetensors")
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(WeightError, match="truncated|outside"):
        load_tensors(d, specs_of(d))
    open(path, "wb").write(struct.pack("<Q", 10 ** 12) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        load_tensors(d, specs_of(d))
    open(path, "wb").write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(WeightError, match="JSON"):
        load_tensors(d, specs_of(d))
    os.remove(path)
    with pytest.raises(WeightError, match="model.safetensors"):
        load_tensors(d, specs_of(d))


def test_sharded_folder(tmp_path):
    d = make_model(tmp_path, "A", dtype="float32")
    path = os.path.join(d, "model.safetensors")
    t = plain_llama.read_safetensors(path)
    names = sorted(t)
    half = len(names) // 2
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {n: t[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), {n: t[n] for n in names[half:]})
    os.remove(path)
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    json.dump(index, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    loaded = load_tensors(d, specs_of(d))
    assert all(torch.equal(loaded[n], t[n]) for n in names)
