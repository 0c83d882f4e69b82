"""Weights: safetensors by tensor name, dtypes, the one error that lists everything wrong, random models."""
import json
import os

import numpy as np
import pytest
import torch

import helpers as H
from infer_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, expected_tensors, load_weights,
                                random_weights, write_random_model, write_safetensors)


def test_random_model_round_trip(tmp_path):
    cfg = H.TINY["b"]
    spec = write_random_model(str(tmp_path), cfg, seed=3, dtype=torch.bfloat16)
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen2ForCausalLM"]
    W = load_weights(str(tmp_path), spec)
    ref = random_weights(spec, 3, torch.bfloat16)
    assert set(W) == set(ref) == set(expected_tensors(spec))
    assert all(W[k].dtype == torch.bfloat16 and torch.equal(W[k], ref[k]) for k in W)
    assert "lm_head.weight" in W                       # untied
    # a different seed gives different values; the same seed the same
    assert not torch.equal(random_weights(spec, 4, torch.bfloat16)["lm_head.weight"], ref["lm_head.weight"])
    norm = W["model.norm.weight"].float()
    assert abs(norm.mean() - 1.0) < 0.1 and W["lm_head.weight"].float().std() < 0.03


def test_stored_precision_is_kept(tmp_path):
    t = {"bf": torch.randn(4, 6).bfloat16(), "f32": torch.randn(3), "f16": torch.randn(5).half(),
         "i64": torch.arange(7, dtype=torch.int64), "i32": torch.arange(3, dtype=torch.int32)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert f.get("bf").dtype == torch.bfloat16 and torch.equal(f.get("bf"), t["bf"])
    assert f.get("f32").dtype == torch.float32 and torch.equal(f.get("f32"), t["f32"])
    assert f.get("f16").dtype == torch.float32 and torch.equal(f.get("f16"), t["f16"].float())
    assert f.get("i64").dtype == torch.int32 and f.get("i32").dtype == torch.int32
    assert f.get("i64").tolist() == list(range(7))
    f.close()


def test_one_error_lists_everything(tmp_path):
    cfg = H.TINY["a"]
    spec = H.spec_of(cfg)
    W = random_weights(spec, 1, torch.float32)
    del W["model.layers.1.mlp.up_proj.weight"]
    del W["model.norm.weight"]
    W["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    W["model.layers.0.extra.weight"] = torch.zeros(2)
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), W)
    with pytest.raises(WeightsError) as e:
        load_weights(str(tmp_path / "m"), spec)
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.0.extra.weight" in msg
    assert "model.layers.0.self_attn.q_proj.weight" in msg and "[64, 64]" in msg and "[64, 63]" in msg
    assert e.value.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.0.extra.weight"]


def test_tied_model_has_no_head_tensor():
    assert "lm_head.weight" not in expected_tensors(H.spec_of(H.TINY["a"]))
    assert "model.layers.0.self_attn.q_proj.bias" not in expected_tensors(H.spec_of(H.TINY["c"]))


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(str(p))
    p.write_bytes((1000).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="bad offsets"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        load_weights(str(tmp_path), H.spec_of(H.TINY["a"]))


def test_sharded_checkpoint(tmp_path):
    spec = H.spec_of(H.TINY["a"])
    W = random_weights(spec, 2, torch.bfloat16)
    names = sorted(W)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: W[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: W[n] for n in names[half:]})
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_weights(str(tmp_path), spec)
    assert all(torch.equal(got[n], W[n]) for n in names)
