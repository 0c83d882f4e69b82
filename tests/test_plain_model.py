"""The plain implementation against the reference engine's own CPU forward (tests/golden), and its parts."""
import json
import os

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as pm

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_matches_reference_forward(name):
    meta = json.load(open(os.path.join(GOLD, "golden.json")))[name]
    W = H.make_weights(meta["config"], meta["seed"], torch.bfloat16)
    gold = np.load(os.path.join(GOLD, name + "_logits.npy"))
    got = pm.forward(meta["config"], W, meta["ids"]).numpy()
    assert got.shape == gold.shape
    assert np.abs(got - gold).max() < 5e-6             # the reference accumulates in float32
    assert (got.argmax(-1) == gold.argmax(-1)).all()
    assert pm.greedy_decode(meta["config"], W, meta["ids"], len(meta["greedy"])) == meta["greedy"]


def test_rope_is_half_split_and_position_zero_is_identity():
    cos, sin = pm.rope_tables(10000.0, 8, 3)
    x = torch.arange(24, dtype=torch.float64).view(3, 1, 8)
    y = pm.apply_rope(x, cos, sin)
    assert torch.equal(y[0], x[0])
    j, p = 1, 2
    c, s = cos[p, j], sin[p, j]
    assert torch.isclose(y[p, 0, j], x[p, 0, j] * c - x[p, 0, j + 4] * s)
    assert torch.isclose(y[p, 0, j + 4], x[p, 0, j + 4] * c + x[p, 0, j] * s)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8, dtype=torch.float64), torch.randn(6, 2, 8, dtype=torch.float64), torch.randn(6, 2, 8, dtype=torch.float64)
    out = pm.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # head 3 reads kv head 1
    k2 = k.clone(); k2[5] += 1.0
    assert torch.allclose(pm.attention(q, k2, v)[:5], out[:5])                           # the future is not seen
    w1 = pm.attention(q, k, v, window=1)
    assert torch.allclose(w1[:, 0], v[:, 0])                                              # a window of one sees itself only
    w3 = pm.attention(q, k, v, window=3)
    k3 = k.clone(); k3[0] += 5.0
    assert torch.allclose(pm.attention(q, k3, v, window=3)[3:], w3[3:])                   # position 0 is outside from t=3 on


def test_rmsnorm_and_silu():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = pm.rmsnorm(x, torch.tensor([1.0, 2.0]), 0.5)
    assert torch.allclose(y, x / np.sqrt(12.5 + 0.5) * torch.tensor([1.0, 2.0], dtype=torch.float64))
    assert abs(float(pm.silu(torch.tensor(1.0, dtype=torch.float64))) - 1 / (1 + np.exp(-1))) < 1e-12


def test_sampler_twin():
    row = np.array([0.1, 2.0, 2.0, -1.0], dtype=np.float32)
    assert pm.sample(row, 0.0, 0, 0) == 1                      # ties go to the lowest id
    a = [pm.sample(row, 0.8, 7, s) for s in range(50)]
    assert a == [pm.sample(row, 0.8, 7, s) for s in range(50)]  # same seed, same stream
    assert a != [pm.sample(row, 0.8, 8, s) for s in range(50)]
    counts = np.bincount([pm.sample(row, 1.0, 3, s) for s in range(4000)], minlength=4) / 4000
    p = np.exp(row - row.max()); p /= p.sum()
    assert 0.5 * np.abs(counts - p).sum() < 0.03               # total variation
