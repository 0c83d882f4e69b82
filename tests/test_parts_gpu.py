"""Each part alone against the plain implementation; run orders that name a layer twice or read another layer's
cache; and a toy mixer with state of its own, registered from here without touching the framework."""
import math

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _rt(dtype, max_seq=256):
    from infer_b200.runtime import Runtime
    return Runtime(dtype=dtype, device=torch.device(DEV), max_seq_len=max_seq)


def _step(cache, entries):
    """A StepContext for entries [(rid, n_tokens)] built by a throw-away engine-like helper."""
    from infer_b200.engine.engine import Engine, StepEntry
    eng = Engine.__new__(Engine)
    eng.cache, eng.max_seq_len = cache, 10 ** 6
    eng.spec = type("S", (), {"vocab_size": 10 ** 6})()
    eng.rt = _rt(torch.float32)
    eng.status = torch.zeros(1, dtype=torch.int32, device=DEV)
    eng.next_tokens = torch.zeros(8, dtype=torch.int32, device=DEV)
    for rid, n in entries:
        if rid not in cache.requests:
            cache.admit(rid)
        assert cache.reserve(rid, n)
    ctx, _ = eng._build_context([StepEntry(rid, [0] * n, []) for rid, n in entries])
    return ctx


def _tol(dtype):
    return dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from infer_b200.config import PartSpec
    from infer_b200.parts import build_part
    part = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 2e-5}), _rt(dtype))
    w = 1 + 0.1 * torch.randn(72)
    part.load({"weight": w.bfloat16() if dtype == torch.bfloat16 else w})
    x = torch.randn(9, 72, device=DEV)
    got = part.forward(x)
    assert got.dtype == dtype
    wv = w.bfloat16().float() if dtype == torch.bfloat16 else w
    assert torch.allclose(got.cpu().double(), pm.rmsnorm(x.cpu().double(), wv, 2e-5), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from infer_b200.config import PartSpec
    from infer_b200.parts import build_part
    H_, I = 40, 104
    part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": H_, "intermediate_size": I}), _rt(dtype))
    W = {n: (torch.randn(s) * 0.2).to(dtype) for n, s in part.param_shapes(part.spec).items()}
    part.load(W)
    x = torch.randn(11, H_).to(dtype)
    res = torch.randn(11, H_)
    got = part.forward(x.to(DEV), res.clone().to(DEV))
    ref = res.double() + pm.swiglu_mlp(x.double(), W["gate_proj.weight"].float(), W["up_proj.weight"].float(),
                                       W["down_proj.weight"].float())
    assert got.dtype == torch.float32 and torch.allclose(got.cpu().double(), ref, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_in_portions(dtype, window):
    """The attention part alone, two requests cut differently, against the plain attention block on whole sequences."""
    from infer_b200.cache import CacheManager
    from infer_b200.config import PartSpec
    from infer_b200.parts import build_part
    Hd, nh, nkv, hd = 48, 6, 2, 16
    cfg = dict(hidden_size=Hd, num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, attention_bias=True)
    rot = PartSpec("rotary_half", {"head_dim": hd, "theta": 777.0, "max_positions": 256})
    spec = PartSpec("attention", {"hidden_size": Hd, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qkv_bias": True,
                                  "window": window, "softmax_scale": None, "position": rot})
    rt = _rt(dtype)
    part = build_part("mixer", spec, rt)
    W = {n: (torch.randn(s) * 0.3).to(dtype) for n, s in part.param_shapes(spec).items()}
    part.load(W)
    cache = CacheManager({0: part.cache_need()}, 12, 8, 2)
    cache.make_storage(dtype, DEV)
    view = cache.view(0)
    xs = {"a": torch.randn(37, Hd).to(dtype), "b": torch.randn(21, Hd).to(dtype)}
    cuts = [[("a", 5), ("b", 21)], [("a", 1)], [("a", 30)], [("a", 1)]]
    done = {"a": 0, "b": 0}
    outs = {"a": [], "b": []}
    for cut in cuts:
        ctx = _step(cache, cut)
        x = torch.cat([xs[r][done[r]:done[r] + n] for r, n in cut]).to(DEV)
        y = part.forward(x, ctx, view, torch.zeros(x.shape[0], Hd, device=DEV)).cpu()
        assert int(ctx.status.item()) == 0
        o = 0
        for r, n in cut:
            outs[r].append(y[o:o + n]); o += n
            cache.advance(r, n); done[r] += n
    cos, sin = pm.rope_tables(777.0, hd, 64)
    Wf = {"p." + k: v.float() for k, v in W.items()}
    for r in xs:
        T = xs[r].shape[0]
        ref = pm.attention_block(cfg, Wf, "p.", xs[r].double(), cos[:T], sin[:T], window)
        got = torch.cat(outs[r]).double()
        # outputs are O(10) here: the error is measured against their size
        rel = 2e-2 if dtype == torch.bfloat16 else 2e-6
        assert (got - ref).abs().max() <= rel * ref.abs().max(), (r, float((got - ref).abs().max()), float(ref.abs().max()))


def _toy_spec(cfg, schedule):
    from dataclasses import replace
    from infer_b200.config import LayerCall
    spec = H.spec_of(cfg)
    return replace(spec, schedule=tuple(LayerCall(*s) for s in schedule))


@pytest.mark.parametrize("dtype", DTYPES)
def test_run_order_may_repeat_a_layer_and_share_a_cache(dtype):
    """Run order: layer 0, layer 1, layer 0 again with a cache of its own, then layer 1 reading layer 0's first cache
    (it writes nothing; its queries meet the keys that call 0 stored)."""
    name = "a"
    cfg = H.TINY[name]
    from infer_b200.engine import Engine
    schedule = [(0, 0, True), (1, 1, True), (0, 2, True), (1, 0, False)]
    W = H.make_weights(name, 3)
    eng = Engine(_toy_spec(cfg, schedule), W, dtype=dtype, max_tokens=256, max_requests=2)
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].cache_ids == [0, 1, 2]
    ids = H.random_ids(cfg, 50, 1)
    got = H.run_trace(eng, H.trace_portions({"x": ids}))["x"]

    Wc = H.as_compute(W, dtype)
    eps, nh, nkv, hd = cfg["rms_norm_eps"], 4, 2, 16
    cos, sin = pm.rope_tables(cfg["rope_theta"], hd, len(ids))
    h = pm.embedding(Wc["model.embed_tokens.weight"], ids)
    kv0 = None
    for layer, cache_id, write in schedule:
        p = f"model.layers.{layer}."
        n = pm.rmsnorm(h, Wc[p + "input_layernorm.weight"], eps)
        if write:
            if cache_id == 0:
                T = len(ids)
                k = pm.linear(n, Wc[p + "self_attn.k_proj.weight"], Wc[p + "self_attn.k_proj.bias"]).view(T, nkv, hd)
                v = pm.linear(n, Wc[p + "self_attn.v_proj.weight"], Wc[p + "self_attn.v_proj.bias"]).view(T, nkv, hd)
                kv0 = (pm.apply_rope(k, cos, sin), v)
            h = h + pm.attention_block(cfg, Wc, p + "self_attn.", n, cos, sin, None)
        else:
            T = len(ids)
            q = pm.linear(n, Wc[p + "self_attn.q_proj.weight"], Wc[p + "self_attn.q_proj.bias"]).view(T, nh, hd)
            ctx = pm.attention(pm.apply_rope(q, cos, sin), kv0[0], kv0[1]).reshape(T, nh * hd)
            h = h + pm.linear(ctx, Wc[p + "self_attn.o_proj.weight"])
        n = pm.rmsnorm(h, Wc[p + "post_attention_layernorm.weight"], eps)
        h = h + pm.swiglu_mlp(n, Wc[p + "mlp.gate_proj.weight"], Wc[p + "mlp.up_proj.weight"], Wc[p + "mlp.down_proj.weight"])
    ref = pm.linear(pm.rmsnorm(h, Wc["model.norm.weight"], eps), Wc["model.embed_tokens.weight"]).numpy()
    g = np.stack([got[p] for p in sorted(got)])
    if dtype == torch.float32:
        H.check_f32(g, ref, "run order")
    else:
        assert np.sqrt(np.mean((g - ref) ** 2)) < 0.03 * np.sqrt(np.mean(ref ** 2)) + 3e-3


def test_toy_mixer_with_state_registers_builds_and_steps():
    """A mixer defined here: s_t = decay * s_{t-1} + x_t W (state per request, fixed size), y_t = s_t. It is
    registered, named by a toy architecture's spec (mixed with attention layers), built by the framework and stepped
    in portions and mixed batches; the state must carry across portions, start at zero for a new request, and not
    leak between requests."""
    from infer_b200.config import (Architecture, LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture,
                                   unregister_architecture)
    from infer_b200.engine import Engine
    from infer_b200.parts import Mixer, StateNeed, register_mixer, unregister
    from infer_b200.weights import random_weights

    @register_mixer("toy_decay")
    class ToyDecay(Mixer):
        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.size, self.decay = int(spec["size"]), float(spec["decay"])

        @classmethod
        def param_shapes(cls, spec):
            return {"mix.weight": (int(spec["size"]), int(spec["size"]))}

        def load(self, params):
            self.w = params["mix.weight"].to(self.rt.device, torch.float32)

        def cache_need(self):
            return StateNeed({"s": ((self.size,), torch.float32)})

        def forward(self, x, step, cache, residual, write_cache=True):
            u = x.float() @ self.w.T
            out = torch.empty_like(u)
            row = 0
            slots = step.seg_slot.tolist()
            for seg, n in enumerate(step.seg_lens):
                s = cache["s"][slots[seg]]
                for t in range(n):
                    s.mul_(self.decay).add_(u[row + t])
                    out[row + t] = s
                row += n
            return residual + out

    try:
        Hd, V = 32, 50
        attn = H.spec_of(dict(H.TINY["a"], hidden_size=Hd, num_attention_heads=2, num_key_value_heads=1, vocab_size=V,
                              intermediate_size=48)).layers[0]
        toy = LayerSpec("prenorm", PartSpec("toy_decay", {"size": Hd, "decay": 0.9}, "toy.1."), attn.feed_forward,
                        attn.mixer_norm, attn.feed_forward_norm)
        toy = LayerSpec("prenorm", toy.mixer, PartSpec("swiglu", dict(attn.feed_forward.params), "toy.1.mlp."),
                        PartSpec("rmsnorm", dict(attn.mixer_norm.params), "toy.1.n1."),
                        PartSpec("rmsnorm", dict(attn.feed_forward_norm.params), "toy.1.n2."))
        spec = ModelSpec("ToyForTests", Hd, V, 256, (attn, toy), (LayerCall(0, 0), LayerCall(1, 1)),
                         PartSpec("rmsnorm", {"size": Hd, "eps": 1e-6}, "model.norm."), "model.embed_tokens.weight", None)
        register_architecture(Architecture("ToyForTests", lambda raw: raw, lambda typed: spec, lambda typed: dict(typed)))
        W = random_weights(spec, 4, torch.float32)
        assert "toy.1.mix.weight" in W
        eng = Engine(spec, W, dtype=torch.float32, max_tokens=256, max_requests=2)
        assert 1 in eng.cache.state_needs and eng.cache.view(1)["s"].shape == (2, Hd)
        ids = {"p": H.random_ids({"vocab_size": V}, 40, 1), "q": H.random_ids({"vocab_size": V}, 23, 2),
               "r": H.random_ids({"vocab_size": V}, 17, 3)}
        reqs = {k: (v, len(v) - 6) for k, v in ids.items()}
        got = H.run_trace(eng, H.trace_mixed(reqs, 192, seed=1, max_live=2))     # r reuses a finished request's slot

        def plain(seq):
            T = len(seq)
            h = pm.embedding(W["model.embed_tokens.weight"], seq)
            cos, sin = pm.rope_tables(10000.0, 16, T)
            cfg = dict(hidden_size=Hd, num_attention_heads=2, num_key_value_heads=1, attention_bias=True)
            n = pm.rmsnorm(h, W["model.layers.0.input_layernorm.weight"], 1e-6)
            h = h + pm.attention_block(cfg, W, "model.layers.0.self_attn.", n, cos, sin, None)
            n = pm.rmsnorm(h, W["model.layers.0.post_attention_layernorm.weight"], 1e-6)
            h = h + pm.swiglu_mlp(n, W["model.layers.0.mlp.gate_proj.weight"], W["model.layers.0.mlp.up_proj.weight"],
                                  W["model.layers.0.mlp.down_proj.weight"])
            n = pm.rmsnorm(h, W["toy.1.n1.weight"], 1e-6)
            u = n @ W["toy.1.mix.weight"].double().T
            s = torch.zeros(Hd, dtype=torch.float64)
            y = torch.zeros_like(u)
            for t in range(T):
                s = 0.9 * s + u[t]
                y[t] = s
            h = h + y
            n = pm.rmsnorm(h, W["toy.1.n2.weight"], 1e-6)
            h = h + pm.swiglu_mlp(n, W["toy.1.mlp.gate_proj.weight"], W["toy.1.mlp.up_proj.weight"], W["toy.1.mlp.down_proj.weight"])
            return pm.linear(pm.rmsnorm(h, W["model.norm.weight"], 1e-6), W["model.embed_tokens.weight"]).numpy()
        for rid, seq in ids.items():
            ref = plain(seq)
            g = np.stack([got[rid][p] for p in sorted(got[rid])])
            assert np.abs(g - ref).max() < 5e-5, rid
    finally:
        unregister("mixer", "toy_decay")
        unregister_architecture("ToyForTests")
