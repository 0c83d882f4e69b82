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
        toy = LayerSpec.standard("prenorm", PartSpec("toy_decay", {"size": Hd, "decay": 0.9}, "toy.1."),
                                 PartSpec("swiglu", dict(attn.part("feed_forward").params), "toy.1.mlp."),
                                 PartSpec("rmsnorm", dict(attn.part("mixer_norm").params), "toy.1.n1."),
                                 PartSpec("rmsnorm", dict(attn.part("feed_forward_norm").params), "toy.1.n2."))
        spec = ModelSpec("ToyForTests", Hd, V, 256, (attn, toy), (LayerCall(0, 0), LayerCall(1, 1)),
                         PartSpec("rmsnorm", {"size": Hd, "eps": 1e-6}, "model.norm."),
                         PartSpec("token_table", {"vocab_size": V, "hidden_size": Hd}, "model.embed_tokens."),
                         PartSpec("linear_head", {"vocab_size": V, "hidden_size": Hd, "tied": True}, "lm_head."))
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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_toy_block_with_three_norms_toy_positions_and_scaled_embedding(dtype):
    """Parts that this engine's architecture does not have, defined and registered here, with no change to a
    framework file: a block arrangement with five slots, three of them norms ("sandwich": h += mixer(norm_in(h));
    h += norm_out(ffn(norm_mid(h)))), a position encoding that is not a rotation and goes through ``apply()`` (so the
    attention part stores keys as it gets them), an
    embedding with a scale, an untied head of its own kind with a soft cap, and a part that says it cannot be
    captured into a CUDA graph, which the engine must honour in bfloat16. Compared with a plain computation."""
    from infer_b200.config import (Architecture, LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture,
                                   unregister_architecture)
    from infer_b200.engine import Engine
    from infer_b200.parts import (Block, Head, PositionEncoding, register_block, register_head, register_position, unregister)
    from infer_b200.parts.linear import Linear
    from infer_b200.weights import random_weights

    @register_position("toy_additive")
    class ToyAdditive(PositionEncoding):
        """q and k get a learned-free additive code: x[..., j] += amp * sin(pos * (j + 1) * rate)."""
        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.amp, self.rate = float(spec["amp"]), float(spec["rate"])

        def rotary_tables(self, n_positions=None):
            return None

        def apply(self, q, k, positions):
            for x in (q, k):
                j = torch.arange(1, x.shape[-1] + 1, device=x.device, dtype=torch.float32)
                code = self.amp * torch.sin(positions.float()[:, None] * j[None, :] * self.rate)      # [T, head_dim]
                x.copy_((x.float() + code[:, None, :]).to(x.dtype))

    @register_block("toy_sandwich")
    class Sandwich(Block):
        def __init__(self, norm_in, mixer, norm_mid, feed_forward, norm_out):
            super().__init__(norm_in=norm_in, mixer=mixer, norm_mid=norm_mid, feed_forward=feed_forward, norm_out=norm_out)

        def forward(self, h, step, cache, write_cache=True):
            h = self.mixer.forward(self.norm_in.forward(h), step, cache, h, write_cache)
            delta = self.feed_forward.forward(self.norm_mid.forward(h), torch.zeros_like(h))
            return h + self.norm_out.forward(delta, torch.float32)

    @register_head("toy_capped")
    class Capped(Head):
        graph_safe = False                     # pretend: this part must never be captured

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.cap = float(spec["cap"])

        @classmethod
        def param_shapes(cls, spec):
            return {"weight": (int(spec["vocab_size"]), int(spec["hidden_size"]))}

        def load(self, params):
            self.linear = Linear(self.rt, params["weight"])

        def forward(self, x):
            assert not torch.cuda.is_current_stream_capturing(), "a part that is not graph-safe was captured"
            return self.cap * torch.tanh(self.linear(x, out_dtype=torch.float32) / self.cap)

    try:
        Hd, V, nh, nkv, hd, I = 48, 61, 3, 1, 16, 80
        pos = PartSpec("toy_additive", {"amp": 0.3, "rate": 0.05})
        layers = []
        for i in range(2):
            p = f"t.{i}."
            layers.append(LayerSpec("toy_sandwich", {
                "norm_in": ("norm", PartSpec("rmsnorm", {"size": Hd, "eps": 1e-5}, p + "n1.")),
                "mixer": ("mixer", PartSpec("attention", {"hidden_size": Hd, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
                                                          "qkv_bias": False, "window": None, "softmax_scale": 0.2, "position": pos},
                                            p + "attn.")),
                "norm_mid": ("norm", PartSpec("rmsnorm", {"size": Hd, "eps": 1e-5}, p + "n2.")),
                "feed_forward": ("feed_forward", PartSpec("swiglu", {"hidden_size": Hd, "intermediate_size": I}, p + "mlp.")),
                "norm_out": ("norm", PartSpec("rmsnorm", {"size": Hd, "eps": 1e-5}, p + "n3."))}))
        spec = ModelSpec("ToySandwich", Hd, V, 256, tuple(layers), (LayerCall(0, 0), LayerCall(1, 1)),
                         PartSpec("rmsnorm", {"size": Hd, "eps": 1e-5}, "final."),
                         PartSpec("token_table", {"vocab_size": V, "hidden_size": Hd, "scale": 3.0}, "emb."),
                         PartSpec("toy_capped", {"vocab_size": V, "hidden_size": Hd, "cap": 2.0}, "out."))
        register_architecture(Architecture("ToySandwich", lambda raw: raw, lambda typed: spec, lambda typed: dict(typed)))
        W = random_weights(spec, 6, torch.bfloat16)
        assert {"t.0.n3.weight", "t.1.attn.q_proj.weight", "out.weight", "emb.weight"} <= set(W) and "t.0.attn.q_proj.bias" not in W
        eng = Engine(spec, W, dtype=dtype, max_tokens=256, max_requests=3)
        assert not eng.use_graphs                                  # the head said so
        ids = {"p": H.random_ids({"vocab_size": V}, 50, 1), "q": H.random_ids({"vocab_size": V}, 33, 2)}
        reqs = {k: (v, len(v) - 10) for k, v in ids.items()}
        got = H.run_trace(eng, H.trace_mixed(reqs, 192, seed=2, max_live=2))
        Wd = {k: v.double() for k, v in W.items()}

        def plain(seq):
            T = len(seq)
            h = pm.embedding(Wd["emb.weight"], seq) * 3.0
            j = torch.arange(1, hd + 1, dtype=torch.float64)
            code = 0.3 * torch.sin(torch.arange(T, dtype=torch.float32).double()[:, None] * j[None, :] * 0.05)
            for i in range(2):
                p = f"t.{i}."
                n = pm.rmsnorm(h, Wd[p + "n1.weight"], 1e-5)
                q = pm.linear(n, Wd[p + "attn.q_proj.weight"]).view(T, nh, hd) + code[:, None, :]
                k = pm.linear(n, Wd[p + "attn.k_proj.weight"]).view(T, nkv, hd) + code[:, None, :]
                v = pm.linear(n, Wd[p + "attn.v_proj.weight"]).view(T, nkv, hd)
                h = h + pm.linear(pm.attention(q, k, v, None, 0.2).reshape(T, nh * hd), Wd[p + "attn.o_proj.weight"])
                n = pm.rmsnorm(h, Wd[p + "n2.weight"], 1e-5)
                d = pm.swiglu_mlp(n, Wd[p + "mlp.gate_proj.weight"], Wd[p + "mlp.up_proj.weight"], Wd[p + "mlp.down_proj.weight"])
                h = h + pm.rmsnorm(d, Wd[p + "n3.weight"], 1e-5)
            return (2.0 * torch.tanh(pm.linear(pm.rmsnorm(h, Wd["final.weight"], 1e-5), Wd["out.weight"]) / 2.0)).numpy()
        for rid, seq in ids.items():
            ref = plain(seq)
            g = np.stack([got[rid][p] for p in sorted(got[rid])])
            if dtype == torch.float32:
                assert np.abs(g - ref).max() < 5e-5, rid
            else:
                assert np.sqrt(np.mean((g - ref) ** 2)) < 0.03 * np.sqrt(np.mean(ref ** 2)) + 3e-3, rid
    finally:
        unregister("position", "toy_additive"), unregister("block", "toy_sandwich"), unregister("head", "toy_capped")
        unregister_architecture("ToySandwich")


def test_a_head_size_beyond_the_kernels_is_refused_when_the_part_is_built():
    from infer_b200 import ops
    from infer_b200.config import PartSpec
    from infer_b200.parts import build_part
    from infer_b200.runtime import Runtime
    too_big = ops.attention_max_head_dim() + 2
    spec = PartSpec("attention", {"hidden_size": 64, "num_heads": 1, "num_kv_heads": 1, "head_dim": too_big, "qkv_bias": False}, "a.")
    with pytest.raises(ValueError, match="beyond what the attention kernels take"):
        build_part("mixer", spec, Runtime(dtype=torch.float32))
