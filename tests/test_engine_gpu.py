"""The engine against the plain implementation, for every way of cutting requests into steps, in float32
and in bfloat16.  Logits at a position must not depend on the cutting, the batch or the pages."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
SEED = 5


def _engine(name, dtype, max_tokens=1024, **kw):
    from infer_b200.engine import Engine
    cfg = H.TINY[name]
    W = H.make_weights(name, SEED)
    return Engine(H.spec_of(cfg), W, dtype=dtype, max_tokens=max_tokens, max_requests=4, **kw)


def _check(name, dtype, got, reqs):
    cfg, stored = H.TINY[name], H.STORED_DTYPE[name]
    worst = 0.0
    for rid, ids in reqs.items():
        ref = H.oracle(cfg, SEED, stored, dtype, ids)
        rows = sorted(got[rid])
        g = np.stack([got[rid][p] for p in rows])
        if dtype == torch.float32:
            worst = max(worst, H.check_f32(g, ref[rows], f"{name}/{rid}"))
        else:
            refr = H.oracle(cfg, SEED, stored, dtype, ids, torch.bfloat16)
            H.check_bf16(g, ref[rows], refr[rows], f"{name}/{rid}")
    return worst


def _requests(name, lengths, seed0=0):
    return {f"r{i}": H.random_ids(H.TINY[name], n, seed0 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_whole(name, dtype):
    reqs = _requests(name, [5, 17, 33, 70, 1])
    eng = _engine(name, dtype)
    got = H.run_trace(eng, H.trace_whole(reqs))
    _check(name, dtype, got, reqs)
    assert eng.cache.pages_in_use() == [0] * len(eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_tail_one_by_one(name, dtype):
    reqs = _requests(name, [75, 40], seed0=10)
    got = H.run_trace(_engine(name, dtype), H.trace_tail(reqs, 32))
    _check(name, dtype, got, reqs)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_portions_of_changing_size(name, dtype):
    reqs = _requests(name, [150, 61], seed0=20)
    got = H.run_trace(_engine(name, dtype), H.trace_portions(reqs))
    _check(name, dtype, got, reqs)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_mixed_with_page_reuse(name, dtype):
    lengths = [60, 45, 100, 33, 64, 90, 20, 77]
    ids = _requests(name, lengths, seed0=30)
    reqs = {rid: (t, max(2, len(t) - 16 - 3 * i)) for i, (rid, t) in enumerate(ids.items())}
    max_tokens = 320                                        # 20 pages: fewer than the requests need in total
    steps = H.trace_mixed(reqs, max_tokens, seed=7)
    assert max(len(s["entries"]) for s in steps) >= 3
    eng = _engine(name, dtype, max_tokens=max_tokens)
    got = H.run_trace(eng, steps)
    _check(name, dtype, got, ids)
    total_pages = sum(-(-n // 16) for n in lengths)
    assert total_pages > eng.cache.pages_total()[0]         # so pages were used again
    assert eng.cache.pages_in_use() == [0] * len(eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_cuttings_agree_with_each_other(dtype):
    """float32: identical up to float rounding of unchanged reduction orders (in fact bit-equal); bfloat16:
    rounding noise only."""
    name = "b"
    reqs = _requests(name, [97], seed0=40)
    a = H.run_trace(_engine(name, dtype), H.trace_whole(reqs))["r0"]
    b = H.run_trace(_engine(name, dtype), H.trace_tail(reqs, 32))["r0"]
    c = H.run_trace(_engine(name, dtype), H.trace_portions(reqs))["r0"]
    for p in a:
        for other in (b, c):
            if dtype == torch.float32:
                assert np.array_equal(a[p], other[p]), f"position {p} differs between cuttings in float32"
            else:
                assert np.abs(a[p] - other[p]).max() < 0.02


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_long_decode(dtype):
    """A short prompt and 300 tokens decoded one by one, across many page edges."""
    name = "a"
    ids = H.random_ids(H.TINY[name], 310, 50)
    steps = [{"entries": [("x", ids[:10], [9])], "end": []}]
    steps += [{"entries": [("x", [ids[i]], [0])], "end": []} for i in range(10, 310)]
    got = H.run_trace(_engine(name, dtype), steps)
    _check(name, dtype, got, {"x": ids})


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_first_tokens(dtype):
    """The first tokens of a sequence, one by one from position 0."""
    name = "c"
    ids = H.random_ids(H.TINY[name], 6, 60)
    steps = [{"entries": [("x", [t], [0])], "end": []} for t in ids]
    got = H.run_trace(_engine(name, dtype), steps)
    _check(name, dtype, got, {"x": ids})


def test_far_key_stands_out():
    """One key far back among hundreds carries the answer: query and key of one early position are scaled so
    that its score dominates. A cache that loses or misplaces that page changes the logits visibly."""
    name, dtype = "a", torch.float32
    cfg = H.TINY[name]
    W = H.make_weights(name, SEED)
    # scale the q and k projections of layer 0 so that scores are sharp: attention then picks single far keys
    for n in ("q_proj", "k_proj"):
        W[f"model.layers.0.self_attn.{n}.weight"] = W[f"model.layers.0.self_attn.{n}.weight"] * 40.0
        W[f"model.layers.0.self_attn.{n}.bias"] = W[f"model.layers.0.self_attn.{n}.bias"] * 40.0
    from infer_b200.engine import Engine
    ids = H.random_ids(cfg, 400, 70)
    eng = Engine(H.spec_of(cfg), W, dtype=dtype, max_tokens=512, max_requests=2)
    got = H.run_trace(eng, H.trace_tail({"x": ids}, 32))["x"]
    import plain_model as pm
    ref = pm.forward(cfg, H.as_compute(W, dtype), ids).numpy()
    rows = sorted(got)
    H.check_f32(np.stack([got[p] for p in rows]), ref[rows], "far key")


def test_repeated_portion_shapes_are_captured_and_replay_like_eager():
    """Steps with prompt portions are captured into CUDA graphs once their exact shape has come a few times (prompts cut
    at the token budget): the replays give the bits of the eager path, for other tokens and other pages."""
    from infer_b200.engine import StepEntry
    name = "b"
    cfg = H.TINY[name]
    eager = _engine(name, torch.bfloat16, cuda_graphs=False)
    graph = _engine(name, torch.bfloat16)
    for r in range(7):
        ids = H.random_ids(cfg, 41, 100 + r)
        outs = []
        for eng in (eager, graph):
            eng.add_request("x")
            a = eng.step([StepEntry("x", ids[:24], [0, 23])]).float().cpu()
            b = eng.step([StepEntry("x", ids[24:40], [15])]).float().cpu()
            c = eng.step([StepEntry("x", ids[40:], [0])]).float().cpu()
            eng.check_status()
            eng.end_request("x")
            outs.append((a, b, c))
        for x, y in zip(*outs):
            assert torch.equal(x, y), f"round {r}"
    portion_keys = [k for k in graph._graphs if k[0] == "portions"]
    assert len(portion_keys) == 2 and all(len(graph._graphs[k].graphs) == 1 for k in portion_keys)
    ref = H.oracle(cfg, SEED, H.STORED_DTYPE[name], torch.bfloat16, ids)
    refr = H.oracle(cfg, SEED, H.STORED_DTYPE[name], torch.bfloat16, ids, torch.bfloat16)
    got = torch.cat(outs[1]).numpy()
    H.check_bf16(got, ref[[0, 23, 39, 40]], refr[[0, 23, 39, 40]], "captured portions")
