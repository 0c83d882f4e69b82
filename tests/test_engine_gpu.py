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


def test_a_captured_portion_shape_replays_at_another_start_position():
    """What a captured step froze on the host (attention slices, product plans) may depend only on the graph's key
    (segment lengths, wanted rows, table widths), never on where the segments start: the same portion shape is
    replayed at a context start several pages away, in a model with a window layer, and must give the eager bits."""
    from infer_b200.engine import StepEntry
    name = "c"
    cfg = H.TINY[name]
    eager = _engine(name, torch.bfloat16, cuda_graphs=False)
    graph = _engine(name, torch.bfloat16)
    # the table width (8 pages = 128 positions) stays the same for starts 0, 7, 50 and 90 with a 24-token portion
    starts = [0, 0, 0, 7, 50, 90, 3]
    for r, start in enumerate(starts):
        ids = H.random_ids(cfg, start + 24, 300 + r)
        outs = []
        for eng in (eager, graph):
            eng.add_request("x")
            if start:
                eng.step([StepEntry("x", ids[:start], [])])
            a = eng.step([StepEntry("x", ids[start:], [0, 23])]).float().cpu()
            eng.check_status()
            eng.end_request("x")
            outs.append(a)
        assert torch.equal(outs[0], outs[1]), f"start {start}"
    key = ("portions", (24,), 2, (8, 8), 0)
    assert key in graph._graphs and len(graph._graphs[key].graphs) == 1, list(graph._graphs)
    ref = H.oracle(cfg, SEED, H.STORED_DTYPE[name], torch.bfloat16, ids)
    refr = H.oracle(cfg, SEED, H.STORED_DTYPE[name], torch.bfloat16, ids, torch.bfloat16)
    H.check_bf16(outs[1].numpy(), ref[[3, 26]], refr[[3, 26]], "replayed at another start")


def test_steps_issued_back_to_back_take_their_own_inputs():
    """A caller may issue captured steps without ever waiting for the device. Each step's integers go through one of
    two pinned staging buffers; the engine waits for the copy that read a buffer last before it writes the buffer
    again. Without that, a step would run with the positions and tables of a later one: the cache rows in between
    would stay unwritten and the final logits would differ."""
    from infer_b200.engine import StepEntry
    name = "b"
    cfg = H.TINY[name]
    ids = [H.random_ids(cfg, 60, 900 + r) for r in range(3)]

    def run(sync_every_step):
        eng = _engine(name, torch.bfloat16)
        for r in range(3):
            eng.add_request(r)
            eng.step([StepEntry(r, ids[r][:10], [])])
        torch.cuda.synchronize()
        out = None
        for i in range(10, 60):
            out = eng.step([StepEntry(r, [ids[r][i]], [0]) for r in range(3)])
            if sync_every_step:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        eng.check_status()
        tables = [eng.cache.block_table(r, 0) for r in range(3)]
        k = torch.stack([eng.cache.groups[0].k[:, p] for t in tables for p in t]).float().cpu()
        return out.float().cpu(), k
    a_logits, a_cache = run(True)
    b_logits, b_cache = run(False)
    assert torch.equal(a_cache, b_cache), "cache rows differ: a step ran with another step's positions"
    assert torch.equal(a_logits, b_logits)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_try_step_leaves_out_what_does_not_fit_and_touches_nothing_of_it(dtype):
    """Per-entry failure (the reference's -1 per row, kernels/batch_gpu.cu:386-410): with 4 pages in the pool, the
    entries are served in order; the one whose pages are not there, and the one that would pass the sequence limit,
    are reported and their requests stay as they were; the others' logits are those of the plain implementation."""
    from infer_b200.engine import Engine, OutOfPages, StepEntry
    name = "a"
    cfg = H.TINY[name]
    eng = Engine(H.spec_of(cfg), H.make_weights(name, SEED), dtype=dtype, max_tokens=4 * 16, max_requests=4, max_seq_len=40)
    ids = {r: H.random_ids(cfg, 48, 950 + i) for i, r in enumerate("abcd")}
    for r in ids:
        eng.add_request(r)
    eng.step([StepEntry("a", ids["a"][:30], [])])                                   # a holds 2 of the 4 pages
    entries = [StepEntry("b", ids["b"][:17], [16]),                                 # needs 2 pages: fits
               StepEntry("c", ids["c"][:5], [4]),                                   # needs 1: nothing left
               StepEntry("a", ids["a"][30:42], [11]),                               # would reach position 42 > 40
               StepEntry("d", [ids["d"][0]], [0])]                                  # needs 1: nothing left
    with pytest.raises(OutOfPages):
        eng.step(entries)
    assert [eng.cache.length(r) for r in "abcd"] == [30, 0, 0, 0] and eng.cache.pages_free() == [2]
    res = eng.try_step(entries)
    assert res.ran == [True, False, False, False] and res.output.shape[0] == 1
    assert [eng.cache.length(r) for r in "abcd"] == [30, 17, 0, 0] and eng.cache.pages_free() == [0]
    eng.cache.check_invariants()
    eng.end_request("b")
    res2 = eng.try_step([StepEntry("a", ids["a"][30:40], [9]), StepEntry("c", ids["c"][:5], [4])])
    assert res2.ran == [True, True]
    eng.check_status()
    got = {"b": {16: res.output[0].float().cpu().numpy()}, "a": {39: res2.output[0].float().cpu().numpy()},
           "c": {4: res2.output[1].float().cpu().numpy()}}
    _check(name, dtype, got, {"a": ids["a"][:40], "b": ids["b"][:17], "c": ids["c"][:5]})


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_sampling_inside_the_step_equals_sampling_from_its_logits(dtype):
    """step(..., sample=...) runs the sampling kernel inside the step (and inside its graph): the ids are those the
    kernel gives on the logits that the same step returns without `sample`, for greedy, seeded temperature and
    top-k/top-p rows, and each id is left on the device for the request's next FEEDBACK_TOKEN."""
    from infer_b200 import ops
    from infer_b200.engine import StepEntry
    from infer_b200.engine.scheduler import SampleParams
    name = "b"
    cfg = H.TINY[name]
    ids = [H.random_ids(cfg, 12, 970 + r) for r in range(3)]
    params = [SampleParams(), SampleParams(0.8, 7), SampleParams(1.1, 3, top_k=5, top_p=0.9)]
    for filtered in (False, True):
        ps = params if filtered else params[:2] + [SampleParams(0.5, 9)]
        a, b = _engine(name, dtype), _engine(name, dtype)
        for eng in (a, b):
            for r in range(3):
                eng.add_request(r)
        logits = a.step([StepEntry(r, ids[r], [11]) for r in range(3)])
        toks = b.step([StepEntry(r, ids[r], [11]) for r in range(3)], sample=[(p, 11) for p in ps])
        dev = logits.device
        t = torch.tensor([p.temperature for p in ps], dtype=torch.float32, device=dev)
        seed = torch.tensor([p.seed for p in ps], dtype=torch.int64, device=dev)
        pos = torch.full((3,), 11, dtype=torch.int64, device=dev)
        if filtered:
            want = ops.sample_filtered(logits, t, seed, pos, torch.tensor([p.top_k for p in ps], dtype=torch.int64, device=dev),
                                       torch.tensor([p.top_p for p in ps], dtype=torch.float32, device=dev))
        else:
            want = ops.sample(logits, t, seed, pos)
        assert toks.dtype == torch.int32 and torch.equal(toks, want)
        slots = [b.cache.slot(r) for r in range(3)]
        assert b.next_tokens[slots].tolist() == toks.tolist()
        # decoding on from the device-side token equals decoding on from the id
        for step in range(4):
            la = a.step([StepEntry(r, [int(toks[r])], [0]) for r in range(3)])
            tb = b.step([StepEntry(r, [-1], [0]) for r in range(3)], sample=[(p, 12 + step) for p in ps])
            if filtered:
                want = ops.sample_filtered(la, t, seed, pos + 1 + step, torch.tensor([p.top_k for p in ps], dtype=torch.int64, device=dev),
                                           torch.tensor([p.top_p for p in ps], dtype=torch.float32, device=dev))
            else:
                want = ops.sample(la, t, seed, pos + 1 + step)
            assert torch.equal(tb, want), f"decode step {step}"
            toks = tb.clone()
        a.check_status(), b.check_status()
