"""Whole-model logits on the path that the benchmark times: Qwen2.5-1.5B layer sizes (two layers, a small
vocabulary so that the plain implementation stays fast) with prompts of 300 and 600 tokens, so that steps of more than
128 tokens run: the persistent tcgen05 product (128 x 176/192/256 tiles) and the tcgen05 attention with several query
and key tiles. Every cutting of the requests is compared with the plain implementation, in float32 and in bfloat16
(src/forward.cpp:170-258 is what the plain implementation restates; tests/test_batch_gpu.cpp:265-269 is the
reference's own teacher-forced comparison).

The bfloat16 tests also assert, from the launchers' counters, that those two kernels are the ones that ran: if the
planner stopped choosing them at these sizes the tests would fail rather than pass on another kernel."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
SEED = 11

CFG = dict(architectures=["Qwen2ForCausalLM"], hidden_size=1536, num_hidden_layers=2, num_attention_heads=12,
           num_key_value_heads=2, intermediate_size=8960, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6,
           max_position_embeddings=4096, tie_word_embeddings=True, use_sliding_window=False)
DTYPES = [torch.float32, torch.bfloat16]


def _reqs():
    return {"long": H.random_ids(CFG, 600, 1), "mid": H.random_ids(CFG, 300, 2)}


def _engine(dtype, max_tokens=1024):
    from infer_b200.engine import Engine
    W = H.make_weights(CFG, SEED, torch.bfloat16)
    return Engine(H.spec_of(CFG), W, dtype=dtype, max_tokens=max_tokens, max_requests=4)


def _check(dtype, got, reqs):
    for rid, ids in reqs.items():
        # the stored values are bfloat16 already, so the plain implementation's result is the same for both paths
        ref = H.oracle(CFG, SEED, torch.bfloat16, torch.bfloat16, ids)
        rows = sorted(got[rid])
        g = np.stack([got[rid][p] for p in rows])
        if dtype == torch.float32:
            H.check_f32(g, ref[rows], rid)
        else:
            refr = H.oracle(CFG, SEED, torch.bfloat16, torch.bfloat16, ids, torch.bfloat16)
            H.check_bf16(g, ref[rows], refr[rows], rid)


def _counts():
    from infer_b200 import ops
    return dict(ops.LAUNCH_KINDS)


def _ran(before, kind):
    return _counts().get(kind, 0) - before.get(kind, 0)


def _assert_bench_kernels_ran(before, dtype):
    if dtype == torch.bfloat16:
        assert _ran(before, "gemm_tc:persistent") > 0, "the persistent tcgen05 product did not run in this model"
        assert _ran(before, "attention_prefill_tc:several_query_tiles") > 0, "the tcgen05 attention ran one query tile only"


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_whole_prompts_of_300_and_600_tokens(dtype):
    reqs = _reqs()
    before = _counts()
    eng = _engine(dtype)
    got = H.run_trace(eng, H.trace_whole(reqs))
    _check(dtype, got, reqs)
    _assert_bench_kernels_ran(before, dtype)
    if dtype == torch.bfloat16:
        # the down product of 300 and 600 tokens: 128 x 256 tiles whose K slices meet in the operand rings
        assert _ran(before, "gemm_tc:sliced_wide") > 0, "no product ran on wide tiles with K slices"
    assert eng.cache.pages_in_use() == [0]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_all_but_the_last_32_at_once_then_one_by_one(dtype):
    reqs = _reqs()
    before = _counts()
    got = H.run_trace(_engine(dtype), H.trace_tail(reqs, 32))
    _check(dtype, got, reqs)
    _assert_bench_kernels_ran(before, dtype)


def _portions(reqs):
    """Portions of changing size, some well above 128 tokens (the persistent product; attention with several
    query tiles over earlier pages), some down to two; every place is wanted."""
    sizes = [2, 150, 3, 131, 17, 200, 2, 64, 129]
    steps = []
    for rid, ids in reqs.items():
        i = k = 0
        while i < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - i)
            k += 1
            if len(ids) - i - n == 1:
                n += 1
            steps.append({"entries": [(rid, ids[i:i + n], list(range(n)))], "end": []})
            i += n
        steps[-1]["end"] = [rid]
    return steps


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_portions_of_changing_size_above_and_below_128_tokens(dtype):
    reqs = _reqs()
    steps = _portions(reqs)
    assert max(len(s["entries"][0][1]) for s in steps) > 128 and min(len(s["entries"][0][1]) for s in steps) == 2
    before = _counts()
    got = H.run_trace(_engine(dtype), steps)
    _check(dtype, got, reqs)
    _assert_bench_kernels_ran(before, dtype)


def test_portions_behind_a_long_context_share_their_query_tiles():
    """A 1,400-token prompt in portions of 300: from 1,024 tokens on a portion's query tiles have eight and more key
    tiles and few CTAs, so the tcgen05 attention shares their keys among CTAs that meet in the workspace (asserted
    from the launcher's counter); its logits against the plain implementation like every other cutting."""
    reqs = {"long": H.random_ids(CFG, 1400, 5)}
    ids = reqs["long"]
    steps = []
    for i in range(0, len(ids), 300):
        n = min(300, len(ids) - i)
        steps.append({"entries": [("long", ids[i:i + n], list(range(max(0, n - 40), n)))], "end": []})
    steps[-1]["end"] = ["long"]
    before = _counts()
    got = H.run_trace(_engine(torch.bfloat16, max_tokens=1472), steps)
    _check(torch.bfloat16, got, reqs)
    assert _ran(before, "attention_prefill_tc:shared_query_tiles") > 0, "no portion's query tiles were shared among CTAs"


def _mixed(reqs, max_tokens, seed=3, max_live=4):
    """Up to four live requests; a step takes a prompt portion of 2..260 tokens from those still in their prompt and
    one token from those decoding. A request starts only when the rounded-up final lengths of the live ones leave
    room, so the pool is never exceeded and pages of finished requests go out again."""
    rng = np.random.default_rng(seed)
    waiting, live, steps = list(reqs), {}, []

    def rounded(rid):
        return -(-len(reqs[rid][0]) // 64) * 64
    while waiting or live:
        while waiting and len(live) < max_live and sum(rounded(r) for r in live) + rounded(waiting[0]) <= max_tokens:
            live[waiting.pop(0)] = 0
        assert live
        entries, end = [], []
        chosen = [r for r in live if rng.random() < 0.75] or [next(iter(live))]
        for rid in chosen:
            ids, plen = reqs[rid]
            i = live[rid]
            if i < plen:
                n = min(int(rng.choice([2, 9, 40, 140, 260])), plen - i)
                if plen - i - n == 1:
                    n += 1
            else:
                n = 1
            n = min(n, len(ids) - i)
            entries.append((rid, ids[i:i + n], list(range(n))))
            live[rid] = i + n
            if live[rid] == len(ids):
                end.append(rid)
        for rid in end:
            del live[rid]
        steps.append({"entries": entries, "end": end})
    return steps


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_mixed_with_four_live_requests_and_pages_used_again(dtype):
    lengths = {"long": 600, "mid": 300, "m3": 200, "m4": 170, "m5": 330}
    ids = {rid: H.random_ids(CFG, n, 1 if rid == "long" else 2 if rid == "mid" else 10 + n) for rid, n in lengths.items()}
    assert ids["long"] == _reqs()["long"] and ids["mid"] == _reqs()["mid"]          # their plain results are cached
    reqs = {rid: (t, len(t) - 8 - 3 * i) for i, (rid, t) in enumerate(ids.items())}
    max_tokens = 1344                                       # 84 pages; the five requests need 102 in total
    steps = _mixed(reqs, max_tokens)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len(s["entries"]) > 1 and max(len(e[1]) for e in s["entries"]) > 128 and min(len(e[1]) for e in s["entries"]) == 1
               for s in steps), "no step mixes a long portion with a decoded token"
    before = _counts()
    eng = _engine(dtype, max_tokens=max_tokens)
    got = H.run_trace(eng, steps)
    _check(dtype, got, ids)
    _assert_bench_kernels_ran(before, dtype)
    assert sum(-(-n // 16) for n in lengths.values()) > eng.cache.pages_total()[0]       # so pages were used again
    assert eng.cache.pages_in_use() == [0]


def test_float32_cuttings_are_bit_equal_at_these_sizes():
    """The 32-bit path chooses no kernel by the number of rows in a step, so every cutting gives the same bits."""
    reqs = {"mid": _reqs()["mid"]}
    whole = H.run_trace(_engine(torch.float32), H.trace_whole(reqs))
    cut = H.run_trace(_engine(torch.float32), _portions(reqs))
    for p, row in whole["mid"].items():
        assert np.array_equal(row, cut["mid"][p]), f"position {p}"
