"""Generation through the Python entry point and the scheduler, on the real engine."""
import numpy as np
import pytest
import torch

import helpers as H
import plain_model as pm

pytestmark = pytest.mark.gpu
SEED = 5


def _llm(name, dtype, **kw):
    from infer_b200.engine.generation import LLM
    cfg = H.TINY[name]
    kw.setdefault("slots", 4)
    kw.setdefault("max_seq", 128)
    return LLM(None, dtype=dtype, spec=H.spec_of(cfg), weights=H.make_weights(name, SEED), **kw)


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_float32_equals_the_plain_implementation(name):
    cfg = H.TINY[name]
    prompts = [H.random_ids(cfg, n, 100 + n) for n in (5, 17, 33, 1)]
    llm = _llm(name, torch.float32, max_batch_tokens=24)
    outs = llm.generate(prompts, max_new=16)
    W = H.as_compute(H.make_weights(name, SEED), torch.float32)
    for p, o in zip(prompts, outs):
        assert o == pm.greedy_decode(cfg, W, p, 16)
    assert llm.engine.cache.pages_in_use() == [0] * len(llm.engine.cache.groups)


@pytest.mark.parametrize("name", ["b", "c"])
def test_greedy_bfloat16_picks_the_maximum_up_to_rounding(name):
    cfg = H.TINY[name]
    prompts = [H.random_ids(cfg, n, 200 + n) for n in (9, 40, 70)]
    outs = _llm(name, torch.bfloat16).generate(prompts, max_new=24)
    for p, o in zip(prompts, outs):
        assert len(o) == 24
        ids = p + o
        ref = H.oracle(cfg, SEED, H.STORED_DTYPE[name], torch.bfloat16, ids)
        refr = H.oracle(cfg, SEED, H.STORED_DTYPE[name], torch.bfloat16, ids, torch.bfloat16)
        noise = max(float(np.sqrt(np.mean((refr - ref) ** 2))), 1e-3 * float(np.sqrt(np.mean(ref ** 2))))
        for i, tok in enumerate(o):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - 12 * noise, f"token {i}: chose a logit {row.max() - row[tok]:.4f} below the maximum"


def test_temperature_sampling_is_seeded_and_independent_of_batching():
    name = "b"
    cfg = H.TINY[name]
    prompts = [H.random_ids(cfg, n, 300 + n) for n in (1, 9, 40, 70)]
    llm = _llm(name, torch.float32, max_seq=256)
    together = llm.generate(prompts, max_new=24, temperature=0.8, seed=11)
    again = llm.generate(prompts, max_new=24, temperature=0.8, seed=11)
    other = llm.generate(prompts, max_new=24, temperature=0.8, seed=12)
    alone = [llm.generate([p], max_new=24, temperature=0.8, seed=11)[0] for p in prompts]
    assert together == again and together == alone and together != other
    assert llm.generate(prompts[:2], max_new=8, temperature=0.0, seed=3) == llm.generate(prompts[:2], max_new=8)
    # the stream is the host twin's, given the logits of the plain implementation
    W = H.as_compute(H.make_weights(name, SEED), torch.float32)
    ids = list(prompts[1])
    for tok in together[1][:6]:
        row = pm.forward(cfg, W, ids)[-1].numpy().astype(np.float32)
        assert tok == pm.sample(row, 0.8, 11, len(ids) - 1)
        ids.append(tok)


def test_few_pages_preemption_keeps_the_streams():
    from infer_b200.engine.scheduler import Request, SampleParams
    name = "a"
    cfg = H.TINY[name]
    prompts = [H.random_ids(cfg, 20, 400 + i) for i in range(4)]
    free = _llm(name, torch.float32, max_seq=64).generate(prompts, max_new=30, temperature=0.7, seed=5)
    tight = _llm(name, torch.float32, max_seq=64, budget_mb=0)
    # shrink the pool: 4 requests x 50 positions need 16 pages; give 9
    from infer_b200.engine import Engine
    from infer_b200.engine.generation import GenerationEngine
    tight.engine = Engine(tight.engine.spec, H.make_weights(name, SEED), dtype=torch.float32, max_tokens=9 * 16,
                          max_requests=4, max_seq_len=64)
    tight.batch_engine = GenerationEngine(tight.engine)
    got = tight.generate(prompts, max_new=30, temperature=0.7, seed=5)
    assert tight.last_scheduler.preemptions > 0
    assert got == free
    assert tight.engine.cache.pages_in_use() == [0]
    tight.engine.cache.check_invariants()


def test_eos_stops_and_is_included():
    name = "a"
    cfg = H.TINY[name]
    p = H.random_ids(cfg, 12, 500)
    llm = _llm(name, torch.float32)
    full = llm.generate([p], max_new=12)[0]
    stop = full[4]
    cut = llm.generate([p], max_new=12, eos_id=stop)[0]
    assert cut == full[:full.index(stop) + 1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_overlap_and_plain_scheduling_generate_the_same(dtype):
    """Launching a step before the last step's tokens reached the host (they stay on the device for the model) gives
    the streams of the one-step-at-a-time scheduler: greedy, seeded sampling, eos, and with few pages."""
    name = "b"
    cfg = H.TINY[name]
    prompts = [H.random_ids(cfg, n, 800 + n) for n in (3, 21, 40, 9, 64)]
    a = _llm(name, dtype, slots=3, max_seq=128, overlap=False)
    b = _llm(name, dtype, slots=3, max_seq=128, overlap=True)
    for kw in (dict(max_new=20), dict(max_new=20, temperature=0.9, seed=3), dict(max_new=12, top_k=5, temperature=1.0, seed=1)):
        assert a.generate(prompts, **kw) == b.generate(prompts, **kw), kw
    full = a.generate(prompts[:2], max_new=16)
    stop = full[1][5]
    assert a.generate(prompts[:2], max_new=16, eos_id=stop) == b.generate(prompts[:2], max_new=16, eos_id=stop)
    assert b.engine.cache.pages_in_use() == [0]


def test_overlap_with_few_pages_preempts_while_a_token_is_in_flight():
    """Overlap scheduling on a pool of 9 pages for four requests that need 16: requests are preempted while the last
    step's tokens are still on their way to the host (they are read before the victim's new prompt is made), and a
    decode item after that reads its token from the device. In float32 the streams are those of the one-step-at-a-time
    scheduler with room for everything; in bfloat16 every request still ends with all its tokens and no page is lost."""
    name = "a"
    cfg = H.TINY[name]
    prompts = [H.random_ids(cfg, 20, 400 + i) for i in range(4)]
    for kw in (dict(max_new=30, temperature=0.7, seed=5), dict(max_new=30)):
        free = _llm(name, torch.float32, max_seq=64, overlap=False).generate(prompts, **kw)
        tight = _llm(name, torch.float32, max_seq=64, kv_blocks=9, overlap=True)
        assert tight.engine.cache.pages_total() == [9]
        got = tight.generate(prompts, **kw)
        sch = tight.last_scheduler
        assert sch.preemptions > 0
        assert got == free
        assert tight.engine.cache.pages_in_use() == [0]
        tight.engine.cache.check_invariants()
        tight.engine.check_status()
    fast = _llm(name, torch.bfloat16, max_seq=64, kv_blocks=9, overlap=True)
    outs = fast.generate(prompts, max_new=30)
    assert fast.last_scheduler.preemptions > 0 and [len(o) for o in outs] == [30] * 4
    assert fast.engine.cache.pages_in_use() == [0]
    fast.engine.check_status()
