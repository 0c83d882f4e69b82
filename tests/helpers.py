"""Shared by the tests: the tiny configurations, random weights, traces (ways of cutting requests into
steps) and comparisons with the plain implementation."""
from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import plain_model as pm

# Three tiny configurations of the architecture that differ in every size and option.
TINY: Dict[str, dict] = {
    # tiny A: tied head, 2:1 grouping, float32 weights
    "a": dict(architectures=["Qwen2ForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              max_position_embeddings=1024, tie_word_embeddings=True, use_sliding_window=False),
    # tiny B: untied head, 3:1 grouping, one kv head, sizes that are no power of two
    "b": dict(architectures=["Qwen2ForCausalLM"], hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, intermediate_size=224, vocab_size=320, rope_theta=1000000.0, rms_norm_eps=1e-5,
              max_position_embeddings=2048, tie_word_embeddings=False, use_sliding_window=False),
    # every head its own kv head, head_dim set apart from hidden/heads, odd vocabulary, no bias, and a
    # window of 40 positions in layers 2 and 3 (so the model has two cache groups)
    "c": dict(architectures=["Qwen2ForCausalLM"], hidden_size=80, num_hidden_layers=4, num_attention_heads=5,
              num_key_value_heads=5, head_dim=48, intermediate_size=176, vocab_size=301, rope_theta=500000.0,
              rms_norm_eps=3e-6, max_position_embeddings=512, tie_word_embeddings=True, attention_bias=False,
              use_sliding_window=True, sliding_window=40, max_window_layers=2),
}
STORED_DTYPE = {"a": torch.float32, "b": torch.bfloat16, "c": torch.bfloat16}


def spec_of(cfg: dict):
    import infer_b200.parts  # noqa: F401
    import infer_b200.models  # noqa: F401
    from infer_b200.config import parse_config
    arch, typed = parse_config(cfg)
    return arch.to_spec(typed)


def make_weights(name_or_cfg, seed: int = 1, dtype=None) -> Dict[str, torch.Tensor]:
    from infer_b200.weights import random_weights
    cfg = TINY[name_or_cfg] if isinstance(name_or_cfg, str) else name_or_cfg
    if dtype is None:
        dtype = STORED_DTYPE[name_or_cfg] if isinstance(name_or_cfg, str) else torch.bfloat16
    return random_weights(spec_of(cfg), seed, dtype)


def as_compute(W: Dict[str, torch.Tensor], dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """The values the engine computes with: matrices rounded to the compute dtype, vectors kept."""
    return {k: (v.to(dtype).float() if v.dim() == 2 else v.float()) for k, v in W.items()}


def random_ids(cfg: dict, n: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab_size"], n).tolist()


# --------------------------------------------------------------------------------------------- traces
# A trace is a list of steps; a step is {"entries": [(rid, tokens, want)], "end": [rid]}.

def trace_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    return [{"entries": [(rid, ids, list(range(len(ids))))], "end": [rid]} for rid, ids in reqs.items()]


def trace_tail(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    steps = []
    for rid, ids in reqs.items():
        head = max(1, len(ids) - tail)
        steps.append({"entries": [(rid, ids[:head], list(range(head)))], "end": []})
        for i in range(head, len(ids)):
            steps.append({"entries": [(rid, [ids[i]], [0])], "end": [rid] if i == len(ids) - 1 else []})
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(reqs: Dict[str, List[int]], seed: int = 0) -> List[dict]:
    """Each request alone, cut into portions of changing size (2, 3, 17, 5, 64, 2, ...)."""
    rng = np.random.default_rng(seed)
    steps = []
    for rid, ids in reqs.items():
        i = 0
        sizes = [2, 3, 17, 5, 64, 2, 31, 16, 7, 33, 2, 128, 9]
        k = 0
        while i < len(ids):
            n = sizes[k % len(sizes)] if k < len(sizes) else int(rng.integers(2, 40))
            k += 1
            n = min(n, len(ids) - i)
            if len(ids) - i - n == 1:      # never leave a single token: portions go down to two, not one
                n += 1
            steps.append({"entries": [(rid, ids[i:i + n], list(range(n)))], "end": []})
            i += n
        steps[-1]["end"] = [rid]
    return steps


def trace_mixed(reqs: Dict[str, Tuple[List[int], int]], max_tokens: int, seed: int = 0, max_live: int = 4,
                round_to: int = 64) -> List[dict]:
    """Up to `max_live` requests at a time; each step takes a random subset of them: a portion of the prompt
    (2..24 tokens) for those still in their prompt, one token for those decoding. reqs: rid -> (ids, prompt_len).
    A request starts only when the rounded-up final lengths of the live ones leave room, so `max_tokens` is never
    exceeded and pages of finished requests are used again."""
    rng = np.random.default_rng(seed)
    waiting = list(reqs)
    live: Dict[str, int] = {}
    steps = []

    def rounded(rid):
        return -(-len(reqs[rid][0]) // round_to) * round_to
    while waiting or live:
        while waiting and len(live) < max_live and sum(rounded(r) for r in live) + rounded(waiting[0]) <= max_tokens:
            live[waiting.pop(0)] = 0
        assert live, "max_tokens is too small for the next request"
        entries, end = [], []
        chosen = [r for r in live if rng.random() < 0.7] or [next(iter(live))]
        for rid in chosen:
            ids, plen = reqs[rid]
            i = live[rid]
            if i < plen:
                n = min(int(rng.integers(2, 25)), plen - i)
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


def run_trace(engine, steps: Sequence[dict]) -> Dict[str, Dict[int, np.ndarray]]:
    """Replays a trace in-process; returns rid -> {position: logits row}."""
    from infer_b200.engine import StepEntry
    out: Dict[str, Dict[int, np.ndarray]] = {}
    pos: Dict[str, int] = {}
    for st in steps:
        entries = []
        for rid, toks, want in st["entries"]:
            if not engine.has_request(rid):
                engine.add_request(rid)
                pos[rid] = 0
            entries.append(StepEntry(rid, toks, want))
        logits = engine.step(entries).float().cpu().numpy()
        engine.check_status()
        r = 0
        for rid, toks, want in st["entries"]:
            for w in want:
                out.setdefault(rid, {})[pos[rid] + w] = logits[r]
                r += 1
            pos[rid] += len(toks)
        for rid in st["end"]:
            engine.end_request(rid)
        engine.cache.check_invariants()
    return out


def trace_to_jsonl(steps: Sequence[dict]) -> str:
    lines = []
    for i, st in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": r, "tokens": list(map(int, t)), "want": list(w)}
                                                        for r, t, w in st["entries"]], "end": list(st["end"])}))
    return "\n".join(lines) + "\n"


# --------------------------------------------------------------------------------------------- comparison

@functools.lru_cache(maxsize=64)
def _oracle_cached(cfg_json: str, seed: int, dtype_name: str, compute_name: str, ids: Tuple[int, ...], rounding_name: str):
    cfg = json.loads(cfg_json)
    W = make_weights(cfg, seed, getattr(torch, dtype_name))
    Wc = as_compute(W, getattr(torch, compute_name))
    rounding = None if rounding_name == "none" else getattr(torch, rounding_name)
    return pm.forward(cfg, Wc, list(ids), rounding).numpy()


def oracle(cfg: dict, seed: int, stored: torch.dtype, compute: torch.dtype, ids: Sequence[int], rounding=None) -> np.ndarray:
    """Logits [T, vocab] of the plain implementation on the values the engine holds (matrices rounded to the
    compute dtype); with `rounding`, also rounding activations where a bfloat16 path stores them."""
    n = lambda d: str(d).replace("torch.", "")
    return _oracle_cached(json.dumps(cfg, sort_keys=True), seed, n(stored), n(compute), tuple(int(i) for i in ids),
                          "none" if rounding is None else n(rounding))


# float32 path: the only differences from the float64 plain implementation are float32 roundings of sums of
# at most a few hundred terms; logits are O(1).
F32_ATOL = 2e-5


def check_f32(got: np.ndarray, ref: np.ndarray, what: str):
    err = float(np.abs(got - ref).max())
    assert err <= F32_ATOL * max(1.0, float(np.abs(ref).max())), f"{what}: max |diff| {err:.3e} (float32 path)"
    return err


def check_bf16(got: np.ndarray, ref: np.ndarray, ref_rounded: np.ndarray, what: str, factor: float = 3.0):
    """The bfloat16 path may differ from the exact plain implementation by the noise that rounding activations
    to bfloat16 makes (measured by the plain implementation with those roundings), times `factor`."""
    noise = float(np.sqrt(np.mean((ref_rounded - ref) ** 2)))
    floor = 1e-3 * float(np.sqrt(np.mean(ref ** 2)))
    rms = float(np.sqrt(np.mean((got - ref) ** 2)))
    mx = float(np.abs(got - ref).max())
    bound = factor * max(noise, floor)
    assert rms <= bound, f"{what}: rms diff {rms:.3e} > {bound:.3e} (bf16 rounding noise {noise:.3e})"
    assert mx <= 6 * bound, f"{what}: max diff {mx:.3e} > {6 * bound:.3e}"
    return rms, noise
