"""The engine as the scheduler sees it (step function + sampler), and the Python entry point ``LLM``.

Option names follow the reference where it has them: ``slots``, ``max_seq``, ``budget_mb``
(src/main_serve_bench.cpp:15-27; kernels/batch_gpu.h:38-40), ``max_new``, ``temperature``, ``seed``, ``eos_id``
(src/scheduler.h:36-87), ``top_k`` / ``top_p`` (src/sampler.h:16-25).
"""
from __future__ import annotations

from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..sampling.sampler import Sampler
from .engine import Engine, StepEntry
from .scheduler import (BatchEngine, BatchItem, Completed, Request, SampleParams, Scheduler, SchedulerConfig)


class PendingTokens:
    """Sampled token ids on their way to the host."""

    def __init__(self, rids, host, event):
        self.rids, self._host, self._event = rids, host, event

    def result(self) -> Dict[Hashable, int]:
        if self._event is None:
            return {}
        self._event.synchronize()
        return {rid: int(t) for rid, t in zip(self.rids, self._host.tolist())}


class GenerationEngine(BatchEngine):
    """Runs a planned batch as ONE step and samples on the device; only token ids cross to the host."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.sampler = Sampler(engine.rt.device)       # for callers that sample from logits themselves
        self.max_seq_len = engine.max_seq_len
        self.max_requests = engine.cache.n_slots
        self._pinned, self._flip = {}, 0

    def capacity_tokens(self) -> int:
        return min(self.engine.cache.pages_total()) * self.engine.cache.page_size if self.engine.cache.groups else 1 << 60

    def add_request(self, rid) -> None:
        self.engine.add_request(rid)

    def end_request(self, rid) -> None:
        self.engine.end_request(rid)

    def can_run(self, wanted) -> bool:
        return self.engine.cache.can_reserve(list(wanted))

    def has_room(self, prompt_len: int) -> bool:
        need = -(-prompt_len // self.engine.cache.page_size) + 1
        return all(f >= need for f in self.engine.cache.pages_free())

    def tokens_that_fit(self, wanted, rid, n: int) -> int:
        cache = self.engine.cache
        lo, hi = 0, n
        while lo < hi:                                  # largest m <= n with can_reserve(wanted + (rid, m))
            mid = (lo + hi + 1) // 2
            if cache.can_reserve(list(wanted) + [(rid, mid)]):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def run_async(self, batch: Sequence[BatchItem]) -> "PendingTokens":
        """Enqueues the step, the sampling and the copy of the sampled ids to pinned host memory, and returns at
        once. Every sampled token also stays on the device (engine.next_tokens[slot]); a later decode item may pass
        FEEDBACK_TOKEN instead of the id."""
        entries = [StepEntry(b.rid, b.tokens, [len(b.tokens) - 1] if b.sample is not None else []) for b in batch]
        rows = [b for b in batch if b.sample is not None]
        # the sampling kernel's inputs travel in the step's one packed buffer and the kernel runs inside the step
        # (inside its CUDA graph when the shape is captured): one copy in, one launch, one copy out per step
        ids = self.engine.step(entries, sample=[(b.sample, b.position) for b in rows])
        if not rows:
            return PendingTokens([], None, None)
        # Pinned buffers for the ids take turns (four per batch size): a buffer comes round again only after the
        # result of the step that used it last has been read, which waits on that step's event.
        self._flip = (self._flip + 1) % 4
        key = (len(rows), self._flip)
        slot = self._pinned.get(key)
        if slot is None:
            slot = self._pinned[key] = (torch.empty(len(rows), dtype=torch.int32).pin_memory(), torch.cuda.Event())
        host, event = slot
        event.synchronize()                     # the copy that wrote this buffer last has landed (no-op if never used)
        host.copy_(ids, non_blocking=True)
        event.record()
        return PendingTokens([b.rid for b in rows], host, event)

    def run(self, batch: Sequence[BatchItem]) -> Dict[Hashable, int]:
        return self.run_async(batch).result()

    def pages_in_use(self) -> int:
        return max(self.engine.cache.pages_in_use(), default=0)

    def pages_total(self) -> int:
        return max(self.engine.cache.pages_total(), default=0)


class LLM:
    """Python entry point: a model folder in, token ids out.

        llm = LLM("/path/to/model", dtype="bfloat16", slots=8, max_seq=4096)
        outs = llm.generate([[1, 2, 3], [4, 5]], max_new=16)                    # greedy
        outs = llm.generate(prompts, max_new=16, temperature=0.8, seed=7)      # seeded sampling
    """

    def __init__(self, model: str, dtype="bfloat16", device: str = "cuda:0", slots: int = 8, max_seq: int = 4096,
                 budget_mb: int = 0, max_batch_tokens: int = 512, page_size: int = 16, eos_id: Optional[int] = None,
                 kernels: Optional[Dict[str, str]] = None, weights=None, spec=None, overlap: bool = True,
                 kv_blocks: int = 0):
        """slots: live requests; max_seq: per-sequence cap; budget_mb: size of the page pool in MiB, or kv_blocks: its
        size in pages (both 0 = reserve slots x max_seq, as the reference does, kernels/batch_gpu.cu:92-95);
        max_batch_tokens: the token budget of a step, which is also the largest prompt portion. ``spec`` + ``weights``
        may replace the folder."""
        from ..config.registry import load_config
        from ..weights.binder import load_weights
        if spec is None:
            arch, typed = load_config(model)
            spec = arch.to_spec(typed)
            weights = load_weights(model, spec)
        self.engine = Engine(spec, weights, dtype=dtype, device=device,
                             max_tokens=int(kv_blocks) * page_size if kv_blocks else slots * max_seq,
                             max_requests=slots, page_size=page_size, max_seq_len=max_seq, kernels=kernels,
                             cache_budget_bytes=int(budget_mb) << 20)
        self.batch_engine = GenerationEngine(self.engine)
        default_eos = eos_id if eos_id is not None else (spec.eos_token_id if spec.eos_token_id is not None else -1)
        self.scheduler_config = SchedulerConfig(eos_id=default_eos, max_batch_tokens=max_batch_tokens, overlap=overlap)
        self._next_id = 0

    def new_scheduler(self, **overrides) -> Scheduler:
        cfg = SchedulerConfig(**{**self.scheduler_config.__dict__, **overrides})
        return Scheduler(self.batch_engine, cfg)

    def generate(self, prompts: Sequence[Sequence[int]], max_new: int = 16, temperature: float = 0.0, seed: int = 0,
                 top_k: int = 0, top_p: float = 1.0, eos_id: Optional[int] = None,
                 on_token: Optional[Callable[[Hashable, int], None]] = None) -> List[List[int]]:
        """Generates up to max_new tokens for every prompt (lists of token ids); returns the new ids per prompt
        (eos included if hit)."""
        sch = self.new_scheduler(on_token=on_token)
        ids = []
        for p in prompts:
            rid = self._next_id
            self._next_id += 1
            ids.append(rid)
            sch.submit(Request(rid, [int(t) for t in p], max_new, 0,
                               SampleParams(temperature, seed, top_k, top_p), eos_id))
        sch.run_until_idle()
        done = {c.id: c.tokens for c in sch.completed}
        self.last_scheduler = sch
        return [done[i] for i in ids]
