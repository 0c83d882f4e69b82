"""Continuous-batching scheduler over the step function.

Names and meanings follow the reference's scheduler (src/scheduler.h:36-161, src/scheduler.cpp):
``Request{id, prompt, max_new, arrival_step, sample{temperature, seed}, eos_id}``,
``Completed{id, reason, tokens, ...}``, ``StopReason``, ``submit / cancel / step / run_until_idle /
completed``, static batching as the comparison baseline, an event ring, and recompute-style
preemption of the most recently admitted request.

What differs, because the step function here takes mixed batches: a prompt is not run whole at
admission (src/scheduler.cpp:102) but cut into portions under a token budget.  Every step takes
one decode token from every request that is decoding, then fills what is left of
``max_batch_tokens`` with prompt portions, oldest request first.

When pages run out (decided here, tested in tests/test_scheduler.py):
  1. prompt portions are dropped from the step, youngest request first, then the oldest remaining
     portion is shortened to what the free pages allow;
  2. if the decode tokens alone do not fit, or no request can move at all, the most recently
     admitted request is preempted: its pages go back, and it re-enters the queue at the front with
     prompt := prompt + generated tokens (src/scheduler.cpp:148-173); a victim that is half way
     through its prompt simply starts again;
  3. a request that could not fit even alone is refused at ``submit`` (prompt + max_new must fit
     both the sequence limit and the page pool), so step 2 always ends.

Overlap (``SchedulerConfig.overlap``): a step is launched before the tokens of the step before it have reached
the host. The engine keeps every request's last sampled token on the device, and a decode item then carries
FEEDBACK_TOKEN instead of an id; the host reads a step's tokens while the next step runs, so callbacks, eos and
retirement come one step late (a request that hit eos has then run one token too many, which is dropped).
max_new and the sequence limit are counted, not read, so they stop a request on time. Before anything is
preempted the tokens in flight are read, so a victim's new prompt holds everything it generated.
"""
from __future__ import annotations

import json
import time
from collections import deque
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

USE_DEFAULT_EOS = None
FEEDBACK_TOKEN = -1        # a decode item's token when the previous step's result has not reached the host yet


@dataclass
class SampleParams:
    """temperature 0 = greedy (exact argmax); otherwise sample logits / temperature with a noise stream keyed by
    (seed, position) (src/scheduler.h:36-39). top_k 0 and top_p 1 switch those filters off (src/sampler.h:16-25)."""
    temperature: float = 0.0
    seed: int = 0
    top_k: int = 0
    top_p: float = 1.0


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    max_new: int = 32
    arrival_step: int = 0
    sample: SampleParams = field(default_factory=SampleParams)
    eos_id: Optional[int] = USE_DEFAULT_EOS           # None: the scheduler's eos_id; -1: never stop on eos
    generated_so_far: List[int] = field(default_factory=list)   # set by preemption


class StopReason(IntEnum):
    EOS = 0
    MAX_NEW = 1
    CACHE_FULL = 2
    CANCELLED = 3


@dataclass
class Completed:
    id: Hashable
    reason: StopReason
    tokens: List[int]
    admitted_step: int = 0
    finished_step: int = 0
    admitted_ms: float = 0.0
    first_token_ms: float = 0.0
    finished_ms: float = 0.0
    preemptions: int = 0


@dataclass
class Event:
    kind: str                 # "admit" | "step" | "retire" | "preempt"
    step: int
    request_id: Hashable = None
    reason: int = 0
    batch_size: int = 0       # live requests after the event
    tokens: int = 0           # step: tokens run (decode + prompt); retire: generated count
    decoded: int = 0
    t_ms: float = 0.0
    dur_ms: float = 0.0
    pool_in_use: int = 0
    pool_total: int = 0


class EventRing:
    """Keeps the last `capacity` events (src/scheduler.h:117-134)."""

    def __init__(self, capacity: int):
        self._buf: List[Optional[Event]] = [None] * max(1, capacity)
        self._head = self._tail = self.dropped = 0

    def push(self, e: Event) -> None:
        self._buf[self._head % len(self._buf)] = e
        self._head += 1
        if self._head - self._tail > len(self._buf):
            self._tail = self._head - len(self._buf)
            self.dropped += 1

    def __len__(self) -> int:
        return self._head - self._tail

    def __getitem__(self, i: int) -> Event:
        return self._buf[(self._tail + i) % len(self._buf)]

    def write_jsonl(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            for i in range(len(self)):
                e = self[i]
                d = dict(e.__dict__)
                d["request_id"] = None if e.request_id is None else str(e.request_id)
                f.write(json.dumps(d) + "\n")


@dataclass
class SchedulerConfig:
    continuous: bool = True             # False = static batching baseline
    eos_id: int = -1                    # -1 = never stop on eos
    max_batch_tokens: int = 512         # token budget of one step
    overlap: bool = False               # launch step n+1 before the tokens of step n have reached the host
    event_capacity: int = 1 << 16
    on_token: Optional[Callable[[Hashable, int], None]] = None
    on_done: Optional[Callable[[Completed], None]] = None


@dataclass
class BatchItem:
    """One request's share of a step: its next tokens, and how to sample if the step ends its prompt
    (or is a decode token). ``position`` is the position of the last token fed: the sampler's step key."""
    rid: Hashable
    tokens: List[int]
    sample: Optional[SampleParams]
    position: int = 0


class BatchEngine:
    """What the scheduler needs from an engine; tests drive the scheduler with a fake one."""
    max_seq_len: int
    max_requests: int

    def capacity_tokens(self) -> int: raise NotImplementedError                # positions the page pool holds
    def add_request(self, rid) -> None: raise NotImplementedError
    def end_request(self, rid) -> None: raise NotImplementedError
    def tokens_that_fit(self, wanted: Sequence[Tuple[Hashable, int]], rid, n: int) -> int:
        """How many of request rid's next n tokens fit, given that `wanted` is already promised."""
        raise NotImplementedError
    def can_run(self, wanted: Sequence[Tuple[Hashable, int]]) -> bool: raise NotImplementedError
    def has_room(self, prompt_len: int) -> bool:
        """Could a prompt of this length get its pages right now, and one more? (kernels/batch_gpu.cu:277-279)"""
        raise NotImplementedError
    def run(self, batch: Sequence[BatchItem]) -> Dict[Hashable, int]:
        """Runs the batch as one step; returns the sampled token of every item that has ``sample``."""
        raise NotImplementedError
    def run_async(self, batch: Sequence[BatchItem]):
        """Starts the step and returns an object whose ``result()`` gives what ``run`` returns. An item's token may
        be FEEDBACK_TOKEN: the token sampled last for that request, which the engine kept. The default runs at once."""
        done = self.run(batch)

        class _Done:
            def result(self_inner):
                return done
        return _Done()
    def pages_in_use(self) -> int: raise NotImplementedError
    def pages_total(self) -> int: raise NotImplementedError


@dataclass
class _Active:
    req: Request
    out: List[int]
    prompt_len: int                 # original prompt length (without tokens generated before a preemption)
    fed: int = 0                    # tokens of req.prompt already in the cache
    last_token: int = -1
    admitted_step: int = 0
    admitted_seq: int = 0
    admitted_ms: float = 0.0
    first_token_ms: float = 0.0
    preemptions: int = 0
    pending: int = 0                # tokens sampled on the device that the host has not read yet (overlap mode)

    @property
    def decoding(self) -> bool:
        return self.fed >= len(self.req.prompt)


class Scheduler:
    def __init__(self, engine: BatchEngine, cfg: Optional[SchedulerConfig] = None):
        self.eng, self.cfg = engine, cfg or SchedulerConfig()
        if self.cfg.max_batch_tokens < 1:
            raise ValueError("max_batch_tokens must be at least 1")
        self.queue: Deque[Request] = deque()
        self.active: Dict[Hashable, _Active] = {}
        self.completed: List[Completed] = []
        self.events = EventRing(self.cfg.event_capacity)
        self._cancelled = set()
        self._step = 0
        self._admit_seq = 0
        self.preemptions = 0
        self._t0 = time.perf_counter()
        self._preempt_counts: Dict[Hashable, int] = {}
        self._pending = None            # (PendingTokens, batch) of the step in flight (overlap mode)

    # ------------------------------------------------------------------ public

    def submit(self, r: Request) -> None:
        if not r.prompt:
            raise ValueError(f"request {r.id!r}: empty prompt")
        total = len(r.prompt) + r.max_new
        limit = min(self.eng.max_seq_len, self.eng.capacity_tokens())
        if total > limit:
            raise ValueError(f"request {r.id!r} does not fit the cache: prompt + max_new = {total} > {limit}")
        self.queue.append(r)

    def cancel(self, request_id) -> None:
        self._cancelled.add(request_id)

    def idle(self) -> bool:
        return not self.queue and not self.active and self._pending is None

    @property
    def steps(self) -> int:
        return self._step

    def run_until_idle(self) -> None:
        while not self.idle():
            self.step()

    # ------------------------------------------------------------------ internals

    def _now(self) -> float:
        return (time.perf_counter() - self._t0) * 1e3

    def _eos(self, r: Request) -> int:
        return self.cfg.eos_id if r.eos_id is None else r.eos_id

    def _event(self, kind, rid=None, reason=0, tokens=0, decoded=0, t=None, dur=0.0):
        self.events.push(Event(kind, self._step, rid, int(reason), len(self.active), tokens, decoded,
                               self._now() if t is None else t, dur, self.eng.pages_in_use(), self.eng.pages_total()))

    def _retire(self, rid, reason: StopReason) -> None:
        a = self.active.pop(rid)
        self.eng.end_request(rid)
        c = Completed(rid, reason, a.out, a.admitted_step, self._step, a.admitted_ms, a.first_token_ms,
                      self._now(), a.preemptions)
        self.completed.append(c)
        self._event("retire", rid, reason, tokens=len(c.tokens))
        if self.cfg.on_done:
            self.cfg.on_done(c)

    def _finish_unstarted(self, r: Request, reason: StopReason) -> None:
        now = self._now()
        c = Completed(r.id, reason, list(r.generated_so_far), self._step, self._step, now, now, now,
                      self._preempt_counts.get(r.id, 0))
        self.completed.append(c)
        if self.cfg.on_done:
            self.cfg.on_done(c)

    def _admit(self) -> None:
        if not self.cfg.continuous and self.active:
            return
        while self.queue and len(self.active) < self.eng.max_requests:
            r = self.queue[0]
            if r.id in self._cancelled:
                self.queue.popleft()
                self._cancelled.discard(r.id)
                self._finish_unstarted(r, StopReason.CANCELLED)
                continue
            if r.arrival_step > self._step:
                break                                   # FIFO: nothing later is due
            if self.active and not self.eng.has_room(len(r.prompt)):
                break                                   # wait for pages (src/scheduler.cpp:95)
            self.queue.popleft()
            self.eng.add_request(r.id)
            a = _Active(r, list(r.generated_so_far), len(r.prompt) - len(r.generated_so_far),
                        admitted_step=self._step, admitted_seq=self._admit_seq, admitted_ms=self._now(),
                        preemptions=self._preempt_counts.get(r.id, 0))
            self._admit_seq += 1
            self.active[r.id] = a
            self._event("admit", r.id, tokens=len(r.prompt))

    def _preempt_one(self) -> Optional[Hashable]:
        """Evicts the most recently admitted request; it will recompute from prompt + generated."""
        if not self.active:
            return None
        rid = max(self.active, key=lambda k: self.active[k].admitted_seq)
        a = self.active.pop(rid)
        self.eng.end_request(rid)
        r = a.req
        r.prompt = list(r.prompt) + a.out[len(r.generated_so_far):]
        r.generated_so_far = list(a.out)
        r.arrival_step = 0
        self._preempt_counts[rid] = a.preemptions + 1
        self.queue.appendleft(r)
        self.preemptions += 1
        self._event("preempt", rid)
        return rid

    def _plan(self) -> List[BatchItem]:
        """One decode token per decoding request, then prompt portions under the token budget, shrunk to the
        free pages."""
        order = sorted(self.active.values(), key=lambda a: a.admitted_seq)
        decode = [a for a in order if a.decoding]
        batch: List[BatchItem] = []
        wanted: List[Tuple[Hashable, int]] = []
        budget = self.cfg.max_batch_tokens
        for a in decode:
            if budget <= 0:
                break
            n_out = len(a.out) + a.pending
            if n_out >= a.req.max_new or a.prompt_len + n_out >= self.eng.max_seq_len:
                continue                                # it ends as soon as its pending token has been read
            pos = len(a.req.prompt) + n_out - len(a.req.generated_so_far) - 1
            batch.append(BatchItem(a.req.id, [FEEDBACK_TOKEN if a.pending else a.last_token], a.req.sample, pos))
            wanted.append((a.req.id, 1))
            budget -= 1
        if wanted and not self.eng.can_run(wanted):
            return []                                   # the caller preempts and plans again
        for a in order:
            if a.decoding or budget <= 0:
                continue
            n = min(len(a.req.prompt) - a.fed, budget)
            n = self.eng.tokens_that_fit(wanted, a.req.id, n)
            if n <= 0:
                break                                   # younger requests wait behind the older one
            toks = a.req.prompt[a.fed:a.fed + n]
            ends = a.fed + n == len(a.req.prompt)
            batch.append(BatchItem(a.req.id, toks, a.req.sample if ends else None, a.fed + n - 1))
            wanted.append((a.req.id, n))
            budget -= n
        return batch

    def _take_tokens(self, batch, sampled) -> int:
        """Appends the sampled tokens to their requests, calls back, and retires what has finished."""
        decoded = 0
        for b in batch:
            if b.sample is None:
                continue
            a = self.active.get(b.rid)
            if a is None or b.rid not in sampled:
                continue                                # retired, cancelled or preempted meanwhile: the token is dropped
            if a.pending:
                a.pending -= 1
            tok = int(sampled[b.rid])
            if a.first_token_ms == 0.0:
                a.first_token_ms = self._now()
            a.last_token = tok
            a.out.append(tok)
            decoded += 1
            if self.cfg.on_token:
                self.cfg.on_token(b.rid, tok)
            if tok == self._eos(a.req):
                self._retire(b.rid, StopReason.EOS)
            elif len(a.out) >= a.req.max_new:
                self._retire(b.rid, StopReason.MAX_NEW)
            elif a.prompt_len + len(a.out) >= self.eng.max_seq_len:
                self._retire(b.rid, StopReason.CACHE_FULL)
        return decoded

    def _apply_pending(self) -> int:
        if self._pending is None:
            return 0
        handle, batch, seqs = self._pending
        self._pending = None
        # a request admitted again after a preemption must not take a token of its earlier life
        live = [b for b in batch if b.rid in self.active and self.active[b.rid].admitted_seq == seqs[b.rid]]
        return self._take_tokens(live, handle.result())

    def step(self) -> int:
        """Cancel -> admit -> plan (preempting while nothing can move) -> run -> retire. Returns tokens decoded."""
        t_start = self._now()
        for rid in [r for r in self.active if r in self._cancelled]:
            self._cancelled.discard(rid)
            self._retire(rid, StopReason.CANCELLED)
        self._admit()
        batch = self._plan()
        while not batch and self.active:
            if self._pending is not None:
                self._apply_pending()                   # a victim's prompt must hold every token it has generated
                batch = self._plan()
                continue
            if len(self.active) == 1:
                only = next(iter(self.active.values()))
                raise RuntimeError(f"scheduler: out of cache pages with nothing to preempt (request {only.req.id!r})")
            self._preempt_one()
            batch = self._plan()
        decoded = 0
        n_tokens = sum(len(b.tokens) for b in batch)
        if self.cfg.overlap:
            launched = None
            if batch:
                for b in batch:
                    a = self.active[b.rid]
                    if not a.decoding:
                        a.fed += len(b.tokens)
                    if b.sample is not None:
                        a.pending += 1
                seqs = {b.rid: self.active[b.rid].admitted_seq for b in batch}
                launched = (self.eng.run_async(batch), batch, seqs)
            decoded = self._apply_pending()             # the previous step's tokens, while this step runs
            self._pending = launched
        elif batch:
            sampled = self.eng.run(batch)
            for b in batch:
                a = self.active[b.rid]
                if not a.decoding:
                    a.fed += len(b.tokens)
            decoded = self._take_tokens(batch, sampled)
        self._event("step", tokens=n_tokens, decoded=decoded, t=t_start, dur=self._now() - t_start)
        self._step += 1
        return decoded
