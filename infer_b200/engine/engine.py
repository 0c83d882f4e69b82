"""The step function: one batch of (request, its next tokens) through the model, from the cache.

``Engine.step(entries)`` runs exactly the tokens it is given, as one batch: portions of prompts
beside single decoded tokens, cut anywhere.  Keys and values of earlier steps come from the
request's pages; the new tokens' keys and values are written before attention runs, so the tokens
of one portion see each other causally (the reference's row model, kernels/batch_gpu.cu:238-275 and
:294-297, generalised from "one prompt" or "one row per slot" to any mix).  It returns float32
logits at the wanted places, in the order of the entries and of their ``want`` lists.

All per-step integers (token ids, positions, which request each token belongs to, block tables,
wanted rows) travel to the device in ONE packed int32 buffer and one copy.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from ..config.registry import load_config
from ..config.specs import ModelSpec
from ..runtime import Runtime, parse_dtype
from ..weights.binder import load_weights
from .model import Model
from .. import parts as _builtin_parts   # noqa: F401  (registers the built-in parts)
from .. import models as _builtin_models  # noqa: F401  (registers the built-in architectures)


class OutOfPages(RuntimeError):
    """The step needs more pages than are free. Nothing was changed."""


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()        # indices into ``tokens`` whose logits are wanted


@dataclass
class StepContext:
    """The device-side description of one step's batch. Every tensor is int32 on the device."""
    n_tokens: int
    n_segments: int
    n_want: int
    token_ids: torch.Tensor          # [T]
    positions: torch.Tensor          # [T] absolute position of each token in its request
    token_seg: torch.Tensor          # [T] which segment (entry of the step) the token belongs to
    seg_start: torch.Tensor          # [S+1] first row of each segment
    seg_pos0: torch.Tensor           # [S] position of each segment's first token = cached length before the step
    seg_slot: torch.Tensor           # [S] state slot of each segment's request
    want_rows: torch.Tensor          # [n_want]
    block_tables: List[torch.Tensor]  # per cache group: [S, max_blocks]
    status: torch.Tensor             # [1] kernels raise it on a page index or token id out of range
    feedback: Optional[torch.Tensor] = None   # [slots] the sampler's last token per request (for token id -1)
    # host copies, for planning kernel launches without a device round trip
    seg_lens: List[int] = field(default_factory=list)
    seg_pos0_host: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_len: int = 0
    decode_only: bool = False
    extras: Dict[str, object] = field(default_factory=dict)   # per-step scratch that fast kernels share
    # sampling at the wanted rows inside the step (None: the step returns logits)
    sampling: Optional["SamplingInputs"] = None


@dataclass
class SamplingInputs:
    """Per wanted row, on the device: what the sampling kernel reads. ``filtered`` selects the top-k / top-p kernel."""
    temperature: torch.Tensor        # float32 [n_want]
    seed: torch.Tensor               # int64 [n_want]
    position: torch.Tensor           # int64 [n_want] position of the token fed: the noise stream's key
    top_k: torch.Tensor              # int64 [n_want]
    top_p: torch.Tensor              # float32 [n_want]
    slot: torch.Tensor               # int64 [n_want] state slot of the row's request (where its token is left)
    filtered: bool = False


@dataclass
class StepResult:
    """What ``Engine.try_step`` returns. ``ran[i]`` is False for an entry that was left out because it could not get
    its pages or would pass the sequence limit; such an entry's request is exactly as it was before the call.
    ``output`` holds the rows of the entries that ran (logits, or token ids when sampling), in their order."""
    output: torch.Tensor
    ran: List[bool]


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


FEEDBACK_TOKEN = -1           # as a decode entry's token: "what the sampler produced last for this request"
GRAPH_WIDTH_PAGES = 32        # decode-only block tables are padded to a multiple of this many pages (512 positions)
GRAPH_WARMUP_STEPS = 2        # eager steps of a shape before its graph is captured
MAX_GRAPHS = 48
GRAPH_COPIES = 2              # executable copies per decode shape, launched in turn
# Steps that hold prompt portions are captured too when their exact shape (segment lengths, wanted rows, table widths)
# comes a second time, as it does when prompts are cut into portions of the token budget or a short prompt joins a full
# batch of decoding requests: the first step of a shape runs eagerly (about 10 microseconds of host time per launch, two
# hundred launches), the second is captured, later ones are replayed. One executable each; a graph keeps its
# activations allocated, so only steps of at most PORTION_GRAPH_MAX_TOKENS tokens are captured and the captured shapes
# together hold at most PORTION_GRAPH_TOKEN_POOL tokens (the oldest goes first).
PORTION_GRAPH_AFTER = 1
MAX_PORTION_GRAPHS = 32
PORTION_GRAPH_MAX_TOKENS = 8192
PORTION_GRAPH_TOKEN_POOL = 16384


class _GraphEntry:
    def __init__(self, static: torch.Tensor):
        self.static, self.graphs, self.turn, self.warm, self.n_launches = static, [], 0, 0, 0
        self.pinned, self.flip = None, 0
        self.copied = None                 # per pinned buffer: the event recorded after the copy that read it last
        self.copies = GRAPH_COPIES


class Engine:
    """A model, its cache and the step function."""

    def __init__(self, spec: ModelSpec, weights: Mapping[str, torch.Tensor], dtype=torch.bfloat16,
                 device="cuda:0", max_tokens: int = 4096, max_requests: int = 8, page_size: int = 16,
                 max_seq_len: Optional[int] = None, kernels: Optional[Dict[str, str]] = None,
                 cache_budget_bytes: int = 0, cuda_graphs: bool = True):
        """max_tokens: positions the page pool of every cache group holds (rounded up to whole pages).
        max_requests: live requests (state slots). max_seq_len: longest request (default: the
        smaller of the model's position limit and max_tokens). cache_budget_bytes, if given, replaces max_tokens:
        the page pools together take at most this many bytes."""
        if not torch.cuda.is_available():
            raise RuntimeError("infer_b200 needs a CUDA device; there is no CPU path")
        dtype = parse_dtype(dtype)
        self.spec = spec
        n_pages = max(1, -(-int(max_tokens) // page_size))
        self.max_seq_len = int(min(spec.max_positions, max_seq_len or n_pages * page_size))
        self.rt = Runtime(dtype=dtype, device=torch.device(device), kernels=dict(kernels or {}),
                          max_seq_len=self.max_seq_len)
        torch.cuda.set_device(self.rt.device)
        self.model = Model(spec, weights, self.rt)
        needs = self.model.cache_needs()
        if cache_budget_bytes:
            probe = CacheManager(needs, 1, page_size, 1)
            n_pages = max(1, int(cache_budget_bytes) // max(1, probe.storage_bytes(dtype)))
        self.cache = CacheManager(needs, n_pages, page_size, max_requests)
        self.cache.make_storage(dtype, self.rt.device)
        self.cache_views = {cid: self.cache.view(cid) for cid in range(spec.num_caches)}
        from ..fast_ops import device_state
        self.status = device_state(self.rt.device).status     # shared with the fast kernels of this device
        self.steps_run = 0
        # The sampler leaves every request's last token here (indexed by state slot); a decode entry whose token is
        # FEEDBACK_TOKEN reads it, so that the host need not see a token before the next step is launched.
        self.next_tokens = torch.zeros(max(1, max_requests), dtype=torch.int32, device=self.rt.device)
        # Decode-only steps of the bfloat16 path are captured into CUDA graphs, one per (batch, wanted rows, table widths);
        # steps with prompt portions once their exact shape has repeated.
        self.use_graphs = bool(cuda_graphs) and dtype == torch.bfloat16 and self.model.graph_safe()
        self._graphs: Dict[tuple, _GraphEntry] = {}
        self._portion_seen: Dict[tuple, int] = {}         # how often a shape with prompt portions has come
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None

    # ------------------------------------------------------------------ construction helpers

    @classmethod
    def from_folder(cls, model_dir: str, **kw) -> "Engine":
        """A folder with config.json and model.safetensors; the model class follows config.json."""
        arch, typed = load_config(model_dir)
        spec = arch.to_spec(typed)
        return cls(spec, load_weights(model_dir, spec), **kw)

    # ------------------------------------------------------------------ requests

    def add_request(self, rid) -> None:
        self.cache.admit(rid)

    def end_request(self, rid) -> None:
        self.cache.release(rid)

    def has_request(self, rid) -> bool:
        return rid in self.cache.requests

    # ------------------------------------------------------------------ the step

    def _build_context(self, entries: Sequence[StepEntry], graphs: bool = False, sample=None):
        """Packs the step's integers on the host and places them on the device. With ``graphs`` and a decode-only
        step, the integers go into the static buffer of the step's shape (tokens, wanted rows, table widths), whose
        tensors a captured CUDA graph reads; returns (context, graph entry or None). ``sample``: one
        (SampleParams, position) per wanted row, in the order of the entries and their ``want`` lists; the sampling
        kernel's inputs then travel in the same buffer."""
        V, cache = self.spec.vocab_size, self.cache
        S = len(entries)
        T = sum(len(e.tokens) for e in entries)
        n_want = sum(len(e.want) for e in entries)
        n_groups = len(cache.groups)
        seg_lens = [len(e.tokens) for e in entries]
        pos0 = [cache.length(e.rid) for e in entries]
        widths = []
        for gi in range(n_groups):
            w = max(-(-(p + n) // cache.page_size) for p, n in zip(pos0, seg_lens))
            # decode-only steps round the table width up further, so that one captured graph serves many steps
            widths.append(_round_up(max(w, 1), GRAPH_WIDTH_PAGES if (graphs and T == S) else 8))
        if sample is not None and len(sample) != n_want:
            raise ValueError(f"sampling needs one (params, position) per wanted row: {len(sample)} given, {n_want} wanted")
        n_s = n_want if sample is not None else 0
        # layout of the packed buffer (int32 words; 64-bit fields take two, and every section starts on 16 bytes)
        sizes = [T, T, T, S + 1, S, S, max(n_want, 1)] + [S * w for w in widths] + [n_s, 2 * n_s, 2 * n_s, 2 * n_s, n_s, 2 * n_s]
        offs = np.concatenate([[0], np.cumsum([_round_up(s, 4) for s in sizes])])
        buf = np.zeros(int(offs[-1]), dtype=np.int32)
        ids, pos, seg = (buf[offs[i]:offs[i] + T] for i in range(3))
        seg_start = buf[offs[3]:offs[3] + S + 1]
        seg_pos0 = buf[offs[4]:offs[4] + S]
        seg_slot = buf[offs[5]:offs[5] + S]
        want = buf[offs[6]:offs[6] + n_want]
        want_slot = []
        r = w_i = 0
        for s, e in enumerate(entries):
            n = seg_lens[s]
            slot = cache.slot(e.rid)
            if n == 1:
                # a decoded token: the common case, kept free of array work
                tok = int(e.tokens[0])
                if tok == FEEDBACK_TOKEN and pos0[s] > 0:
                    pass                                # the request's last sampled token, still on the device
                elif not 0 <= tok < V:
                    raise ValueError(f"request {e.rid!r}: token id {tok} is outside the vocabulary [0, {V})")
                if pos0[s] + 1 > self.max_seq_len:
                    raise ValueError(f"request {e.rid!r}: {pos0[s] + 1} positions exceed the limit of {self.max_seq_len}")
                ids[r] = tok
                pos[r] = pos0[s]
                seg[r] = s
                seg_start[s] = r
                seg_pos0[s] = pos0[s]
                seg_slot[s] = slot
                for wi in e.want:
                    if int(wi) != 0:
                        raise ValueError(f"request {e.rid!r}: wanted place {wi} is outside its 1 tokens")
                    want[w_i] = r
                    want_slot.append(slot)
                    w_i += 1
                r += 1
                continue
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.ndim != 1 or n == 0:
                raise ValueError(f"request {e.rid!r}: a step entry needs at least one token")
            if toks.min() < 0 or toks.max() >= V:
                bad = int(toks[(toks < 0) | (toks >= V)][0])
                raise ValueError(f"request {e.rid!r}: token id {bad} is outside the vocabulary [0, {V})")
            if pos0[s] + n > self.max_seq_len:
                raise ValueError(f"request {e.rid!r}: {pos0[s] + n} positions exceed the limit of {self.max_seq_len}")
            ids[r:r + n] = toks
            pos[r:r + n] = np.arange(pos0[s], pos0[s] + n)
            seg[r:r + n] = s
            seg_start[s] = r
            seg_pos0[s] = pos0[s]
            seg_slot[s] = slot
            for wi in e.want:
                if not 0 <= int(wi) < n:
                    raise ValueError(f"request {e.rid!r}: wanted place {wi} is outside its {n} tokens")
                want[w_i] = r + int(wi)
                want_slot.append(slot)
                w_i += 1
            r += n
        seg_start[S] = T
        for gi in range(n_groups):
            tab = buf[offs[7 + gi]:offs[7 + gi] + S * widths[gi]].reshape(S, widths[gi])
            tab[:] = -1
            for s, e in enumerate(entries):
                t = cache.block_table(e.rid, gi)
                tab[s, :len(t)] = t
        o_s = 7 + n_groups                                  # first of the six sampling sections
        filtered = False
        if n_s:
            temp = buf[offs[o_s]:offs[o_s] + n_s].view(np.float32)
            seed = buf[offs[o_s + 1]:offs[o_s + 1] + 2 * n_s].view(np.int64)
            spos = buf[offs[o_s + 2]:offs[o_s + 2] + 2 * n_s].view(np.int64)
            topk = buf[offs[o_s + 3]:offs[o_s + 3] + 2 * n_s].view(np.int64)
            topp = buf[offs[o_s + 4]:offs[o_s + 4] + n_s].view(np.float32)
            sslot = buf[offs[o_s + 5]:offs[o_s + 5] + 2 * n_s].view(np.int64)
            for i, (p, position) in enumerate(sample):
                temp[i] = max(0.0, float(p.temperature))
                seed[i] = int(p.seed) & 0x7FFFFFFFFFFFFFFF
                spos[i] = int(position)
                topk[i] = int(getattr(p, "top_k", 0) or 0)
                topp[i] = float(getattr(p, "top_p", 1.0))
                sslot[i] = want_slot[i]
                if temp[i] > 0 and (topk[i] > 0 or topp[i] < 1.0):
                    filtered = True
        mode = 0 if sample is None else (2 if filtered else 1)
        entry = None
        key = None
        if graphs and T == S:
            key = (S, n_want, tuple(widths), mode)
        elif graphs and T <= PORTION_GRAPH_MAX_TOKENS:
            pkey = ("portions", tuple(seg_lens), n_want, tuple(widths), mode)
            if pkey in self._graphs:
                key = pkey
            else:
                if len(self._portion_seen) > 256:
                    self._portion_seen.clear()
                seen = self._portion_seen[pkey] = self._portion_seen.get(pkey, 0) + 1
                if seen > PORTION_GRAPH_AFTER:
                    key = pkey
        if key is not None:
            entry = self._graphs.get(key)
            if entry is None:
                portion = key[0] == "portions"
                if portion:
                    old = [k for k in self._graphs if k[0] == "portions"]
                    while old and (len(old) >= MAX_PORTION_GRAPHS or sum(sum(k[1]) for k in old) + T > PORTION_GRAPH_TOKEN_POOL):
                        self._graphs.pop(old.pop(0))
                elif len(self._graphs) >= MAX_GRAPHS:
                    self._graphs.pop(next(k for k in self._graphs if k[0] != "portions"))
                entry = self._graphs[key] = _GraphEntry(torch.empty(buf.size, dtype=torch.int32, device=self.rt.device))
                entry.pinned = [torch.empty(buf.size, dtype=torch.int32).pin_memory() for _ in range(2)]
                entry.copied = [torch.cuda.Event() for _ in range(2)]
                if portion:
                    entry.copies, entry.warm = 1, GRAPH_WARMUP_STEPS          # the shape has run eagerly before
            # Two pinned staging buffers alternate. The copy out of a buffer is asynchronous: before the buffer is
            # written again, the copy that read it last (two steps ago) must have run, or a caller that issues steps
            # without ever waiting for the device would overwrite integers that an earlier step has not yet taken.
            entry.flip ^= 1
            entry.copied[entry.flip].synchronize()
            host = entry.pinned[entry.flip]
            host.numpy()[:] = buf
            dev = entry.static
            dev.copy_(host, non_blocking=True)
            entry.copied[entry.flip].record()
        else:
            dev = torch.from_numpy(buf).pin_memory().to(self.rt.device, non_blocking=True)
        self.last_h2d_bytes = buf.nbytes

        def cut(i, n):
            return dev[int(offs[i]):int(offs[i]) + n]
        sampling = None
        if n_s:
            sampling = SamplingInputs(
                temperature=cut(o_s, n_s).view(torch.float32), seed=cut(o_s + 1, 2 * n_s).view(torch.int64),
                position=cut(o_s + 2, 2 * n_s).view(torch.int64), top_k=cut(o_s + 3, 2 * n_s).view(torch.int64),
                top_p=cut(o_s + 4, n_s).view(torch.float32), slot=cut(o_s + 5, 2 * n_s).view(torch.int64), filtered=filtered)
        ctx = StepContext(
            n_tokens=T, n_segments=S, n_want=n_want,
            token_ids=cut(0, T), positions=cut(1, T), token_seg=cut(2, T), seg_start=cut(3, S + 1),
            seg_pos0=cut(4, S), seg_slot=cut(5, S), want_rows=cut(6, n_want),
            block_tables=[cut(7 + gi, S * widths[gi]).view(S, widths[gi]) for gi in range(n_groups)],
            feedback=self.next_tokens, status=self.status, seg_lens=seg_lens, seg_pos0_host=pos0, max_q_len=max(seg_lens),
            max_ctx_len=max(p + n for p, n in zip(pos0, seg_lens)), decode_only=all(n == 1 for n in seg_lens),
            sampling=sampling)
        if entry is not None:
            # a graph's launch shapes must not depend on the step: bound the context by the table width
            ctx.max_ctx_len = max(widths) * cache.page_size if widths else ctx.max_ctx_len
        return ctx, entry

    def _run_model(self, ctx: StepContext) -> torch.Tensor:
        """The model on the step's tokens; with sampling inputs, the sampling kernel on the logits as well (each
        token is also left at next_tokens[slot] for a later FEEDBACK_TOKEN)."""
        logits = self.model.forward(ctx, self.cache_views)
        sp = ctx.sampling
        if sp is None or ctx.n_want == 0:
            return logits
        if sp.filtered:
            return ops.sample_filtered(logits, sp.temperature, sp.seed, sp.position, sp.top_k, sp.top_p,
                                       self.next_tokens, sp.slot)
        return ops.sample(logits, sp.temperature, sp.seed, sp.position, self.next_tokens, sp.slot)

    def step(self, entries: Sequence[StepEntry], sample=None) -> torch.Tensor:
        """Runs one batch; returns float32 logits [wanted places, vocab] on the device. With ``sample`` (one
        (SampleParams, position) per wanted place, in order) the step samples on the device as well and returns
        int32 token ids [wanted places] instead; each id also stays on the device for its request (FEEDBACK_TOKEN).
        With CUDA graphs on, the tensor returned by a captured step is reused by the next step of the same shape:
        read it, or enqueue its copy, before that. Steps may be issued back to back without waiting for the device.
        Raises OutOfPages (nothing changed) if the pages for all entries together are not free."""
        return self._step(entries, sample, False).output

    def try_step(self, entries: Sequence[StepEntry], sample=None) -> StepResult:
        """As ``step``, but an entry that cannot get its pages (after the entries before it have taken theirs) or
        that would pass the sequence limit is left out instead of failing the call: the others run, the result says
        which (``ran``), and a request that was left out is untouched (the reference's per-row -1,
        kernels/batch_gpu.cu:386-410). ``sample`` still has one item per wanted place of ALL entries."""
        return self._step(entries, sample, True)

    def _step(self, entries, sample, partial: bool) -> StepResult:
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        empty_dtype = torch.int32 if sample is not None else torch.float32
        empty_shape = (0,) if sample is not None else (0, self.spec.vocab_size)
        if not entries:
            return StepResult(torch.empty(empty_shape, dtype=empty_dtype, device=self.rt.device), [])
        rids = [e.rid for e in entries]
        if len(set(rids)) != len(rids):
            raise ValueError("a request may appear once in a step")
        for e in entries:
            if e.rid not in self.cache.requests:
                raise KeyError(f"request {e.rid!r} is not admitted (add_request first)")
        ran = [True] * len(entries)
        if partial:
            taken = []
            for i, e in enumerate(entries):
                fits = self.cache.length(e.rid) + len(e.tokens) <= self.max_seq_len
                if fits and self.cache.can_reserve(taken + [(e.rid, len(e.tokens))]):
                    taken.append((e.rid, len(e.tokens)))
                else:
                    ran[i] = False
            if sample is not None:
                keep, w = [], 0
                for e, ok in zip(entries, ran):
                    keep += list(sample[w:w + len(e.want)]) if ok else []
                    w += len(e.want)
                sample = keep
            entries = [e for e, ok in zip(entries, ran) if ok]
            if not entries:
                return StepResult(torch.empty(empty_shape, dtype=empty_dtype, device=self.rt.device), ran)
        wanted = [(e.rid, len(e.tokens)) for e in entries]
        if not self.cache.can_reserve(wanted):
            raise OutOfPages(f"step needs more pages than are free (free per group: {self.cache.pages_free()})")
        for rid, n in wanted:
            if not self.cache.reserve(rid, n):
                raise AssertionError("reserve failed after can_reserve succeeded")
        try:
            ctx, entry = self._build_context(entries, self.use_graphs, sample)
        except Exception:
            for rid, _ in wanted:
                self.cache.unreserve(rid)
            raise
        with torch.cuda.device(self.rt.device):
            if entry is None:
                out = self._run_model(ctx)
            elif len(entry.graphs) == entry.copies:
                # Copies of the graph take turns: launching an executable graph again while its previous launch is
                # still running is serialised by the driver, which would put the launch cost between two steps.
                entry.turn = (entry.turn + 1) % entry.copies
                graph, out = entry.graphs[entry.turn]
                graph.replay()
                ops._LAUNCHES[0] += entry.n_launches
            elif entry.warm < GRAPH_WARMUP_STEPS:
                # The first steps of a shape run eagerly: they build libraries, size workspaces, set attributes.
                entry.warm += 1
                out = self._run_model(ctx)
            else:
                graph = torch.cuda.CUDAGraph()
                n0 = ops.kernel_launches()
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    out = self._run_model(ctx)
                entry.n_launches = ops.kernel_launches() - n0        # kernels of this package inside the graph
                ops._LAUNCHES[0] = n0
                entry.graphs.append((graph, out))
                graph.replay()
                ops._LAUNCHES[0] += entry.n_launches
        for rid, n in wanted:
            self.cache.advance(rid, n)
        self.steps_run += 1
        if sample is not None and ctx.n_want == 0:
            out = torch.empty((0,), dtype=torch.int32, device=self.rt.device)
        return StepResult(out, ran)

    def check_status(self) -> None:
        """Synchronises and raises if a kernel met a page index or token id out of range."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            what = {1: "a token id outside the table", 2: "a cache write through an invalid page",
                    3: "a cache read through an invalid page", 101: "a tensor-core GEMM's copy wait ran out",
                    102: "a tensor-core GEMM's operand wait ran out", 103: "a tensor-core GEMM's accumulator wait ran out",
                    }.get(code, f"code {code}")
            raise RuntimeError(f"device status word was raised: {what}")
