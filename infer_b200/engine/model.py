"""A model put together from a ModelSpec: token table, blocks of parts, run order, final norm, head.

The class is the same for every architecture; what differs is the spec.  ``forward`` runs the
tokens of one step (any mix of prompt portions and single decoded tokens) and returns float32
logits at the wanted rows only.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from .. import ops
from ..config.specs import LayerSpec, ModelSpec
from ..parts.base import Block, build_part, part_class
from ..parts.linear import Linear
from ..runtime import Runtime
from ..weights.binder import check_weights, expected_tensors


class Model:
    def __init__(self, spec: ModelSpec, weights: Mapping[str, torch.Tensor], runtime: Runtime):
        spec.validate()
        check_weights(weights, spec)
        self.spec, self.rt = spec, runtime
        self.blocks: List[Block] = [self._build_block(ls, weights) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self._load_part(self.final_norm, "norm", spec.final_norm, weights)
        table = weights[spec.embedding_name]
        # The token table is read row by row; it keeps the compute dtype of the matrices.
        self.embedding = table.to(device=runtime.device, dtype=runtime.dtype).contiguous()
        if spec.head_name is None:
            self.head = Linear.__new__(Linear)
            self.head.rt, self.head.weight, self.head.bias = runtime, self.embedding, None
            self.head.out_features, self.head.in_features = self.embedding.shape
        else:
            self.head = Linear(runtime, weights[spec.head_name])
        self.head.prefetch_next = None
        self.plan_prefetch()

    def plan_prefetch(self, distance: int = 2) -> None:
        """Walks the kernels of a step in run order and tells each to fetch, while it runs, the weights of the kernel
        `distance` places later (a decode step's kernels are bound by latency and leave HBM idle most of the time;
        with the hint the next products find their weights in L2)."""
        line = []
        for call in self.spec.schedule:
            b = self.blocks[call.layer]
            line += list(b.mixer.stations()) + list(b.feed_forward.stations())
        line.append((self.head, self.head.weight))
        for i, (holder, _) in enumerate(line):
            ahead = [w for _, w in line[i + distance:i + distance + 1] if w is not None]
            holder.prefetch_next = ahead[0] if ahead else None

    def _load_part(self, part, family, pspec, weights):
        names = part_class(family, pspec.kind).param_shapes(pspec)
        part.load({local: weights[pspec.prefix + local] for local in names})

    def _build_block(self, ls: LayerSpec, weights) -> Block:
        parts = {}
        for attr, family, pspec in (("mixer", "mixer", ls.mixer), ("feed_forward", "feed_forward", ls.feed_forward),
                                    ("mixer_norm", "norm", ls.mixer_norm), ("feed_forward_norm", "norm", ls.feed_forward_norm)):
            part = build_part(family, pspec, self.rt)
            self._load_part(part, family, pspec, weights)
            parts[attr] = part
        return part_class("block", ls.block)(**parts)

    def cache_needs(self) -> Dict[int, object]:
        """cache index -> what the mixer that writes it needs from the cache manager."""
        needs: Dict[int, object] = {}
        for call in self.spec.schedule:
            need = self.blocks[call.layer].mixer.cache_need()
            if call.write_cache:
                needs[call.cache] = need
            elif needs.get(call.cache) != need:
                raise ValueError(f"layer {call.layer} reads cache {call.cache}, whose writer has another layout")
        return needs

    def forward(self, step, cache_views: Mapping[int, object]) -> torch.Tensor:
        h = ops.embedding(self.embedding, step.token_ids, step.status, getattr(step, "feedback", None),
                          step.token_seg, step.seg_slot)                          # float32 [T, hidden]
        for call in self.spec.schedule:
            h = self.blocks[call.layer].forward(h, step, cache_views[call.cache], call.write_cache)
        if step.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        normed = self.final_norm.forward(h, rows=step.want_rows)                  # [wanted, hidden]
        return self.head(normed, out_dtype=torch.float32)                          # float32 [wanted, vocab]

    def weight_bytes(self) -> int:
        """Bytes of every distinct parameter tensor on the device (a decode step reads each once)."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, Linear):
                visit(obj.weight), visit(obj.bias)
            elif hasattr(obj, "__dict__"):
                for k, v in vars(obj).items():
                    if k not in ("rt", "spec"):
                        visit(v)
        for b in self.blocks:
            for p in (b.mixer, b.feed_forward, b.mixer_norm, b.feed_forward_norm):
                visit(p)
        visit(self.final_norm), visit(self.head), visit(self.embedding)
        return total
