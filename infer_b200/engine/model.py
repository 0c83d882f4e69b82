"""A model put together from a ModelSpec: embedding, blocks of parts, run order, final norm, head.

The class is the same for every architecture; what differs is the spec.  ``forward`` runs the
tokens of one step (any mix of prompt portions and single decoded tokens) and returns float32
logits at the wanted rows only.  The model names no slot of a layer and no kind of part: it builds
what the spec lists and calls ``forward`` on the embedding, the blocks, the final norm and the head.
"""
from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from ..config.specs import LayerSpec, ModelSpec, PartSpec
from ..parts.base import Block, Part, build_part, part_class
from ..parts.linear import Linear
from ..runtime import Runtime
from ..weights.binder import check_weights


class Model:
    def __init__(self, spec: ModelSpec, weights: Mapping[str, torch.Tensor], runtime: Runtime):
        spec.validate()
        check_weights(weights, spec)
        self.spec, self.rt = spec, runtime
        self.embedding = self._build_part("embedding", spec.embedding, weights)
        self.blocks: List[Block] = [self._build_block(ls, weights) for ls in spec.layers]
        self.final_norm = self._build_part("norm", spec.final_norm, weights)
        self.head = self._build_part("head", spec.head, weights)
        self.head.tie(self.embedding)

    def _build_part(self, family: str, pspec: PartSpec, weights) -> Part:
        part = build_part(family, pspec, self.rt)
        names = part_class(family, pspec.kind).param_shapes(pspec)
        part.load({local: weights[pspec.prefix + local] for local in names})
        return part

    def _build_block(self, ls: LayerSpec, weights) -> Block:
        parts = {slot: self._build_part(family, pspec, weights) for slot, (family, pspec) in ls.parts.items()}
        return part_class("block", ls.block)(**parts)

    def all_parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts.values()
        yield self.final_norm
        yield self.head

    def graph_safe(self) -> bool:
        """True if every part allows its forward() to be captured into a CUDA graph."""
        return all(getattr(p, "graph_safe", True) for p in self.all_parts())

    def cache_needs(self) -> Dict[int, object]:
        """cache index -> what the layer that writes it needs from the cache manager."""
        needs: Dict[int, object] = {}
        for call in self.spec.schedule:
            need = self.blocks[call.layer].cache_need()
            if call.write_cache:
                needs[call.cache] = need
            elif needs.get(call.cache) != need:
                raise ValueError(f"layer {call.layer} reads cache {call.cache}, whose writer has another layout")
        return needs

    def forward(self, step, cache_views: Mapping[int, object]) -> torch.Tensor:
        h = self.embedding.forward(step)                                           # float32 [T, hidden]
        for call in self.spec.schedule:
            h = self.blocks[call.layer].forward(h, step, cache_views[call.cache], call.write_cache)
        if step.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        normed = self.final_norm.forward(h, rows=step.want_rows)                  # [wanted, hidden]
        return self.head.forward(normed)                                           # float32 [wanted, vocab]

    def weight_bytes(self) -> int:
        """Bytes of every distinct parameter tensor on the device (a decode step reads each once)."""
        seen, total = set(), 0

        def visit(obj, depth=0):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.is_cuda and obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, Linear):
                visit(obj.weight), visit(obj.bias)
            elif isinstance(obj, Part) and depth < 3:
                for k, v in vars(obj).items():
                    if k not in ("rt", "spec") and not k.startswith("_"):
                        visit(v, depth + 1)
        for p in self.all_parts():
            visit(p)
        return total
