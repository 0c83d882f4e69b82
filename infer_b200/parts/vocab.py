"""The two ends of a model: the token table (ids -> rows of the residual stream) and the output matrix
(normalised rows -> logits).

h[t, :] = float32(table[ids[t], :]), optionally times a constant ``scale`` (src/forward.cpp:181-187 has none);
logits = x . W^T without bias, W being the head's own matrix or, when tied, the token table itself
(src/forward.cpp:246-257, src/model.h:52). An architecture whose ends do more (a soft cap on the logits, a bias)
registers its own ``Embedding`` / ``Head`` kinds; the model only calls ``forward``.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Embedding, Head, register_embedding, register_head
from .linear import Linear


@register_embedding("token_table")
class TokenTable(Embedding):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        if self.vocab <= 0 or self.hidden <= 0:
            raise ValueError("token_table needs a positive vocab_size and hidden_size")
        scale = spec.get("scale")
        self.scale = 1.0 if scale is None else float(scale)
        self.weight = None

    @classmethod
    def param_shapes(cls, spec):
        return {"weight": (int(spec["vocab_size"]), int(spec["hidden_size"]))}

    def load(self, params):
        # The table is read row by row; it keeps the compute dtype of the matrices (a tied head multiplies by it).
        self.weight = params["weight"].to(device=self.rt.device, dtype=self.rt.dtype).contiguous()

    def table(self):
        return self.weight

    def forward(self, step):
        return ops.embedding(self.weight, step.token_ids, step.status, getattr(step, "feedback", None),
                             step.token_seg, step.seg_slot, self.scale)


@register_head("linear_head")
class LinearHead(Head):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.tied = bool(spec.get("tied", False))
        self.linear = None

    @classmethod
    def param_shapes(cls, spec):
        return {} if spec.get("tied", False) else {"weight": (int(spec["vocab_size"]), int(spec["hidden_size"]))}

    def load(self, params):
        if not self.tied:
            self.linear = Linear(self.rt, params["weight"])

    def tie(self, embedding):
        if not self.tied:
            return
        table = embedding.table()
        if table is None or tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError("a tied head needs an embedding part with a [vocab, hidden] table")
        self.linear = Linear.share(self.rt, table)

    def forward(self, x):
        return self.linear(x, out_dtype=torch.float32)
