"""SwiGLU feed-forward: out = residual + (silu(x Wg^T) * (x Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g)),
no biases (src/forward.cpp:231-238, kernels/ops/elementwise.cu:6-11). Gate and up are one matrix
product over the concatenated rows [Wg; Wu] (kernels/model_gpu.cu:40-48)."""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import FeedForward, register_feed_forward
from .linear import Linear


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    accepts_deferred_norm = True

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        if self.hidden <= 0 or self.inter <= 0:
            raise ValueError("swiglu needs positive sizes")
        self.gate_up = self.down = None

    @classmethod
    def param_shapes(cls, spec):
        H, I = int(spec["hidden_size"]), int(spec["intermediate_size"])
        return {"gate_proj.weight": (I, H), "up_proj.weight": (I, H), "down_proj.weight": (H, I)}

    def load(self, params):
        g, u = params["gate_proj.weight"], params["up_proj.weight"]
        # For the fused kernels, gate and up rows alternate in blocks of 8, so that one thread (or two lanes of a
        # warp) holds a gate value and its up value.
        self.interleaved = self.rt.dtype == torch.bfloat16 and self.inter % 8 == 0
        if self.interleaved:
            w = torch.stack([g.reshape(self.inter // 8, 8, self.hidden), u.reshape(self.inter // 8, 8, self.hidden)], dim=1)
            w = w.reshape(2 * self.inter, self.hidden)
        else:
            w = torch.cat([g, u], dim=0)
        self.gate_up = Linear(self.rt, w)
        self.down = Linear(self.rt, params["down_proj.weight"])

    def forward(self, x, residual):
        act = None
        if self.interleaved and self.rt.fast("swiglu") and self.rt.fast("linear"):
            from .. import fast_ops
            act = fast_ops.gate_up_swiglu(x, self.gate_up.weight)
        if act is None:
            act = ops.swiglu(self.gate_up(x), self.interleaved)      # Linear materialises a deferred norm
        return self.down(act, residual=residual)
