"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w; eps inside the root, added after the mean; no mean
subtraction, no bias, the weight multiplies as it is (src/forward.cpp:21-31, kernels/ops/rmsnorm.cu:9-28)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    # Kernels that take (float32 rows, weight, eps) can apply this norm themselves: the streaming product of a
    # decode step normalises its lanes' fragments of the rows in registers, once per CTA, which saves the norm
    # kernel and its round trip through memory.
    fusable = True

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.size, self.eps = int(spec["size"]), float(spec["eps"])
        if self.size <= 0 or self.eps <= 0:
            raise ValueError("rmsnorm needs a positive size and eps")
        self.weight = None

    @classmethod
    def param_shapes(cls, spec):
        return {"weight": (int(spec["size"]),)}

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)

    def load(self, params):
        self.weight = params["weight"].to(device=self.rt.device, dtype=torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype or self.rt.dtype, rows)
