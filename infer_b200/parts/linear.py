"""A weight matrix on the device and the choice of kernel that multiplies by it.

``out = x @ W.T (+ bias) (+ residual)``; W is kept [out, in] as checkpoints store it (row-major,
so the reduction dimension is contiguous: the layout both the plain kernel and the tensor-core
kernels want).  The matrix is held in the runtime's compute dtype, the bias in float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..runtime import Runtime


class Linear:
    def __init__(self, rt: Runtime, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.rt = rt
        self.weight = weight.to(device=rt.device, dtype=rt.dtype).contiguous()
        self.bias = None if bias is None else bias.to(device=rt.device, dtype=torch.float32).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.prefetch_next = None      # weights of a product that runs later; decode kernels fetch them into L2

    def __call__(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x [rows, in] in the compute dtype (or a DeferredNorm of float32 rows). With ``residual`` (float32 [rows, out]) the result is
        float32 and is written over ``residual``. Otherwise the result has ``out_dtype`` (default:
        the compute dtype)."""
        from .base import DeferredNorm
        out = residual
        if residual is not None:
            out_dtype = torch.float32
        if self.rt.fast("linear"):
            from .. import fast_ops
            y = fast_ops.linear(x, self.weight, self.bias, residual, out_dtype or self.rt.dtype, out,
                                prefetch=self.prefetch_next)
            if y is not None:
                return y
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        return ops.linear_plain(x, self.weight, self.bias, residual, out_dtype or self.rt.dtype, out)
