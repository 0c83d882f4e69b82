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

    @classmethod
    def share(cls, rt: Runtime, weight: torch.Tensor) -> "Linear":
        """A product by a matrix that already lies on the device in the compute dtype (no copy is made)."""
        if weight.device != rt.device or weight.dtype != rt.dtype or not weight.is_contiguous():
            raise ValueError("a shared matrix must lie on the device, contiguous, in the compute dtype")
        self = cls.__new__(cls)
        self.rt, self.weight, self.bias = rt, weight, None
        self.out_features, self.in_features = weight.shape
        return self

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
            y = fast_ops.linear(x, self.weight, self.bias, residual, out_dtype or self.rt.dtype, out)
            if y is not None:
                return y
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        return ops.linear_plain(x, self.weight, self.bias, residual, out_dtype or self.rt.dtype, out)
