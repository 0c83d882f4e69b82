"""Half-split rotary position encoding.

inv_freq[j] = 1 / theta^(2j / head_dim) in float32, angle = float32(pos) * inv_freq[j] (a float32
product), and element j of a head is rotated together with element j + head_dim/2:
x1' = x1*cos - x2*sin, x2' = x2*cos + x1*sin (src/forward.cpp:52-95).  As in the reference
(kernels/batch_gpu.cu:122-127) the tables are built on the host in float32 and uploaded, so the host's
plain implementation and the device rotate by identical angles.
"""
from __future__ import annotations

import torch

from ..config.specs import PartSpec
from .base import PositionEncoding, register_position


def rotary_tables(head_dim: int, theta: float, n_positions: int):
    """(cos, sin), float32 [n_positions, head_dim/2], on the CPU."""
    half = head_dim // 2
    exponent = torch.arange(0, half, dtype=torch.float32) * 2.0 / float(head_dim)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    angle = torch.arange(n_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(angle), torch.sin(angle)


@register_position("rotary_half")
class RotaryHalf(PositionEncoding):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.head_dim, self.theta = int(spec["head_dim"]), float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.head_dim % 2 or self.head_dim <= 0:
            raise ValueError(f"rotary_half needs an even head_dim, got {self.head_dim}")
        if self.theta <= 0:
            raise ValueError("rotary_half needs a positive theta")
        self._tables = {}

    def rotary_tables(self, n_positions: int = None):
        """Tables for positions [0, n_positions) on the device; cached per length."""
        n = min(self.max_positions, n_positions or self.max_positions)
        cache_key = (self.head_dim, self.theta, n, str(self.rt.device))
        t = _SHARED_TABLES.get(cache_key)
        if t is None:
            cos, sin = rotary_tables(self.head_dim, self.theta, n)
            t = (cos.to(self.rt.device).contiguous(), sin.to(self.rt.device).contiguous())
            _SHARED_TABLES[cache_key] = t
        return t

    def apply(self, q, k, positions):
        raise NotImplementedError("rotary_half is applied by the attention part's rotate-and-store kernel")


# Layers of one model share their tables (same head size, theta and length).
_SHARED_TABLES = {}
