"""Grouped-query causal attention over the paged cache.

q = x Wq^T + bq, k = x Wk^T + bk, v = x Wv^T + bv (one matrix product over the concatenated rows
[Wq; Wk; Wv], as the reference lays them out on the device, kernels/model_gpu.cu:31-34); positions are
encoded into q and k; k and v go to the request's pages; query head h reads kv head h / (heads /
kv_heads); score = (q . k) * scale with scale = 1/sqrt(head_dim) unless given; keys j <= p, and
j > p - window if the layer has a window; softmax in float32; out = residual + ctx Wo^T
(src/forward.cpp:101-136,208-224; kernels/ops/batch.cu:207-316).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Mixer, PagedKVNeed, build_part, register_mixer
from .linear import Linear


@register_mixer("attention")
class Attention(Mixer):
    accepts_deferred_norm = True

    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads, self.n_kv, self.head_dim = int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"])
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.window = spec.get("window")
        if self.window is not None:
            self.window = int(self.window)
            if self.window <= 0:
                raise ValueError("an attention window must be positive (or None for all keys)")
        if self.n_kv <= 0 or self.n_heads % self.n_kv:
            raise ValueError(f"heads ({self.n_heads}) must be a multiple of kv heads ({self.n_kv})")
        if self.head_dim <= 0 or self.head_dim % 2:
            raise ValueError(f"head_dim must be positive and even, got {self.head_dim}")
        if self.head_dim > ops.attention_max_head_dim():
            raise ValueError(f"head_dim {self.head_dim} is beyond what the attention kernels take ({ops.attention_max_head_dim()})")
        scale = spec.get("softmax_scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(self.head_dim))
        pos = spec.get("position")
        self.position = build_part("position", pos, runtime) if pos is not None else None
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    @classmethod
    def param_shapes(cls, spec):
        H, nh, nkv, hd = int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"])
        shapes = {"q_proj.weight": (nh * hd, H), "k_proj.weight": (nkv * hd, H), "v_proj.weight": (nkv * hd, H),
                  "o_proj.weight": (H, nh * hd)}
        if spec.get("qkv_bias", False):
            shapes.update({"q_proj.bias": (nh * hd,), "k_proj.bias": (nkv * hd,), "v_proj.bias": (nkv * hd,)})
        return shapes

    def load(self, params):
        w = torch.cat([params["q_proj.weight"], params["k_proj.weight"], params["v_proj.weight"]], dim=0)
        b = None
        if self.qkv_bias:
            b = torch.cat([params["q_proj.bias"].float(), params["k_proj.bias"].float(), params["v_proj.bias"].float()])
        self.qkv = Linear(self.rt, w, b)
        self.o = Linear(self.rt, params["o_proj.weight"])

    def cache_need(self):
        return PagedKVNeed(self.n_kv, self.head_dim, self.window)

    def forward(self, x, step, cache, residual, write_cache=True):
        qkv = self.qkv(x)                                              # [T, (heads + 2 kv) * head_dim]
        table = step.block_tables[cache.group]
        tables = self.position.rotary_tables(self.rt.max_seq_len) if self.position is not None else None
        if self.position is not None and tables is None:
            T = qkv.shape[0]
            q_view = qkv[:, : self.n_heads * self.head_dim].view(T, self.n_heads, self.head_dim)
            k_view = qkv[:, self.n_heads * self.head_dim: (self.n_heads + self.n_kv) * self.head_dim].view(T, self.n_kv, self.head_dim)
            self.position.apply(q_view, k_view, step.positions)
        cos, sin = tables if tables is not None else (None, None)
        if step.decode_only and cos is not None and self.rt.fast("rope") and self.rt.fast("attention"):
            # one token per request: rotation, cache write and attention in one kernel
            from .. import fast_ops
            ctx = fast_ops.attention_decode_fused(qkv, cos, sin, cache.k, cache.v, table, step.seg_start, step.seg_pos0,
                                                  self.n_heads, self.n_kv, self.head_dim, self.window, self.scale,
                                                  step.max_ctx_len, write_cache)
            if ctx is not None:
                return self.o(ctx, residual=residual)
        q = ops.rope_kv_write(qkv, cos, sin, step.positions, step.token_seg, table, cache.k, cache.v,
                              self.n_heads, self.n_kv, self.head_dim, write_cache, step.status)
        ctx = None
        if self.rt.fast("attention"):
            from .. import fast_ops
            ctx = fast_ops.attention(q, cache, table, step, self.n_heads, self.n_kv, self.head_dim, self.window, self.scale)
        if ctx is None:
            ctx = ops.attention_plain(q, cache.k, cache.v, table, step.token_seg, step.positions,
                                      self.n_heads, self.n_kv, self.head_dim, self.window, self.scale, step.status)
        return self.o(ctx, residual=residual)
