"""The plain implementation: the architecture written out slowly, for whole sequences, without a cache.

One function per part, each from the reference engine's formula (cited per function, paths within
RyanXiaoo/infer).  It shares no code with ``infer_b200``: it reads the raw config.json dictionary and a
dictionary of checkpoint tensors, and computes with torch on the CPU in float64 (``dtype`` below), except
where the reference fixes float32 arithmetic that matters (rotation angles).  tests/golden/ holds logits of
the reference's own C++ forward (src/forward.cpp, compiled on the CPU) on a tiny random model; this file is
compared with them in test_plain_model.py, and everything else is compared with this file.

``rounding``: None computes exactly.  ``torch.bfloat16`` rounds activations to bfloat16 at the places
where a bfloat16 serving path stores them (normalised rows, q/k/v, rotated q/k, attention output, gate/up
and activation), which gives the size of the rounding noise that path must have.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Mapping, Optional, Sequence

import numpy as np
import torch

F = torch.float64


def _rnd(x: torch.Tensor, rounding) -> torch.Tensor:
    return x if rounding is None else x.to(rounding).to(x.dtype)


def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """h[t, :] = table[ids[t], :], no scaling; ids outside the table are an error (src/forward.cpp:181-187)."""
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    if ids.numel() and (ids.min() < 0 or ids.max() >= table.shape[0]):
        raise ValueError("token id out of range")
    return table.to(F)[ids]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * w per row; eps inside the root, after the mean; no mean subtraction,
    no bias, weight as it is (src/forward.cpp:21-31)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x / torch.sqrt(ms + eps) * w.to(F)


def linear(x: torch.Tensor, W: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t, o] = sum_i W[o, i] x[t, i] (+ b[o]); W is [out, in] as stored (src/forward.cpp:35-47)."""
    y = x @ W.to(F).T
    return y if b is None else y + b.to(F)


def rope_tables(theta: float, head_dim: int, n_positions: int):
    """inv_freq[j] = 1 / theta^(2j/head_dim) and angle = pos * inv_freq[j], both in float32 as the reference
    computes them; cos/sin of that float32 angle (src/forward.cpp:52-72). Returns [n_positions, head_dim/2]."""
    half = head_dim // 2
    inv_freq = np.float32(1.0) / np.power(np.float32(theta), np.arange(half, dtype=np.float32) * np.float32(2.0) / np.float32(head_dim))
    inv_freq = inv_freq.astype(np.float32)
    angle = (np.arange(n_positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    a = torch.from_numpy(angle.astype(np.float64))
    return torch.cos(a), torch.sin(a)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, heads, head_dim]; element j is rotated with element j + head_dim/2 (half-split, not interleaved):
    x1' = x1 cos - x2 sin, x2' = x2 cos + x1 sin; q and k only, never v (src/forward.cpp:79-95)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None,
              scale: Optional[float] = None) -> torch.Tensor:
    """q [T, heads, hd], k/v [T, kv_heads, hd] -> [T, heads, hd]. Query head h reads kv head h // (heads/kv_heads);
    score = (q . k) * scale, scale = 1/sqrt(hd) applied after the dot; position t sees s <= t (and s > t - window
    when the layer has a window); softmax with the maximum subtracted; out = sum_s p_s v_s
    (src/forward.cpp:101-136). The window is not in the reference, which refuses nothing and ignores the key;
    it follows the architecture's config keys: a layer with a window sees the last `window` positions."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(float(hd)) if scale is None else scale
    out = torch.zeros_like(q)
    for h in range(nh):
        g = h // group
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k[lo:t + 1, g, :] @ q[t, h, :]) * scale
            p = torch.exp(s - s.max())
            p = p / p.sum()
            out[t, h, :] = p @ v[lo:t + 1, g, :]
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)) (src/forward_internal.h:42)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x: torch.Tensor, Wg, Wu, Wd, rounding=None) -> torch.Tensor:
    """(silu(x Wg^T) * (x Wu^T)) Wd^T, no biases (src/forward.cpp:231-238)."""
    g, u = _rnd(linear(x, Wg), rounding), _rnd(linear(x, Wu), rounding)
    return linear(_rnd(silu(g) * u, rounding), Wd)


def layer_window(cfg: Mapping, layer: int) -> Optional[int]:
    """Layers with index >= max_window_layers use sliding_window when use_sliding_window is true."""
    if cfg.get("use_sliding_window", False) and layer >= int(cfg.get("max_window_layers") or 0):
        return int(cfg["sliding_window"])
    return None


def attention_block(cfg: Mapping, W: Mapping[str, torch.Tensor], prefix: str, x: torch.Tensor, cos, sin,
                    window: Optional[int], rounding=None) -> torch.Tensor:
    """q/k/v projections with bias, rotation of q and k, attention, output projection without bias
    (src/forward.cpp:208-224)."""
    T = x.shape[0]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    bias = cfg.get("attention_bias", True)

    def proj(name):
        b = W[prefix + name + ".bias"] if bias else None
        return _rnd(linear(x, W[prefix + name + ".weight"], b), rounding)
    q = proj("q_proj").view(T, nh, hd)
    k = proj("k_proj").view(T, nkv, hd)
    v = proj("v_proj").view(T, nkv, hd)
    q, k = _rnd(apply_rope(q, cos, sin), rounding), _rnd(apply_rope(k, cos, sin), rounding)
    ctx = _rnd(attention(q, k, v, window), rounding).reshape(T, nh * hd)
    return linear(ctx, W[prefix + "o_proj.weight"])


def forward(cfg: Mapping, W: Mapping[str, torch.Tensor], ids: Sequence[int], rounding=None,
            taps: Optional[Dict[str, torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of a whole sequence (src/forward.cpp:170-258):
    h = table[ids]; per layer h += attn(norm(h)), h += mlp(norm(h)); logits = norm(h) head^T, the head being
    lm_head.weight, or the token table when tie_word_embeddings (src/model.h:52)."""
    T = len(ids)
    nh = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg["rms_norm_eps"]
    h = embedding(W["model.embed_tokens.weight"], ids)
    cos, sin = rope_tables(cfg["rope_theta"], hd, T)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        n = _rnd(rmsnorm(h, W[p + "input_layernorm.weight"], eps), rounding)
        h = h + attention_block(cfg, W, p + "self_attn.", n, cos, sin, layer_window(cfg, i), rounding)
        n = _rnd(rmsnorm(h, W[p + "post_attention_layernorm.weight"], eps), rounding)
        h = h + swiglu_mlp(n, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                           W[p + "mlp.down_proj.weight"], rounding)
        if taps is not None:
            taps[f"hidden_state_{i + 1}"] = h.clone()
    n = _rnd(rmsnorm(h, W["model.norm.weight"], eps), rounding)
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else W["lm_head.weight"]
    return linear(n, head)


def greedy(logits_row: torch.Tensor) -> int:
    """First index of the maximum: strict >, so ties go to the lowest id (src/forward.cpp:264-266)."""
    return int(np.argmax(logits_row.numpy()))


def greedy_decode(cfg, W, ids: Sequence[int], n_new: int, rounding=None) -> List[int]:
    """Recompute-style greedy generation (src/forward.cpp:260-271)."""
    ids, out = list(ids), []
    for _ in range(n_new):
        tok = greedy(forward(cfg, W, ids, rounding)[-1])
        out.append(tok)
        ids.append(tok)
    return out


# ---------------------------------------------------------------------------------------------- sampling

_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    """splitmix64 finaliser (kernels/ops/ops.cuh:26-30)."""
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def hash_uniform(seed: int, step: int, v: int) -> np.float32:
    """Uniform in (0,1) from (seed, step, index): two finaliser rounds, top 24 bits, never 0
    (kernels/ops/ops.cuh:31-35)."""
    x = _mix64((seed + 0x9E3779B97F4A7C15 * (step + 1)) & _M64)
    x = _mix64(x ^ ((v + 0x632BE59BD9B4E019) & _M64))
    return np.float32((np.float32((x >> 40) & 0xFFFFFF) + np.float32(0.5)) / np.float32(16777216.0))


def sample(logits_row: np.ndarray, temperature: float, seed: int, step: int) -> int:
    """temperature 0: argmax, ties to the lowest id. Otherwise argmax of logit/T + g, g = -log(-log(u)) with u
    from hash_uniform(seed, step, index): a sample of softmax(logits/T) that depends on nothing but
    (seed, step) (kernels/ops/batch.cu:450-478, kernels/ops/ops.cuh:36-38)."""
    row = np.asarray(logits_row, dtype=np.float32)
    if temperature <= 0:
        return int(np.argmax(row))
    u = np.array([hash_uniform(seed, step, v) for v in range(row.shape[0])], dtype=np.float32)
    g = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
    return int(np.argmax(row / np.float32(temperature) + g))
