"""Python face of the CUDA kernels: checks arguments, passes raw pointers, raises on failure.

There is no other implementation behind these functions.  If the library cannot be built or
loaded, or a tensor is not on a CUDA device, the call raises; nothing falls back to the CPU or to
a library's model code.
"""
from __future__ import annotations

import collections
import ctypes
from typing import Optional

import torch

from .csrc.build import load_module

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 storage, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The raw handle of torch's current stream on the current device (asked of torch's C layer directly: the Python
    wrapper costs several microseconds, which counts when a step launches two hundred kernels)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _check(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_SIGS = {}


def _fn(module: str, name: str, argtypes, defines=None, restype=c_int):
    key = (module, name, tuple(sorted(defines.items())) if defines else None)
    f = _SIGS.get(key)
    if f is None:
        lib = load_module(module, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = restype
        f._lib = lib
        _SIGS[key] = f
    return f


_LAUNCHES = [0]
# How often each kind of launch was made from the host (a replayed CUDA graph does not pass here): tests read it to
# assert that the kernel they mean to cover is the one that ran. Launchers add kinds of their own with ``note``.
LAUNCH_KINDS = collections.Counter()


def note(kind: str) -> None:
    LAUNCH_KINDS[kind] += 1


def kernel_launches() -> int:
    """How many launcher calls of this package's own kernels have been made in this process."""
    return _LAUNCHES[0]


def _call(f, *args) -> None:
    _LAUNCHES[0] += 1
    LAUNCH_KINDS[f.__name__] += 1
    rc = f(*args)
    if rc != 0:
        msg = f._lib.ib_last_error()
        raise KernelError(f"{f.__name__} failed ({rc}): {msg.decode() if msg else 'no message'}")


# ----------------------------------------------------------------------------- plain kernels

def embedding(table: torch.Tensor, ids: torch.Tensor, status: Optional[torch.Tensor] = None,
              feedback: Optional[torch.Tensor] = None, token_seg: Optional[torch.Tensor] = None,
              seg_slot: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """float32 rows of ``table`` ([vocab, hidden], float32 or bfloat16) for int32 ``ids``, times ``scale``. An id of
    -1 is replaced by ``feedback[seg_slot[token_seg[t]]]``: the token the sampler left on the device for that request."""
    _check(table, "table")
    _check(ids, "ids", torch.int32)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    if feedback is not None:
        _check(feedback, "feedback", torch.int32)
        _check(token_seg, "token_seg", torch.int32, (T,))
        _check(seg_slot, "seg_slot", torch.int32)
    f = _fn("plain", "ib_embedding", [c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64] + [c_void_p] * 5 + [c_float, c_void_p])
    _call(f, table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), T, H, V, out.data_ptr(), _ptr(status),
          _ptr(feedback), _ptr(token_seg), _ptr(seg_slot), float(scale), _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows; ``rows`` (int32) selects and orders the input rows."""
    _check(x, "x", torch.float32)
    H = x.shape[-1]
    _check(weight, "weight", torch.float32, (H,))
    if rows is not None:
        _check(rows, "rows", torch.int32)
    n = rows.numel() if rows is not None else x.numel() // H
    out = torch.empty((n, H), dtype=out_dtype, device=x.device)
    f = _fn("plain", "ib_rmsnorm", [c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, x.data_ptr(), weight.data_ptr(), float(eps), n, H, _ptr(rows), out.data_ptr(), dtype_code(out_dtype), _stream())
    return out


def linear_plain(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x @ w.T (+ bias) (+ residual) with float accumulation in ascending k."""
    _check(x, "x")
    _check(w, "w", x.dtype)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x is [{M},{K}] but w is {tuple(w.shape)}")
    out_dtype = out_dtype or (out.dtype if out is not None else x.dtype)
    if bias is not None:
        _check(bias, "bias", torch.float32, (N,))
    if residual is not None:
        _check(residual, "residual", torch.float32, (M, N))
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        _check(out, "out", out_dtype, (M, N))
    f = _fn("plain", "ib_linear_plain", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                         c_int, c_int, c_void_p])
    _call(f, x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual), out.data_ptr(), M, N, K,
          dtype_code(x.dtype), dtype_code(out_dtype), _stream())
    return out


def rope_kv_write(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                  positions: torch.Tensor, token_seg: torch.Tensor, block_table: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                  write_cache: bool = True, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotates q and k of packed rows [q|k|v], stores k and v into their pages, returns q [T, heads*head_dim].
    Caches are [pages, kv_heads, page_size, head_dim]."""
    _check(qkv, "qkv")
    T = qkv.shape[0]
    _check(qkv, "qkv", None, (T, (n_heads + 2 * n_kv) * head_dim))
    _check(k_cache, "k_cache", qkv.dtype)
    _check(v_cache, "v_cache", qkv.dtype, k_cache.shape)
    n_pages, ckv, page_size, chd = k_cache.shape
    if ckv != n_kv or chd != head_dim:
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={n_kv}, head_dim={head_dim}")
    _check(positions, "positions", torch.int32, (T,))
    _check(token_seg, "token_seg", torch.int32, (T,))
    _check(block_table, "block_table", torch.int32)
    if cos is not None:
        _check(cos, "cos", torch.float32)
        _check(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != head_dim // 2:
            raise KernelError("rotary tables must be [max_positions, head_dim/2]")
    q = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    f = _fn("plain", "ib_rope_kv_write", [c_void_p] * 6 + [c_int64] + [c_void_p] * 3 + [c_int64] + [c_int] * 5 +
            [c_int64, c_int, c_void_p, c_void_p])
    _call(f, qkv.data_ptr(), _ptr(cos), _ptr(sin), positions.data_ptr(), token_seg.data_ptr(), block_table.data_ptr(),
          block_table.shape[1], q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T, n_heads, n_kv, head_dim,
          page_size, int(write_cache), n_pages, dtype_code(qkv.dtype), _ptr(status), _stream())
    return q


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                    token_seg: torch.Tensor, positions: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                    window: Optional[int], scale: float, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token over its request's pages; returns [T, heads*head_dim]."""
    _check(q, "q")
    T = q.shape[0]
    _check(q, "q", None, (T, n_heads * head_dim))
    _check(k_cache, "k_cache", q.dtype)
    _check(v_cache, "v_cache", q.dtype, k_cache.shape)
    n_pages, ckv, page_size, chd = k_cache.shape
    if ckv != n_kv or chd != head_dim:
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={n_kv}, head_dim={head_dim}")
    _check(positions, "positions", torch.int32, (T,))
    _check(token_seg, "token_seg", torch.int32, (T,))
    _check(block_table, "block_table", torch.int32)
    out = torch.empty_like(q)
    f = _fn("plain", "ib_attention_plain", [c_void_p] * 4 + [c_int64] + [c_void_p] * 3 + [c_int64] + [c_int] * 5 +
            [c_float, c_int64, c_int, c_void_p, c_void_p])
    _call(f, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          token_seg.data_ptr(), positions.data_ptr(), out.data_ptr(), T, n_heads, n_kv, head_dim, page_size,
          int(window or 0), float(scale), n_pages, dtype_code(q.dtype), _ptr(status), _stream())
    return out


def attention_max_head_dim() -> int:
    """The largest head size the attention kernels of this package take."""
    return int(_fn("plain", "ib_attention_plain_max_head_dim", [])())


def swiglu(gate_up: torch.Tensor, interleave8: bool = False) -> torch.Tensor:
    """rows [gate | up] -> silu(gate) * up. With interleave8 the rows are blocks of 8 gate then 8 up features."""
    _check(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("swiglu input rows must hold gate and up halves")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("plain", "ib_swiglu", [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p])
    _call(f, gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, dtype_code(gate_up.dtype), int(interleave8), _stream())
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
           feedback: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token id per row of float32 logits: argmax at temperature 0, else Gumbel-max with a
    hash of (seed, step, index). temperature float32 [B]; seed, step int64 [B]. Returns int32 [B].
    With ``feedback`` (int32 [slots]) and ``slots`` (int64 [B]) each token is also left at feedback[slots[b]]."""
    _check(logits, "logits", torch.float32)
    B, V = logits.shape
    _check(temperature, "temperature", torch.float32, (B,))
    _check(seed, "seed", torch.int64, (B,))
    _check(step, "step", torch.int64, (B,))
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    f = _fn("plain", "ib_sample", [c_void_p, c_int64, c_int64] + [c_void_p] * 7)
    _call(f, logits.data_ptr(), B, V, temperature.data_ptr(), seed.data_ptr(), step.data_ptr(), out.data_ptr(),
          _ptr(feedback), _ptr(slots), _stream())
    return out


def sample_filtered(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
                    top_k: torch.Tensor, top_p: torch.Tensor, feedback: Optional[torch.Tensor] = None,
                    slots: Optional[torch.Tensor] = None) -> torch.Tensor:
    """As ``sample``, after keeping the top_k (int64 [B], 0 = all) largest logits and then the smallest set of
    largest probabilities whose mass reaches top_p (float32 [B], 1 = all)."""
    _check(logits, "logits", torch.float32)
    B, V = logits.shape
    _check(temperature, "temperature", torch.float32, (B,))
    _check(seed, "seed", torch.int64, (B,))
    _check(step, "step", torch.int64, (B,))
    _check(top_k, "top_k", torch.int64, (B,))
    _check(top_p, "top_p", torch.float32, (B,))
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    f = _fn("plain", "ib_sample_filtered", [c_void_p, c_int64, c_int64] + [c_void_p] * 9)
    _call(f, logits.data_ptr(), B, V, temperature.data_ptr(), seed.data_ptr(), step.data_ptr(), top_k.data_ptr(),
          top_p.data_ptr(), out.data_ptr(), _ptr(feedback), _ptr(slots), _stream())
    return out
