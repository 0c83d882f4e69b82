"""The fast kernels of the bfloat16 serving path (sm_100a): each function returns its result, or None
when the kernel does not take the shape, in which case the caller uses the plain kernel."""
from __future__ import annotations


def linear(x, weight, bias, residual, out_dtype, out):
    return None


def rope_kv_write(qkv, cos, sin, step, table, cache, n_heads, n_kv, head_dim, write_cache):
    return None


def attention(q, cache, table, step, n_heads, n_kv, head_dim, window, scale):
    return None


def gate_up_swiglu(x, gate_up):
    return None
