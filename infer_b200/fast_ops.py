"""The fast kernels of the bfloat16 serving path (sm_100a): each function returns its result, or None
when the kernel does not take the shape, in which case the caller uses the plain kernel.

Kernels that need scratch memory (split-K partial tiles, flash-decoding partial results) share one
workspace per device, allocated once and grown on demand; calls on one stream run in order, so they
may share it.  One status word per device collects failures that kernels report (a page index out of
range, a bounded wait that ran out).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from . import ops
from .ops import KernelError, _call, _check, _fn, _ptr, _stream, c_float, c_int, c_int64, c_void_p, dtype_code


class DeviceState:
    """Per-device scratch shared by the fast kernels."""

    def __init__(self, device: torch.device):
        self.device = device
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self._workspace = torch.empty(0, dtype=torch.float32, device=device)
        self._counters = torch.zeros(4096, dtype=torch.int32, device=device)

    def workspace(self, n_floats: int) -> torch.Tensor:
        if self._workspace.numel() < n_floats:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("the kernel workspace must be sized before a CUDA graph is captured")
            self._workspace = torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=self.device)
        return self._workspace

    def counters(self, n: int) -> torch.Tensor:
        if self._counters.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("the kernel counters must be sized before a CUDA graph is captured")
            self._counters = torch.zeros(max(n, 4096), dtype=torch.int32, device=self.device)
        return self._counters


_STATES: Dict[torch.device, DeviceState] = {}


def device_state(device) -> DeviceState:
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    st = _STATES.get(device)
    if st is None:
        st = _STATES[device] = DeviceState(device)
    return st


# ----------------------------------------------------------------------------- tensor-core GEMM

_PLAN_CACHE: Dict[tuple, Optional[tuple]] = {}


def gemm_plan(M: int, N: int, K: int, sm_count: int):
    """(swap, bn, splits, workspace floats, counters) for a product, or None if the kernel refuses the sizes."""
    key = (M, N, K, sm_count)
    if key not in _PLAN_CACHE:
        f = _fn("gemm", "ib_gemm_tc_plan", [c_int64, c_int64, c_int64, c_int] + [c_void_p] * 5)
        swap, bn, splits = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        ws, nc = ctypes.c_int64(), ctypes.c_int64()
        rc = f(M, N, K, sm_count, ctypes.byref(swap), ctypes.byref(bn), ctypes.byref(splits), ctypes.byref(ws), ctypes.byref(nc))
        _PLAN_CACHE[key] = None if rc != 0 else (swap.value, bn.value, splits.value, ws.value, nc.value)
    return _PLAN_CACHE[key]


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
            out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None, plan=None) -> Optional[torch.Tensor]:
    """out = x @ w.T (+ bias) (+ residual) on the tcgen05 tensor cores; None if the sizes are refused.
    x [M, K], w [N, K] bfloat16; bias float32 [N]; residual float32 [M, N] (may be `out`)."""
    _check(x, "x", torch.bfloat16)
    _check(w, "w", torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: x is [{M},{K}] but w is {tuple(w.shape)}")
    st = device_state(x.device)
    plan = plan or gemm_plan(M, N, K, st.sm_count)
    if plan is None or (x.data_ptr() & 15) or (w.data_ptr() & 15):
        return None
    swap, bn, splits, ws_floats, n_counters = plan
    if bias is not None:
        _check(bias, "bias", torch.float32, (N,))
    if residual is not None:
        _check(residual, "residual", torch.float32, (M, N))
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        _check(out, "out", out_dtype, (M, N))
    ws = st.workspace(ws_floats) if splits > 1 else None
    cnt = st.counters(n_counters) if splits > 1 else None
    f = _fn("gemm", "ib_gemm_tc", [c_void_p] * 5 + [c_int64] * 3 + [c_int] * 4 + [c_void_p] * 4)
    _call(f, x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual), out.data_ptr(), M, N, K, dtype_code(out_dtype),
          swap, bn, splits, _ptr(ws), _ptr(cnt), st.status.data_ptr(), _stream())
    return out


def linear(x, weight, bias, residual, out_dtype, out):
    if x.dtype != torch.bfloat16:
        return None
    return gemm_tc(x, weight, bias, residual, out_dtype, out)


def rope_kv_write(qkv, cos, sin, step, table, cache, n_heads, n_kv, head_dim, write_cache):
    return None


def attention(q, cache, table, step, n_heads, n_kv, head_dim, window, scale):
    return None


def gate_up_swiglu(x, gate_up):
    return None
