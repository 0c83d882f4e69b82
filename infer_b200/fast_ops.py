"""The fast kernels of the bfloat16 serving path (sm_100a): each function returns its result, or None
when the kernel does not take the shape, in which case the caller uses the plain kernel.

Kernels that need scratch memory (split-K partial tiles, flash-decoding partial results) share one
workspace per device, allocated once and grown on demand; calls on one stream run in order, so they
may share it.  One status word per device collects failures that kernels report (a page index out of
range, a bounded wait that ran out).
"""
from __future__ import annotations

import ctypes
import os
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
        self._retired = []

    def workspace(self, n_floats: int) -> torch.Tensor:
        if self._workspace.numel() < n_floats:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("the kernel workspace must be sized before a CUDA graph is captured")
            self._retired.append(self._workspace)        # captured graphs may still point at it
            self._workspace = torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=self.device)
        return self._workspace

    def counters(self, n: int) -> torch.Tensor:
        if self._counters.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("the kernel counters must be sized before a CUDA graph is captured")
            self._retired.append(self._counters)
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
            out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None, plan=None,
            swiglu: bool = False) -> Optional[torch.Tensor]:
    """out = x @ w.T (+ bias) (+ residual) on the tcgen05 tensor cores; None if the sizes are refused.
    x [M, K], w [N, K] bfloat16; bias float32 [N]; residual float32 [M, N] (may be `out`). With ``swiglu`` the
    rows of w are gate/up features interleaved in blocks of 8 and the result is silu(gate) * up, [M, N/2]."""
    _check(x, "x", torch.bfloat16)
    _check(w, "w", torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: x is [{M},{K}] but w is {tuple(w.shape)}")
    st = device_state(x.device)
    plan = plan or gemm_plan(M, N, K, st.sm_count)
    if plan is None or (x.data_ptr() & 15) or (w.data_ptr() & 15) or (swiglu and N % 16):
        return None
    swap, bn, splits, ws_floats, n_counters = plan
    if bias is not None:
        _check(bias, "bias", torch.float32, (N,))
    if residual is not None:
        _check(residual, "residual", torch.float32, (M, N))
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    else:
        _check(out, "out", out_dtype, (M, n_out))
    # split-K of the swapped mapping goes through the cluster's shared memory and needs neither
    ws = st.workspace(ws_floats) if splits > 1 and ws_floats > 0 else None
    cnt = st.counters(n_counters) if splits > 1 and ws_floats > 0 else None
    f = _fn("gemm", "ib_gemm_tc", [c_void_p] * 5 + [c_int64] * 3 + [c_int] * 5 + [c_void_p] * 4)
    _call(f, x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual), out.data_ptr(), M, N, K, dtype_code(out_dtype),
          2 if swiglu else 0, swap, bn, splits, _ptr(ws), _ptr(cnt), st.status.data_ptr(), _stream())
    ops.note("gemm_tc:sliced_wide" if bn == 768 else "gemm_tc:persistent" if bn >= 256 else ("gemm_tc:swapped" if swap else "gemm_tc:one_tile"))
    return out


_SKINNY_LIMITS = None


def skinny_limits():
    """(most rows, longest row the fused norm takes) of the streaming kernel, as its library states them."""
    global _SKINNY_LIMITS
    if _SKINNY_LIMITS is None:
        f = _fn("gemvb", "ib_linear_skinny_bulk_limits", [c_void_p, c_void_p])
        rows, k = ctypes.c_int(), ctypes.c_int()
        f(ctypes.byref(rows), ctypes.byref(k))
        _SKINNY_LIMITS = (rows.value, k.value)
    return _SKINNY_LIMITS


def linear_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
                  out: Optional[torch.Tensor] = None, swiglu: bool = False, cluster: int = 0,
                  norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 0.0) -> Optional[torch.Tensor]:
    """The decode kernel: x [M <= 16, K] against w [N, K], weights streamed once; same epilogues as gemm_tc.
    With ``norm_weight`` x is the float32 residual stream and is RMS-normalised inside the kernel (rows up to
    ``skinny_limits()[1]`` long).
    cluster: CTAs sharing one tile's K range (0 = chosen by the kernel)."""
    fused = norm_weight is not None
    _check(x, "x", torch.float32 if fused else torch.bfloat16)
    _check(w, "w", torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear_skinny: x is [{M},{K}] but w is {tuple(w.shape)}")
    max_rows, max_norm_k = skinny_limits()
    if M > max_rows or K % 8 or (x.data_ptr() & 15) or (w.data_ptr() & 15) or (swiglu and N % 16):
        return None
    if fused:
        _check(norm_weight, "norm_weight", torch.float32, (K,))
        if K > max_norm_k or (norm_weight.data_ptr() & 15):
            return None
    if bias is not None:
        _check(bias, "bias", torch.float32, (N,))
    if residual is not None:
        _check(residual, "residual", torch.float32, (M, N))
        out_dtype = torch.float32
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    else:
        _check(out, "out", out_dtype, (M, n_out))
    st = device_state(x.device)
    epi = 2 if swiglu else (1 if residual is not None else 0)
    f = _fn("gemvb", "ib_linear_skinny_bulk", [c_void_p, c_void_p, c_float] + [c_void_p] * 4 + [c_int64] * 3 + [c_int] * 4 +
            [c_void_p] * 2 + [c_int64, c_void_p])
    _call(f, x.data_ptr(), _ptr(norm_weight), float(norm_eps), w.data_ptr(), _ptr(bias), _ptr(residual), out.data_ptr(),
          M, N, K, dtype_code(out_dtype), epi, int(cluster), st.sm_count, st.status.data_ptr(), None, 0, _stream())
    return out


def linear(x, weight, bias, residual, out_dtype, out, swiglu=False):
    """The bfloat16 matrix product of the serving path: the streaming kernel for up to 16 rows, the tcgen05 kernel
    above that; None if neither takes the shape. x may be a DeferredNorm (the float32 residual stream plus the norm
    that is still to be applied): the streaming kernel then normalises inside, anything else materialises it."""
    from .parts.base import DeferredNorm
    if isinstance(x, DeferredNorm):
        if weight.dtype == torch.bfloat16 and x.h.shape[0] <= skinny_limits()[0]:
            y = linear_skinny(x.h, weight, bias, residual, out_dtype, out, swiglu, 0, x.norm.weight, x.norm.eps)
            if y is not None:
                return y
        x = x.materialize()
    if x.dtype != torch.bfloat16:
        return None
    if x.shape[0] <= skinny_limits()[0]:
        y = linear_skinny(x, weight, bias, residual, out_dtype, out, swiglu)
        if y is not None:
            return y
    return gemm_tc(x, weight, bias, residual, out_dtype, out, swiglu=swiglu)


def attention_supported(n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 128 and page_size == 16 and n_heads // n_kv <= 16


ATTENTION_MAX_CLUSTERS = 32       # clusters of 8 slices per (segment, kv head), for long contexts at small batches
ATTENTION_CLUSTER_PAGES = 16      # pages a slice keeps at least when a (segment, kv head) gets several clusters
ATTENTION_CLUSTER_FROM = 96       # ... which it gets when one cluster's slices would each walk at least this many pages


def _decode_splits(st, n_decode: int, n_kv: int, visible: int):
    """(slices per cluster, clusters per (segment, kv head)). Slices: a power of two up to 8, enough CTAs for about
    one per SM, and at least 8 pages (two per warp) in a slice. Clusters: more than one only for long contexts (the
    second level costs about 5 us per layer: measured at batch 8 it loses at 8,192 tokens, 1.56 against 1.44 ms per
    step, and wins at 30,000, 2.50 against 2.78; at batch 1 and 30,000 tokens 1.41 against 2.21), then as many as keep
    16 pages (four per warp) in a slice, up to two CTAs per SM."""
    units = max(1, n_decode * n_kv)
    pages = max(1, -(-visible // 16))
    n = 1
    # (with nearly a CTA per SM already, two slices do not pay for their merge: 25.1 against 26.2 us at batch 64)
    while n < 8 and units * n < st.sm_count and pages // (2 * n) >= 8 and not (n == 1 and 6 * units >= 5 * st.sm_count):
        n *= 2
    clusters = 1
    if n == 8 and pages >= 8 * ATTENTION_CLUSTER_FROM:
        clusters = max(1, min(pages // (8 * ATTENTION_CLUSTER_PAGES), (2 * st.sm_count) // (units * 8), ATTENTION_MAX_CLUSTERS))
    return n, clusters


def _decode_scratch(st, n_segments: int, n_kv: int, head_dim: int, clusters: int):
    """Workspace and counters for several clusters per (segment, kv head); (None, None) for one."""
    if clusters <= 1:
        return None, None
    return st.workspace(n_segments * n_kv * clusters * (16 * head_dim + 32)), st.counters(n_segments * n_kv)


# The prefill kernel on tcgen05 / tensor memory (attention_tc.cu) serves head sizes 64 and 128; INFER_B200_ATTN_TC=0
# leaves prefill to the mma.sync kernel.
ATTENTION_TC = os.environ.get("INFER_B200_ATTN_TC", "1") == "1"
ATTENTION_TC_HEAD_DIMS = (64, 128)
# Sharing a query tile's keys among CTAs (INFER_B200_ATTN_TC_SPLIT=1 switches it off): the kernel's limits.
ATTENTION_TC_MAX_SPLIT = int(os.environ.get("INFER_B200_ATTN_TC_SPLIT", "4"))
ATTENTION_TC_PART_MIN_TILES = 4


def prefill_split(sm_count: int, n_heads: int, n_prefill: int, max_q_len: int, max_ctx_len: int, window: Optional[int]) -> int:
    """Into how many parts the tcgen05 prefill kernel may cut the keys of a query tile. One CTA serves 128 queries of a
    head and walks over their keys in tiles of 128; it has an SM to itself, and starting and finishing a CTA costs
    about as much as three key tiles. So keys are shared only while all CTAs still run at once (a portion behind a
    long context on few heads: 48 CTAs of 36 key tiles become 144 of 12); with more CTAs than SMs the extra starts
    cost more than the evening-out gains (measured at 2,048 tokens on 12 heads: 38.5 us whole, 42 us shared)."""
    if n_prefill <= 0 or max_q_len <= 1:
        return 1
    ctx0 = max_ctx_len - max_q_len
    key_tiles = []
    for q_first in range(ctx0, max_ctx_len, 128):
        q_last = min(max_ctx_len - 1, q_first + 127)
        lo = max(0, q_first - window + 1) if window else 0
        key_tiles.append(q_last // 128 - lo // 128 + 1)
    if max(key_tiles) < 2 * ATTENTION_TC_PART_MIN_TILES:
        return 1
    for split in range(ATTENTION_TC_MAX_SPLIT, 1, -1):
        ctas = n_heads * n_prefill * sum(max(1, min(split, n // ATTENTION_TC_PART_MIN_TILES)) for n in key_tiles)
        if ctas <= sm_count:
            return split
    return 1


def attention_fast(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                   seg_start: torch.Tensor, seg_pos0: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                   window: Optional[int], scale: float, has_decode: bool, max_q_len: int, max_ctx_len: int,
                   n_decode: Optional[int] = None, n_splits: Optional[int] = None, n_clusters: int = 1,
                   tc_split: Optional[int] = None) -> Optional[torch.Tensor]:
    """Tensor-core attention of a step's segments over the paged bfloat16 cache; None if the shape is refused.
    The library is compiled for this head size at first use."""
    n_pages, ckv, page_size, chd = k_cache.shape
    if q.dtype != torch.bfloat16 or not attention_supported(n_heads, n_kv, head_dim, page_size):
        return None
    _check(q, "q", torch.bfloat16)
    T = q.shape[0]
    _check(q, "q", None, (T, n_heads * head_dim))
    _check(k_cache, "k_cache", torch.bfloat16)
    _check(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
    if ckv != n_kv or chd != head_dim:
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={n_kv}, head_dim={head_dim}")
    S = seg_pos0.numel()
    _check(seg_start, "seg_start", torch.int32, (S + 1,))
    _check(seg_pos0, "seg_pos0", torch.int32, (S,))
    _check(block_table, "block_table", torch.int32)
    st = device_state(q.device)
    if n_splits is None:
        visible = min(max_ctx_len, window) if window else max_ctx_len
        n_splits, n_clusters = _decode_splits(st, n_decode if n_decode is not None else S, n_kv, visible) if has_decode else (1, 1)
    ws, cnt = _decode_scratch(st, S, n_kv, head_dim, n_clusters)
    out = torch.empty_like(q)
    # Segments of two or more tokens go to the tcgen05 kernel where it takes the head size; one-token segments, and
    # everything else, to the mma.sync kernels (a call with max_q_len = 1 launches no prefill kernel).
    tc = ATTENTION_TC and max_q_len > 1 and head_dim in ATTENTION_TC_HEAD_DIMS and page_size == 16
    if tc:
        g = _fn("attn_tc", "ib_attention_prefill_tc", [c_void_p] * 5 + [c_int] + [c_void_p] * 2 + [c_int, c_int64] + [c_int] * 5 +
                [c_float, c_int64, c_int] + [c_void_p] * 2 + [c_int, c_void_p, c_int64, c_void_p, c_int64, c_int], {"IB_HEAD_DIM": head_dim})
        n_prefill = S - (n_decode or 0)
        split = prefill_split(st.sm_count, n_heads, n_prefill, max_q_len, max_ctx_len, window) if tc_split is None else tc_split
        tc_ws = tc_cnt = None
        if split > 1:
            tiles = max(1, n_prefill) * n_heads * -(-max_q_len // 128)
            tc_ws, tc_cnt = st.workspace(tiles * split * (128 * head_dim + 256)), st.counters(tiles)
            ops.note("attention_prefill_tc:shared_query_tiles")
        _call(g, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], seg_start.data_ptr(), seg_pos0.data_ptr(), S, T, n_heads, n_kv, head_dim, page_size,
              int(window or 0), float(scale), n_pages, int(max_q_len), st.status.data_ptr(), _stream(), int(split),
              _ptr(tc_ws), 0 if tc_ws is None else tc_ws.numel(), _ptr(tc_cnt), 0 if tc_cnt is None else tc_cnt.numel(),
              int(n_prefill) if n_decode is not None else 0)
        if max_q_len > 128:
            ops.note("attention_prefill_tc:several_query_tiles")
        if not has_decode:
            return out
    f = _fn("attn", "ib_attention_fast", [c_void_p] * 5 + [c_int] + [c_void_p] * 2 + [c_int] * 6 + [c_float, c_int64] +
            [c_int] * 3 + [c_void_p] * 2 + [c_int] + [c_void_p] * 2, {"IB_HEAD_DIM": head_dim})
    _call(f, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), block_table.data_ptr(),
          block_table.shape[1], seg_start.data_ptr(), seg_pos0.data_ptr(), S, n_heads, n_kv, head_dim, page_size,
          int(window or 0), float(scale), n_pages, int(has_decode), 1 if tc else int(max_q_len), int(n_splits),
          st.status.data_ptr(), _stream(), int(n_clusters), _ptr(ws), _ptr(cnt))
    return out


def decode_fused_supported(n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    return attention_supported(n_heads, n_kv, head_dim, page_size) and head_dim % 32 == 0


def attention_decode_fused(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, block_table: torch.Tensor, seg_start: torch.Tensor,
                           seg_pos0: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, window: Optional[int],
                           scale: float, max_ctx_len: int, write_cache: bool = True,
                           n_splits: Optional[int] = None, n_clusters: int = 1) -> Optional[torch.Tensor]:
    """Decode-only steps: rotation of q and k, the cache write of the new positions and attention in ONE kernel.
    qkv [S, (heads + 2 kv) * head_dim] packed rows with the bias added. Returns [S, heads * head_dim]."""
    n_pages, ckv, page_size, chd = k_cache.shape
    if qkv.dtype != torch.bfloat16 or not decode_fused_supported(n_heads, n_kv, head_dim, page_size):
        return None
    S = seg_pos0.numel()
    _check(qkv, "qkv", torch.bfloat16, (S, (n_heads + 2 * n_kv) * head_dim))
    _check(k_cache, "k_cache", torch.bfloat16)
    _check(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
    if ckv != n_kv or chd != head_dim:
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={n_kv}, head_dim={head_dim}")
    _check(cos, "cos", torch.float32)
    _check(sin, "sin", torch.float32, cos.shape)
    if cos.shape[1] != head_dim // 2:
        raise KernelError("rotary tables must be [max_positions, head_dim/2]")
    _check(seg_start, "seg_start", torch.int32, (S + 1,))
    _check(seg_pos0, "seg_pos0", torch.int32, (S,))
    _check(block_table, "block_table", torch.int32)
    st = device_state(qkv.device)
    if n_splits is None:
        visible = min(max_ctx_len, window) if window else max_ctx_len
        n_splits, n_clusters = _decode_splits(st, S, n_kv, visible)
    ws, cnt = _decode_scratch(st, S, n_kv, head_dim, n_clusters)
    out = torch.empty((S, n_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    f = _fn("attn", "ib_attention_decode_fused", [c_void_p] * 7 + [c_int] + [c_void_p] * 2 + [c_int] * 6 + [c_float, c_int64] +
            [c_int] * 2 + [c_void_p] * 2 + [c_int64, c_void_p] + [c_int] + [c_void_p] * 2, {"IB_HEAD_DIM": head_dim})
    _call(f, qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], seg_start.data_ptr(), seg_pos0.data_ptr(), S, n_heads, n_kv,
          head_dim, page_size, int(window or 0), float(scale), n_pages, int(write_cache), int(n_splits),
          st.status.data_ptr(), None, 0, _stream(), int(n_clusters), _ptr(ws), _ptr(cnt))
    return out


def attention(q, cache, table, step, n_heads, n_kv, head_dim, window, scale):
    n_decode = sum(1 for n in step.seg_lens if n == 1)
    return attention_fast(q, cache.k, cache.v, table, step.seg_start, step.seg_pos0, n_heads, n_kv, head_dim, window,
                          scale, n_decode > 0, step.max_q_len, step.max_ctx_len, n_decode)


def gate_up_swiglu(x, gate_up_weight):
    """silu(x Wg^T) * (x Wu^T) in one kernel; gate_up_weight rows interleaved in blocks of 8."""
    return linear(x, gate_up_weight, None, None, torch.bfloat16, None, swiglu=True)
