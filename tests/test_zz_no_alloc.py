"""The entry point that allocates nothing (infer_b200/csrc/gemm_static.h), called through its exported C symbol the
way a caller without an allocator would: raw device pointers in, nothing created on the way. Its result must equal
the regular entry point's, twice in a row (the second call meets the scratch that the first one left behind).

Who needs it: code that has handed every byte of device memory out at start-up, or that runs inside a latency-critical
loop where cudaMalloc's device-wide synchronisation is not acceptable, and so cannot provide split-K scratch per call.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_fn():
    from infer_b200.csrc.build import load_module
    lib = load_module("gemm")
    f = lib.ib_gemm_tc_static
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 3 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return lib, f


# shapes whose plan cuts K into slices (they use the built-in scratch) and one that does not
@pytest.mark.parametrize("M,N,K", [(8, 1536, 1536), (64, 1536, 8960), (40, 300, 2048), (300, 512, 1536), (1024, 2048, 256)])
def test_static_entry_point_matches_the_regular_one(M, N, K):
    from infer_b200 import fast_ops
    lib, f = _static_fn()
    st = fast_ops.device_state(DEV)
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    res = torch.randn(M, N, device=DEV, generator=g)
    want = fast_ops.gemm_tc(x, w, bias, res.clone(), torch.float32)
    cond = x.float().abs() @ w.float().abs().T + 1.0
    stream = torch.cuda.current_stream().cuda_stream
    before = torch.cuda.memory_allocated()
    for call in range(2):
        out = res.clone()                       # the residual is added in place, as the engine does
        base = torch.cuda.memory_allocated()
        rc = f(x.data_ptr(), w.data_ptr(), bias.data_ptr(), out.data_ptr(), out.data_ptr(), M, N, K, 0, st.sm_count,
               st.status.data_ptr(), stream)
        assert rc == 0, lib.ib_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == base, "the call allocated through torch"
        assert st.status.item() == 0
        assert ((out - want).abs() / cond).max().item() < 2e-6, f"call {call}"
    del out
    assert torch.cuda.memory_allocated() <= before + res.numel() * 4


def test_static_entry_point_refuses_what_does_not_fit():
    lib, f = _static_fn()
    from infer_b200 import fast_ops
    st = fast_ops.device_state(DEV)
    # a GPU reported as huge against few tiles: 12 tiles x 16 slices x 128 x 128 floats = 12.6 MB through the workspace
    # (products of up to 128 rows, and larger ones whose slices fill the GPU in clusters of 2, 4 or 8, need no scratch
    # at all: their slices meet in the cluster's shared memory)
    M, N, K = 256, 768, 16384
    plan = fast_ops.gemm_plan(M, N, K, 1000)
    assert plan[2] > 1 and plan[3] * 4 > (8 << 20) - 16384
    x = torch.zeros(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(M, N, device=DEV)
    rc = f(x.data_ptr(), w.data_ptr(), None, None, out.data_ptr(), M, N, K, 0, 1000, st.status.data_ptr(),
           torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"built-in array" in lib.ib_last_error()
