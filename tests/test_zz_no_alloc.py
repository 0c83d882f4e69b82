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


# Shapes whose K slices are summed through global memory: these are the ones that read and write the built-in array
# (the plan states how many floats). Both calls are compared with a float64 product, so a wrong address, size or
# counter offset shows; the second call meets the partial tiles and counters that the first one left.
SCRATCH_SHAPES = [(300, 300, 1536), (200, 136, 4096), (300, 256, 1024)]
# Shapes that need none of it: up to 128 rows and clusters of slices meet in shared memory, large ones are not cut.
OTHER_SHAPES = [(8, 1536, 1536), (64, 1536, 8960), (40, 300, 2048), (300, 512, 1536), (1024, 2048, 256)]


def _inputs(M, N, K):
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    res = torch.randn(M, N, device=DEV, generator=g)
    return x, w, bias, res


def _call_static(lib, f, st, x, w, bias, out):
    M, K = x.shape
    base = torch.cuda.memory_allocated()
    rc = f(x.data_ptr(), w.data_ptr(), bias.data_ptr(), out.data_ptr(), out.data_ptr(), M, w.shape[0], K, 0, st.sm_count,
           st.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ib_last_error().decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == base, "the call allocated through torch"
    assert st.status.item() == 0


@pytest.mark.parametrize("M,N,K", SCRATCH_SHAPES)
def test_static_entry_point_sums_its_slices_in_the_built_in_array(M, N, K):
    from infer_b200 import fast_ops
    lib, f = _static_fn()
    st = fast_ops.device_state(DEV)
    plan = fast_ops.gemm_plan(M, N, K, st.sm_count)
    assert plan is not None and plan[2] > 1 and plan[3] > 0, f"this shape no longer reaches the scratch array: plan {plan}"
    assert plan[3] * 4 <= (8 << 20) - 16384
    x, w, bias, res = _inputs(M, N, K)
    exact = x.double() @ w.double().T + bias.double() + res.double()
    cond = x.float().abs() @ w.float().abs().T + 1.0
    regular = fast_ops.gemm_tc(x, w, bias, res.clone(), torch.float32)
    for call in range(2):
        out = res.clone()                       # the residual is added in place, as the engine does
        _call_static(lib, f, st, x, w, bias, out)
        assert ((out.double() - exact).abs() / cond).max().item() < 2e-6, f"call {call} against float64"
        assert ((out - regular).abs() / cond).max().item() < 2e-6, f"call {call} against the regular entry point"


@pytest.mark.parametrize("M,N,K", OTHER_SHAPES)
def test_static_entry_point_matches_the_regular_one(M, N, K):
    from infer_b200 import fast_ops
    lib, f = _static_fn()
    st = fast_ops.device_state(DEV)
    plan = fast_ops.gemm_plan(M, N, K, st.sm_count)
    assert plan is not None and plan[3] == 0
    x, w, bias, res = _inputs(M, N, K)
    want = fast_ops.gemm_tc(x, w, bias, res.clone(), torch.float32)
    for call in range(2):
        out = res.clone()
        _call_static(lib, f, st, x, w, bias, out)
        # without a workspace both entry points add the slices in the same fixed order: the same bits
        assert torch.equal(out, want), f"call {call}"


def test_static_entry_point_refuses_what_does_not_fit():
    lib, f = _static_fn()
    from infer_b200 import fast_ops
    st = fast_ops.device_state(DEV)
    # a GPU reported as huge against few tiles: 12 tiles x 16 slices x 128 x 128 floats = 12.6 MB through the workspace
    M, N, K = 256, 768, 16384
    plan = fast_ops.gemm_plan(M, N, K, 1000)
    assert plan[2] > 1 and plan[3] * 4 > (8 << 20) - 16384
    x = torch.zeros(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(M, N, device=DEV)
    rc = f(x.data_ptr(), w.data_ptr(), None, None, out.data_ptr(), M, N, K, 0, 1000, st.status.data_ptr(),
           torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"built-in array" in lib.ib_last_error()
