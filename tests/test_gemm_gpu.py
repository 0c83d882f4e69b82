"""The tcgen05 matrix product alone against the plain kernel (same bfloat16 inputs, float accumulation), at sizes
that the engine's tests do not use: both tile mappings, K tails, ragged M and N, bias, residual, split-K."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = [
    # (M, N, K)            mapping / what is special
    (1, 128, 64),          # swap, one k-block
    (1, 1536, 1536),       # swap, decode of one token
    (8, 2048, 1536),       # swap, bn 16, split-K
    (17, 300, 520),        # swap, bn 32, ragged N, K tail (520 = 8*64 + 8)
    (64, 1536, 8960),      # swap, bn 64, long K, split-K
    (5, 301, 80),          # swap, odd N (scalar stores), K < 128
    (65, 96, 224),         # swap, bn 128, one ragged tile each way, K tail
    (128, 128, 128),       # swap, bn 128, exact tiles
    (100, 1536, 8960),     # swap, bn 128, long K in 8 slices that push 16 columns each to their owners
    (128, 2048, 1536),     # swap, bn 128, three k-blocks per slice
    (129, 128, 128),       # plain, the first size beyond the swapped mapping
    (200, 300, 4096),      # plain, 6 tiles: 16 slices of K through the workspace, summed by the CTA that arrives last
    (256, 1536, 8960),     # plain, 24 tiles: 4 slices of K as a cluster
    (400, 2048, 1536),     # plain, 64 tiles: 2 slices of K as a cluster, three-stage ring wraps
    (300, 1000, 1536),     # plain, ragged M and N
    (2048, 2048, 1536),    # plain, prefill-sized
    (130, 301, 96),        # plain, odd N
    (2, 320, 96),          # swap, K = 1.5 k-blocks
    (1100, 3000, 520),     # persistent (128 x 256 tiles, two accumulators): ragged M and N, K tail, several tiles per CTA
    (4000, 4100, 72),      # persistent, many tiles of two k-blocks: the accumulators alternate quickly
    (1800, 1500, 136),     # persistent with 128 x 176 tiles (they fill the SMs better than 256 columns), ragged M and N
    (2048, 1536, 1536),    # persistent with 128 x 176 tiles, the model's o product at prefill
]


def _ref(x, w, bias, residual):
    from infer_b200 import ops
    return ops.linear_plain(x, w, bias, residual.clone() if residual is not None else None, torch.float32)


@pytest.mark.parametrize("M,N,K", SIZES)
def test_gemm_tc_matches_plain(M, N, K):
    from infer_b200 import fast_ops
    g = torch.Generator(device=DEV).manual_seed(M * 7 + N * 3 + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    res = torch.randn(M, N, device=DEV, generator=g)
    cond = x.float().abs() @ w.float().abs().T + 1.0
    st = fast_ops.device_state(DEV)
    st.status.zero_()
    for b, r in ((None, None), (bias, None), (bias, res)):
        ref = _ref(x, w, b, r)
        got = fast_ops.gemm_tc(x, w, b, r.clone() if r is not None else None, torch.float32)
        assert got is not None, "the kernel refused sizes it documents as supported"
        assert st.status.item() == 0
        err = ((got - ref).abs() / cond).max().item()
        assert err < 2e-6, f"float output differs: {err:.3e} of the conditioning"
    low = fast_ops.gemm_tc(x, w, bias, None, torch.bfloat16)
    assert low.dtype == torch.bfloat16
    ref16 = _ref(x, w, bias, None)
    assert ((low.float() - ref16).abs() <= ref16.abs() * 2 ** -8 + 1e-6 * cond).all()
    # in place over the residual, as the engine calls it
    r2 = res.clone()
    same = fast_ops.gemm_tc(x, w, None, r2, torch.float32, out=r2)
    assert same.data_ptr() == r2.data_ptr()
    assert ((r2 - _ref(x, w, None, res)).abs() / cond).max().item() < 2e-6
    assert st.status.item() == 0


def test_gemm_tc_repeated_calls_share_the_workspace():
    """Split-K counters must be back at zero after every call."""
    from infer_b200 import fast_ops
    x = torch.randn(8, 1536, device=DEV).bfloat16()
    w = (torch.randn(1536, 1536, device=DEV) * 0.05).bfloat16()
    plan = fast_ops.gemm_plan(8, 1536, 1536, fast_ops.device_state(DEV).sm_count)
    assert plan[0] == 1 and plan[2] > 1
    first = fast_ops.gemm_tc(x, w, out_dtype=torch.float32)
    for _ in range(5):
        assert torch.equal(fast_ops.gemm_tc(x, w, out_dtype=torch.float32), first)     # the same bits every time
    assert int(fast_ops.device_state(DEV)._counters.abs().sum()) == 0


def test_gemm_tc_split_choices_agree():
    from infer_b200 import fast_ops
    x = torch.randn(16, 2048, device=DEV).bfloat16()
    w = (torch.randn(512, 2048, device=DEV) * 0.05).bfloat16()
    ref = _ref(x, w, None, None)
    cond = x.float().abs() @ w.float().abs().T + 1.0
    for splits in (1, 2, 5, 16):
        plan = (1, 16, splits, splits * 4 * 128 * 16, 4)
        got = fast_ops.gemm_tc(x, w, out_dtype=torch.float32, plan=plan)
        assert ((got - ref).abs() / cond).max().item() < 2e-6, splits


@pytest.mark.parametrize("code", [256, 352, 384, 512])
@pytest.mark.parametrize("M,N,K", [(2048, 1536, 1536), (1100, 3000, 520), (300, 260, 72)])
def test_gemm_tc_wide_tiles(M, N, K, code):
    """The persistent kernel's tiles chosen by hand: 256 x 128 (plan code 256, two MMAs per k-step) and 128 rows by 176,
    192 and 256 columns (codes 352, 384, 512: one MMA): exact and ragged tiles, a K tail, fewer tiles than SMs; bias, residual in place, SwiGLU."""
    from infer_b200 import fast_ops
    g = torch.Generator(device=DEV).manual_seed(M + N + K + code)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    res = torch.randn(M, N, device=DEV, generator=g)
    cond = x.float().abs() @ w.float().abs().T + 1.0
    st = fast_ops.device_state(DEV)
    st.status.zero_()
    plan = (0, code, 1, 0, 0)
    got = fast_ops.gemm_tc(x, w, bias, None, torch.float32, plan=plan)
    assert ((got - _ref(x, w, bias, None)).abs() / cond).max().item() < 2e-6
    r2 = res.clone()
    fast_ops.gemm_tc(x, w, None, r2, torch.float32, out=r2, plan=plan)
    assert ((r2 - _ref(x, w, None, res)).abs() / cond).max().item() < 2e-6
    if N % 16 == 0:
        act = fast_ops.gemm_tc(x, w, out_dtype=torch.bfloat16, plan=plan, swiglu=True)
        same = fast_ops.gemm_tc(x, w, out_dtype=torch.bfloat16, plan=(0, 128, 1, 0, 0), swiglu=True)
        assert torch.equal(act, same)
    assert st.status.item() == 0


@pytest.mark.parametrize("M,N,K,slices", [(512, 3584, 4736, 2), (540, 1000, 2056, 4), (130, 520, 8192, 8), (300, 256, 1024, 2)])
def test_gemm_tc_wide_tiles_with_k_slices(M, N, K, slices):
    """128 x 256 tiles whose K slices are the CTAs of a cluster and exchange their columns through the operand rings
    (plan code 768): ragged M and N, a K tail, 2, 4 and 8 slices; bias, residual in place, SwiGLU; against float64."""
    from infer_b200 import fast_ops
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    res = torch.randn(M, N, device=DEV, generator=g)
    ref = x.double() @ w.double().T
    cond = x.float().abs() @ w.float().abs().T + 1.0
    st = fast_ops.device_state(DEV)
    st.status.zero_()
    plan = (0, 768, slices, 0, 0)
    got = fast_ops.gemm_tc(x, w, bias, None, torch.float32, plan=plan)
    assert ((got.double() - (ref + bias.double())).abs() / cond).max().item() < 2e-6
    r2 = res.clone()
    fast_ops.gemm_tc(x, w, None, r2, torch.float32, out=r2, plan=plan)
    assert ((r2.double() - (ref + res.double())).abs() / cond).max().item() < 2e-6
    if N % 16 == 0:
        act = fast_ops.gemm_tc(x, w, out_dtype=torch.bfloat16, plan=plan, swiglu=True)
        same = fast_ops.gemm_tc(x, w, out_dtype=torch.bfloat16, plan=(0, 128, 1, 0, 0), swiglu=True)
        assert (act.float() - same.float()).abs().max().item() <= 2.0 ** -6 * same.float().abs().max().item()
    assert st.status.item() == 0


def test_gemm_tc_refuses_what_it_cannot_do():
    from infer_b200 import fast_ops
    x = torch.randn(4, 100, device=DEV).bfloat16()            # K = 100 is not a multiple of 8
    w = torch.randn(32, 100, device=DEV).bfloat16()
    assert fast_ops.gemm_tc(x, w) is None


SKINNY = [(1, 1536, 1536), (8, 2048, 1536), (8, 1536, 8960), (3, 300, 520), (16, 96, 224), (9, 301, 80), (5, 17, 8),
          (2, 320, 96), (1, 151936, 64)]


@pytest.mark.parametrize("M,N,K", SKINNY)
def test_skinny_matches_plain(M, N, K):
    from infer_b200 import fast_ops
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    res = torch.randn(M, N, device=DEV, generator=g)
    cond = x.float().abs() @ w.float().abs().T + 1.0
    for b, r in ((None, None), (bias, None), (bias, res), (None, res)):
        ref = _ref(x, w, b, r)
        got = fast_ops.linear_skinny(x, w, b, r.clone() if r is not None else None, torch.float32)
        assert got is not None
        assert ((got - ref).abs() / cond).max().item() < 2e-6
    low = fast_ops.linear_skinny(x, w, bias, None, torch.bfloat16)
    ref16 = _ref(x, w, bias, None)
    assert ((low.float() - ref16).abs() <= ref16.abs() * 2 ** -8 + 1e-6 * cond).all()
    r2 = res.clone()
    fast_ops.linear_skinny(x, w, None, r2, out=r2)
    assert ((r2 - _ref(x, w, None, res)).abs() / cond).max().item() < 2e-6
    # rows of the result do not depend on how many rows there are
    one = fast_ops.linear_skinny(x[:1].contiguous(), w, bias, None, torch.float32)
    assert torch.equal(one, fast_ops.linear_skinny(x, w, bias, None, torch.float32)[:1])


@pytest.mark.parametrize("M", [1, 8, 13, 40, 64, 100, 128, 200, 1500])
@pytest.mark.parametrize("I,H", [(8960, 1536), (224, 96), (176, 80)])
def test_fused_swiglu_matches_the_two_kernels(M, I, H):
    """gate/up product with the SwiGLU epilogue (rows interleaved in blocks of 8) against plain product + plain SwiGLU,
    through all three kernels: streaming (M <= 16), tcgen05 swapped (M <= 128), tcgen05 plain."""
    from infer_b200 import fast_ops, ops
    g = torch.Generator(device=DEV).manual_seed(M + I)
    x = torch.randn(M, H, device=DEV, generator=g).bfloat16()
    wg = (torch.randn(I, H, device=DEV, generator=g) * 0.1).bfloat16()
    wu = (torch.randn(I, H, device=DEV, generator=g) * 0.1).bfloat16()
    w_il = torch.stack([wg.view(I // 8, 8, H), wu.view(I // 8, 8, H)], 1).reshape(2 * I, H).contiguous()
    gate = ops.linear_plain(x, wg, out_dtype=torch.float32)
    up = ops.linear_plain(x, wu, out_dtype=torch.float32)
    ref = gate / (1 + torch.exp(-gate)) * up
    two = ops.swiglu(ops.linear_plain(x, w_il), interleave8=True)                       # plain kernels, interleaved rows
    assert (two.float() - ref).abs().max() < 0.05 * ref.abs().max() + 1e-3
    for fn in ([fast_ops.linear_skinny] if M <= 16 else []) + [fast_ops.gemm_tc]:
        got = fn(x, w_il, out_dtype=torch.bfloat16, swiglu=True)
        assert got is not None and got.shape == (M, I)
        assert ((got.float() - ref).abs() <= ref.abs() * 2 ** -7 + 1e-4 * ref.abs().max()).all(), fn.__name__
    assert fast_ops.device_state(DEV).status.item() == 0


@pytest.mark.parametrize("M", [1, 8, 11, 16])
@pytest.mark.parametrize("N,K", [(2048, 1536), (96, 64), (301, 80), (448, 96)])
def test_skinny_with_fused_norm(M, N, K):
    """The streaming kernel normalising the float32 rows itself against norm kernel + plain product."""
    from infer_b200 import fast_ops, ops
    g = torch.Generator(device=DEV).manual_seed(M * N + K)
    h = torch.randn(M, K, device=DEV, generator=g) * 3
    nw = 1 + 0.1 * torch.randn(K, device=DEV, generator=g)
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    x = ops.rmsnorm(h, nw, 1e-5, torch.bfloat16)
    ref = ops.linear_plain(x, w, bias, None, torch.float32)
    got = fast_ops.linear_skinny(h, w, bias, None, torch.float32, norm_weight=nw, norm_eps=1e-5)
    assert got is not None
    cond = x.float().abs() @ w.float().abs().T + 1.0
    # the normalised rows may differ from the norm kernel's by one bfloat16 rounding where a value sits on a tie
    assert ((got - ref).abs() / cond).max().item() < 2e-4
    if N % 16 == 0:
        act = fast_ops.linear_skinny(h, w, None, None, torch.bfloat16, swiglu=True, norm_weight=nw, norm_eps=1e-5)
        two = ops.swiglu(ops.linear_plain(x, w), interleave8=True)
        assert (act.float() - two.float()).abs().max() <= 0.03 * two.float().abs().max() + 1e-3


@pytest.mark.parametrize("M,N,K", [(2048, 1536, 8960), (2048, 17920, 1536), (1100, 3000, 520), (100, 1536, 8960), (300, 1000, 1536)])
def test_gemm_tc_against_float64(M, N, K):
    """The tensor-core product against torch in float64, directly (not through the plain kernel): the persistent
    kernel at the model's down and gate/up shapes of a 2,048-token prompt and at a ragged shape, the swapped mapping
    and the one-tile mapping once each. Bias, and the residual added in place."""
    from infer_b200 import fast_ops
    g = torch.Generator(device=DEV).manual_seed(M + 3 * N + 5 * K)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV, generator=g)
    res = torch.randn(M, N, device=DEV, generator=g)
    plan = fast_ops.gemm_plan(M, N, K, fast_ops.device_state(DEV).sm_count)
    if M >= 1024:
        assert plan[1] >= 256, f"this shape is meant to take the persistent kernel, the plan is {plan}"
    exact = x.double() @ w.double().T
    cond = (x.float().abs() @ w.float().abs().T + 1.0).double()
    got = fast_ops.gemm_tc(x, w, bias, None, torch.float32)
    assert ((got.double() - (exact + bias.double())).abs() / cond).max().item() < 2e-6
    r2 = res.clone()
    fast_ops.gemm_tc(x, w, None, r2, torch.float32, out=r2)
    assert ((r2.double() - (exact + res.double())).abs() / cond).max().item() < 2e-6
    assert fast_ops.device_state(DEV).status.item() == 0
