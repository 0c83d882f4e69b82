"""The chain kernel (several skinny products with grid barriers in one cooperative launch) against the plain kernels,
phase by phase: a chain of p phases is run for p = 1..4 and the output of its last phase is compared with the plain
kernels applied to what the chain's own earlier phases produced (the kernel is deterministic, so a shorter chain
yields exactly the intermediates of a longer one)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# (hidden, attention width, intermediate, q/k/v width)
SIZES = [
    (1536, 1536, 8960, 2048),     # the serving model's layer
    (328, 264, 1000, 456),        # nothing a power of two; K tails in every phase; ragged tiles
    (96, 64, 48, 80),             # smaller than one stage
    (1280, 4096, 4608, 1024),     # several stages of K, with and without a tail
]


def _layer(H, A, I, Q, M, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    rnd = lambda *s, scale=1.0: torch.randn(*s, device=DEV, generator=g) * scale
    wg, wu = rnd(I, H, scale=0.08).bfloat16(), rnd(I, H, scale=0.08).bfloat16()
    pad = (-I) % 8
    return dict(
        ctx=rnd(M, A).bfloat16(), h=rnd(M, H, scale=2.0),
        wo=rnd(H, A, scale=0.05).bfloat16(), g2=1 + 0.1 * rnd(H), eps2=1e-5,
        wg=wg, wu=wu, wd=rnd(H, I, scale=0.05).bfloat16(),
        g1=1 + 0.1 * rnd(H), eps1=3e-6, wqkv=rnd(Q, H, scale=0.05).bfloat16(), bqkv=rnd(Q),
        w_il=torch.stack([wg.view(I // 8, 8, H), wu.view(I // 8, 8, H)], 1).reshape(2 * I, H).contiguous() if not pad else None,
    )


def _run(L, M, n_phases):
    from infer_b200 import fast_ops as F
    H, I, Q = L["wo"].shape[0], L["wd"].shape[1], L["wqkv"].shape[0]
    h = L["h"].clone()
    act = torch.full((M, I), 7.0, dtype=torch.bfloat16, device=DEV)
    qkv = torch.full((M, Q), 7.0, dtype=torch.bfloat16, device=DEV)
    phases = [
        F.chain_phase(L["wo"], L["ctx"], h, F.CHAIN_EPI_RESIDUAL),
        F.chain_phase(L["w_il"], h, act, F.CHAIN_EPI_SWIGLU, norm_weight=L["g2"], eps=L["eps2"]),
        F.chain_phase(L["wd"], act, h, F.CHAIN_EPI_RESIDUAL),
        F.chain_phase(L["wqkv"], h, qkv, F.CHAIN_EPI_STORE, bias=L["bqkv"], norm_weight=L["g1"], eps=L["eps1"]),
    ][:n_phases]
    assert all(p is not None for p in phases)
    F.linear_chain(phases, M, DEV)
    torch.cuda.synchronize()
    assert F.device_state(DEV).status.item() == 0
    return h, act, qkv


@pytest.mark.parametrize("M", [1, 3, 8, 11, 16])
@pytest.mark.parametrize("H,A,I,Q", SIZES)
def test_chain_matches_plain_kernels_phase_by_phase(H, A, I, Q, M):
    from infer_b200 import ops
    L = _layer(H, A, I, Q, M, seed=H + M)
    cond = lambda x, w: x.float().abs() @ w.float().abs().T + 1.0
    # phase 1: o product into the residual stream
    h1, _, _ = _run(L, M, 1)
    ref = ops.linear_plain(L["ctx"], L["wo"], None, L["h"].clone(), torch.float32)
    assert ((h1 - ref).abs() / cond(L["ctx"], L["wo"])).max().item() < 2e-6
    # phase 2: norm, gate/up product, SwiGLU
    h1b, act, _ = _run(L, M, 2)
    assert torch.equal(h1b, h1)
    x2 = ops.rmsnorm(h1, L["g2"], L["eps2"], torch.bfloat16)
    gate = ops.linear_plain(x2, L["wg"], out_dtype=torch.float32)
    up = ops.linear_plain(x2, L["wu"], out_dtype=torch.float32)
    ref = gate / (1 + torch.exp(-gate)) * up
    # the normalised rows may differ from the norm kernel's by one bfloat16 rounding where a value sits on a tie
    assert ((act.float() - ref).abs() <= ref.abs() * 2 ** -7 + 2e-3 * ref.abs().max()).all()
    # phase 3: down product into the residual stream, from the chain's own activations
    h2, act_b, _ = _run(L, M, 3)
    assert torch.equal(act_b, act)
    ref = ops.linear_plain(act, L["wd"], None, h1.clone(), torch.float32)
    assert ((h2 - ref).abs() / cond(act, L["wd"])).max().item() < 2e-6
    # phase 4: the next norm and the q/k/v product with bias
    h2b, _, qkv = _run(L, M, 4)
    assert torch.equal(h2b, h2)
    x3 = ops.rmsnorm(h2, L["g1"], L["eps1"], torch.bfloat16)
    ref = ops.linear_plain(x3, L["wqkv"], L["bqkv"], None, torch.float32)
    c = cond(x3, L["wqkv"])
    assert ((qkv.float() - ref).abs() <= ref.abs() * 2 ** -8 + 2e-4 * c).all()


def test_chain_rows_do_not_depend_on_the_batch():
    """A token's results are the same bits alone and among 8 or 16 rows (tile heights and grids differ)."""
    H, A, I, Q = 328, 264, 1000, 456
    L16 = _layer(H, A, I, Q, 16, seed=5)
    full = _run(L16, 16, 4)
    for M in (1, 8):
        Lm = dict(L16, ctx=L16["ctx"][:M].contiguous(), h=L16["h"][:M].contiguous())
        part = _run(Lm, M, 4)
        for a, b in zip(part, full):
            assert torch.equal(a, b[:M])


def test_chain_repeats_and_graph_capture():
    """Launch after launch leaves the barrier words ready for the next; a captured launch replays to the same bits."""
    from infer_b200 import fast_ops as F
    L = _layer(1536, 1536, 8960, 2048, 8, seed=11)
    first = _run(L, 8, 4)
    for _ in range(20):
        again = _run(L, 8, 4)
    for a, b in zip(first, again):
        assert torch.equal(a, b)
    st = F.device_state(DEV)
    assert st.grid_barrier[0].item() == 0 and st.grid_barrier[2].item() == 0
    h = L["h"].clone()
    act = torch.empty((8, 8960), dtype=torch.bfloat16, device=DEV)
    qkv = torch.empty((8, 2048), dtype=torch.bfloat16, device=DEV)
    phases = [
        F.chain_phase(L["wo"], L["ctx"], h, F.CHAIN_EPI_RESIDUAL),
        F.chain_phase(L["w_il"], h, act, F.CHAIN_EPI_SWIGLU, norm_weight=L["g2"], eps=L["eps2"]),
        F.chain_phase(L["wd"], act, h, F.CHAIN_EPI_RESIDUAL),
        F.chain_phase(L["wqkv"], h, qkv, F.CHAIN_EPI_STORE, bias=L["bqkv"], norm_weight=L["g1"], eps=L["eps1"]),
    ]
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        F.linear_chain(phases, 8, DEV)
        s.synchronize()
        h.copy_(L["h"])
        with torch.cuda.graph(graph, stream=s):
            F.linear_chain(phases, 8, DEV)
        for _ in range(3):
            h.copy_(L["h"])
            graph.replay()
        s.synchronize()
    assert torch.equal(h, first[0]) and torch.equal(qkv, first[2])
    assert st.status.item() == 0


def test_chain_refuses_what_it_cannot_do():
    from infer_b200 import fast_ops as F
    from infer_b200.ops import KernelError
    x = torch.zeros(4, 72, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(40, 72, dtype=torch.bfloat16, device=DEV)
    assert F.chain_phase(w, x, torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV), F.CHAIN_EPI_SWIGLU) is None   # N % 16
    x5 = torch.zeros(4, 44, dtype=torch.bfloat16, device=DEV)
    assert F.chain_phase(torch.zeros(8, 44, dtype=torch.bfloat16, device=DEV), x5,
                         torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV), F.CHAIN_EPI_STORE) is None          # K % 8
    big = torch.zeros(2, 1544, device=DEV)
    assert F.chain_phase(torch.zeros(8, 1544, dtype=torch.bfloat16, device=DEV), big,
                         torch.zeros(2, 8, dtype=torch.bfloat16, device=DEV), F.CHAIN_EPI_STORE,
                         norm_weight=torch.ones(1544, device=DEV)) is None                                       # a norm over more than one stage
    ok = F.chain_phase(w, x, torch.zeros(4, 40, dtype=torch.bfloat16, device=DEV), F.CHAIN_EPI_STORE)
    with pytest.raises(KernelError):
        F.linear_chain([ok] * 5, 4, DEV)
    with pytest.raises(KernelError):
        F.linear_chain([ok], 17, DEV)
