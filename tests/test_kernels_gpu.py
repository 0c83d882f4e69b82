"""Each plain kernel alone against a float64 torch formula, at sizes other than the engine tests use."""
import math

import numpy as np
import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from infer_b200 import ops
    return ops


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    ops = _ops()
    table = torch.randn(37, 24).to(dtype).to(DEV)
    ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.embedding(table, ids, status)
    assert out.dtype == torch.float32 and torch.equal(out, table.float()[ids.long()])
    assert status.item() == 0
    bad = torch.tensor([3, 37], dtype=torch.int32, device=DEV)
    out = ops.embedding(table, bad, status)
    assert status.item() == 1 and float(out[1].abs().sum()) == 0.0      # refused, not read out of bounds


@pytest.mark.parametrize("hidden", [1, 33, 96, 1536, 3000, 6148, 8192])
def test_rmsnorm(hidden):
    ops = _ops()
    x = torch.randn(7, hidden, device=DEV) * 3
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    ref = pm.rmsnorm(x.double().cpu(), w.cpu(), 1e-5)
    got = ops.rmsnorm(x, w, 1e-5, torch.float32)
    assert torch.allclose(got.cpu().double(), ref, rtol=2e-6, atol=2e-6)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    sel = ops.rmsnorm(x, w, 1e-5, torch.bfloat16, rows)
    assert sel.dtype == torch.bfloat16 and torch.equal(sel, got[rows.long()].bfloat16())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 127, 31), (65, 64, 33), (130, 70, 896), (2, 301, 80)])
def test_linear_plain(M, N, K, dtype):
    ops = _ops()
    x, w = torch.randn(M, K).to(dtype).to(DEV), torch.randn(N, K).to(dtype).to(DEV)
    b, r = torch.randn(N, device=DEV), torch.randn(M, N, device=DEV)
    ref = x.double() @ w.double().T
    cond = (x.double().abs() @ w.double().abs().T)                      # conditioning of each dot product
    got = ops.linear_plain(x, w, out_dtype=torch.float32)
    assert ((got.double() - ref).abs() / cond.clamp_min(1e-30)).max() < 5e-6   # the reference's GEMV tolerance
    got = ops.linear_plain(x, w, b, r.clone(), torch.float32)
    assert ((got.double() - (ref + b.double() + r.double())).abs() / (cond + 1)).max() < 5e-6
    res = r.clone()
    same = ops.linear_plain(x, w, b, res, out=res)                      # written over the residual
    assert same.data_ptr() == res.data_ptr() and torch.equal(res, got)
    if dtype == torch.bfloat16:
        low = ops.linear_plain(x, w, b)
        assert low.dtype == torch.bfloat16 and torch.equal(low, (ops.linear_plain(x, w, b, out_dtype=torch.float32)).bfloat16())


def test_linear_rows_do_not_depend_on_the_batch():
    ops = _ops()
    x, w = torch.randn(200, 300, device=DEV), torch.randn(77, 300, device=DEV)
    full = ops.linear_plain(x, w)
    for lo, hi in ((0, 1), (63, 66), (199, 200), (5, 150)):
        assert torch.equal(ops.linear_plain(x[lo:hi].contiguous(), w), full[lo:hi])


def _paged_setup(dtype, n_heads, n_kv, hd, page, lens, n_pages, seed=0):
    """Random q/k/v for requests of the given lengths, caches filled through a shuffled block table."""
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    max_blocks = max(-(-n // page) for n in lens) + 1
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((S, max_blocks), -1, dtype=torch.int32)
    k_cache = torch.full((n_pages, n_kv, page, hd), float("nan"))
    v_cache = torch.full((n_pages, n_kv, page, hd), float("nan"))
    ks, vs = [], []
    for s, n in enumerate(lens):
        k, v = torch.randn(n, n_kv, hd, generator=g), torch.randn(n, n_kv, hd, generator=g)
        ks.append(k.to(dtype).float()), vs.append(v.to(dtype).float())
        for b in range(-(-n // page)):
            pg = perm.pop()
            table[s, b] = pg
            m = min(page, n - b * page)
            k_cache[pg, :, :m] = ks[-1][b * page:b * page + m].transpose(0, 1)
            v_cache[pg, :, :m] = vs[-1][b * page:b * page + m].transpose(0, 1)
    return table, k_cache.to(dtype), v_cache.to(dtype), ks, vs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,hd,page,window", [(14, 2, 64, 16, None), (12, 2, 128, 16, None), (4, 4, 8, 4, None),
                                                     (8, 1, 16, 8, 5), (5, 5, 48, 16, 40), (2, 1, 256, 32, None)])
def test_attention_plain(heads, kv, hd, page, window, dtype):
    """Queries at chosen positions of several requests, pages shuffled, unused cache rows NaN."""
    ops = _ops()
    lens = [1, 2, 33, 257, 130]
    table, kc, vc, ks, vs = _paged_setup(dtype, heads, kv, hd, page, lens, n_pages=sum(-(-n // page) for n in lens) + 3)
    toks = [(s, p) for s, n in enumerate(lens) for p in sorted({0, n // 2, n - 1, max(0, n - 2)})]
    g = torch.Generator().manual_seed(1)
    q = torch.randn(len(toks), heads, hd, generator=g).to(dtype)
    scale = 1 / math.sqrt(hd)
    ref = torch.zeros(len(toks), heads, hd, dtype=torch.float64)
    for i, (s, p) in enumerate(toks):
        qq = torch.zeros(p + 1, heads, hd, dtype=torch.float64)
        qq[p] = q[i].double()
        ref[i] = pm.attention(qq, ks[s][:p + 1].double(), vs[s][:p + 1].double(), window, scale)[p]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = ops.attention_plain(q.reshape(len(toks), -1).contiguous().to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV),
                              torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV),
                              torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV),
                              heads, kv, hd, window, scale, status)
    assert status.item() == 0
    err = (got.cpu().double().view_as(ref) - ref).abs().max()
    assert err < (2e-2 if dtype == torch.bfloat16 else 5e-5), err      # reference tolerance 5e-5 (tests/test_ops_gpu.cu:264)


def test_attention_spike_at_a_far_key():
    """One key far back gets nearly all the weight; first, middle and last positions (tests/test_ops_gpu.cu:277-285)."""
    ops = _ops()
    heads = kv = 1
    hd, page, n = 32, 16, 700
    for spike in (0, 351, 699):
        table, kc, vc, ks, vs = _paged_setup(torch.float32, heads, kv, hd, page, [n], n_pages=50, seed=spike)
        q = torch.randn(1, hd)
        pg, off = int(table[0, spike // page]), spike % page
        kc[pg, 0, off] = q[0] * 3.0
        ks[0][spike, 0] = q[0] * 3.0
        out = ops.attention_plain(q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                  torch.tensor([n - 1], dtype=torch.int32, device=DEV), 1, 1, hd, None, 1 / math.sqrt(hd))
        qq = torch.zeros(n, 1, hd, dtype=torch.float64); qq[n - 1] = q.double()
        ref = pm.attention(qq, ks[0].double(), vs[0].double())[n - 1]
        assert (out.cpu().double() - ref.view(1, -1)).abs().max() < 5e-5
        assert (out.cpu() - vs[0][spike].view(1, -1)).abs().max() < 0.2   # the spike's value dominates


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_kv_write(dtype):
    ops = _ops()
    heads, kv, hd, page, n_pages = 3, 2, 24, 8, 9
    from infer_b200.parts.rotary import rotary_tables
    cos, sin = rotary_tables(hd, 12345.0, 64)
    pc, ps = pm.rope_tables(12345.0, hd, 64)
    assert torch.allclose(cos.double(), pc, atol=1e-6) and torch.allclose(sin.double(), ps, atol=1e-6)
    positions = torch.tensor([5, 6, 7, 8, 0, 40], dtype=torch.int32)
    seg = torch.tensor([0, 0, 0, 0, 1, 2], dtype=torch.int32)
    table = torch.tensor([[3, 7, -1, -1, -1, -1], [1, -1, -1, -1, -1, -1], [0, 2, 4, 5, 6, 8]], dtype=torch.int32)
    qkv = torch.randn(6, (heads + 2 * kv) * hd).to(dtype)
    kc = torch.zeros(n_pages, kv, page, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = ops.rope_kv_write(qkv.to(DEV), cos.to(DEV), sin.to(DEV), positions.to(DEV), seg.to(DEV), table.to(DEV), kc, vc,
                          heads, kv, hd, True, status)
    assert status.item() == 0
    x = qkv.double()
    c, s = pc[positions.long()], ps[positions.long()]
    q_ref = pm.apply_rope(x[:, :heads * hd].view(6, heads, hd), c, s)
    k_ref = pm.apply_rope(x[:, heads * hd:(heads + kv) * hd].view(6, kv, hd), c, s)
    v_ref = x[:, (heads + kv) * hd:].view(6, kv, hd)
    tol = _tol(dtype)
    assert torch.allclose(q.cpu().double().view(6, heads, hd), q_ref, **tol)
    for t in range(6):
        pg, off = int(table[seg[t], positions[t] // page]), int(positions[t] % page)
        assert torch.allclose(kc[pg, :, off].cpu().double(), k_ref[t], **tol)
        assert torch.equal(vc[pg, :, off].cpu().double(), v_ref[t])
    assert int((kc != 0).any(-1).sum()) == 6 * kv                       # nothing else was written
    # without the tables nothing is rotated; without write_cache nothing is stored
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    q2 = ops.rope_kv_write(qkv.to(DEV), None, None, positions.to(DEV), seg.to(DEV), table.to(DEV), kc2, vc2, heads, kv, hd, False)
    assert torch.equal(q2.cpu(), qkv[:, :heads * hd]) and float(kc2.abs().sum()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    ops = _ops()
    x = (torch.randn(5, 2 * 37) * 3).to(dtype)
    got = ops.swiglu(x.to(DEV)).cpu().double()
    ref = pm.silu(x[:, :37].double()) * x[:, 37:].double()
    assert torch.allclose(got, ref, **_tol(dtype))


def test_sampling_matches_the_host_twin_and_the_distribution():
    ops = _ops()
    V = 301
    logits = torch.randn(6, V) * 2
    logits[0, 17] = logits[0, 250] = logits[0].max() + 1                # a planted tie: the lower id wins
    temp = torch.tensor([0.0, 0.0, 0.8, 0.8, 1.3, 0.8])
    seed = torch.tensor([0, 0, 7, 7, 9, 8], dtype=torch.int64)
    step = torch.tensor([0, 5, 3, 4, 3, 3], dtype=torch.int64)
    got = ops.sample(logits.to(DEV), temp.to(DEV), seed.to(DEV), step.to(DEV)).cpu().tolist()
    want = [pm.sample(logits[i].numpy(), float(temp[i]), int(seed[i]), int(step[i])) for i in range(6)]
    assert got[0] == 17 and got[1] == int(logits[1].argmax())
    assert got == want
    # distribution: 32768 draws of one row follow softmax(logits / T) (tests/test_ops_gpu.cu:755-800)
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, 3.0, -5.0])
    n = 32768
    draws = ops.sample(row.repeat(n, 1).to(DEV), torch.full((n,), 0.7, device=DEV), torch.full((n,), 5, dtype=torch.int64, device=DEV),
                       torch.arange(n, dtype=torch.int64, device=DEV)).cpu().numpy()
    p = torch.softmax(row / 0.7, 0).numpy()
    assert 0.5 * np.abs(np.bincount(draws, minlength=7) / n - p).sum() < 0.03


def test_sampling_with_top_k_and_top_p():
    ops = _ops()
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, 3.0, -5.0, 2.5])
    n = 8192
    def draw(k, p, T=1.0):
        return ops.sample_filtered(row.repeat(n, 1).to(DEV), torch.full((n,), T, device=DEV),
                                   torch.full((n,), 3, dtype=torch.int64, device=DEV), torch.arange(n, dtype=torch.int64, device=DEV),
                                   torch.full((n,), k, dtype=torch.int64, device=DEV), torch.full((n,), p, device=DEV)).cpu().numpy()
    d = draw(3, 1.0)
    assert set(d.tolist()) == {5, 7, 0}                                  # the three largest logits
    pk = torch.softmax(row[[0, 5, 7]], 0).numpy()
    assert 0.5 * np.abs(np.bincount(d, minlength=8)[[0, 5, 7]] / n - pk).sum() < 0.03
    probs = torch.softmax(row, 0)
    order = torch.argsort(probs, descending=True)
    keep = order[: int((torch.cumsum(probs[order], 0) < 0.8).sum()) + 1].tolist()   # smallest prefix reaching 0.8
    d = draw(0, 0.8)
    assert set(d.tolist()) == set(keep)
    assert set(draw(1, 1.0).tolist()) == {5} and set(draw(0, 1e-6).tolist()) == {5}
    assert set(draw(5, 0.999, 0.0).tolist()) == {5}                      # temperature 0 stays greedy
    assert len(set(draw(0, 1.0).tolist())) >= 6                          # no filter: nearly everything appears
