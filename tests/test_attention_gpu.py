"""The tensor-core attention kernels alone (flash-decoding with slices, causal prefill tiles) against the plain
attention formula in float64, on shuffled pages with NaN in every cache row that is not in use."""
import math

import pytest
import torch

import plain_model as pm
from test_kernels_gpu import _paged_setup

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(heads, kv, hd, window, segs, n_splits=None, seed=0, n_clusters=1, tc_split=None, count_decode=False):
    """segs: list of (context length before the step, tokens in the step)."""
    from infer_b200 import fast_ops
    lens = [c + n for c, n in segs]
    table, kc, vc, ks, vs = _paged_setup(torch.bfloat16, heads, kv, hd, 16, lens, n_pages=sum(-(-n // 16) for n in lens) + 5, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    T = sum(n for _, n in segs)
    q = torch.randn(T, heads, hd, generator=g).bfloat16()
    seg_start = [0]
    for _, n in segs:
        seg_start.append(seg_start[-1] + n)
    scale = 1 / math.sqrt(hd)
    ref = torch.zeros(T, heads, hd, dtype=torch.float64)
    r = 0
    for s, (c, n) in enumerate(segs):
        # the step's queries sit at rows c .. c + n - 1 of a sequence of c + n positions; causal, so one call serves all
        qq = torch.zeros(c + n, heads, hd, dtype=torch.float64)
        qq[c:] = q[r:r + n].double()
        ref[r:r + n] = pm.attention(qq, ks[s][:c + n].double(), vs[s][:c + n].double(), window, scale)[c:]
        r += n
    st = fast_ops.device_state(DEV)
    st.status.zero_()
    out = fast_ops.attention_fast(
        q.reshape(T, -1).contiguous().to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV),
        torch.tensor(seg_start, dtype=torch.int32, device=DEV), torch.tensor([c for c, _ in segs], dtype=torch.int32, device=DEV),
        heads, kv, hd, window, scale, any(n == 1 for _, n in segs), max(n for _, n in segs), max(lens), n_splits=n_splits,
        n_decode=sum(1 for _, n in segs if n == 1) if count_decode else None, n_clusters=n_clusters, tc_split=tc_split)
    assert out is not None
    assert st.status.item() == 0
    got = out.cpu().double().view_as(ref)
    assert not torch.isnan(got).any(), "a cache row that is not in use reached a sum"
    err = (got - ref).abs().max().item()
    assert err < 2e-2, f"max |diff| {err:.4f}"
    return got


LAYOUTS = [(12, 2, 128), (14, 2, 64), (4, 4, 16), (8, 1, 32), (5, 5, 48), (3, 1, 96), (16, 1, 64), (24, 2, 32)]


@pytest.mark.parametrize("heads,kv,hd", LAYOUTS)
@pytest.mark.parametrize("splits", [1, 4, None])
def test_decode(heads, kv, hd, splits):
    _run(heads, kv, hd, None, [(0, 1), (1, 1), (15, 1), (16, 1), (255, 1), (1000, 1), (33, 1)], splits)


@pytest.mark.parametrize("heads,kv,hd,clusters", [(12, 2, 128, 2), (12, 2, 128, 32), (14, 2, 64, 5), (3, 1, 96, 3)])
def test_decode_with_several_clusters_per_kv_head(heads, kv, hd, clusters):
    """Long contexts at small batches: several clusters of 8 slices share a (segment, kv head) and meet in the
    workspace. Contexts that leave most slices empty (1 and 40 keys over up to 256 slices), ragged ones, and a key
    range of thousands; twice, so that the counters must have come back to zero; the same bits whoever arrives last."""
    from infer_b200 import fast_ops
    segs = [(0, 1), (39, 1), (1300, 1), (2051, 1)]
    first = _run(heads, kv, hd, None, segs, 8, seed=3, n_clusters=clusters)
    again = _run(heads, kv, hd, None, segs, 8, seed=3, n_clusters=clusters)
    assert torch.equal(first, again)
    assert int(fast_ops.device_state(DEV)._counters.abs().sum()) == 0
    _run(heads, kv, hd, 700, segs[1:], 8, seed=4, n_clusters=clusters)      # a window that begins inside a late slice


def test_decode_cluster_count_follows_context_and_batch():
    from infer_b200 import fast_ops
    st = fast_ops.device_state(DEV)
    assert fast_ops._decode_splits(st, 8, 2, 2048) == (8, 1)                # the serving shape: one cluster
    n, c = fast_ops._decode_splits(st, 1, 2, 30000)
    assert n == 8 and c > 1 and 2 * 8 * c <= 2 * st.sm_count and (30000 // 16) // (8 * c) >= 16
    assert fast_ops._decode_splits(st, 8, 2, 8192) == (8, 1)                # not long enough to pay for the second level
    assert fast_ops._decode_splits(st, 64, 2, 30000)[1] == 1                # enough requests: no second level
    with pytest.raises(fast_ops.KernelError):
        _run(12, 2, 128, None, [(300, 1)], 4, n_clusters=2)                 # several clusters need 8 slices each


@pytest.mark.parametrize("heads,kv,hd", LAYOUTS)
def test_decode_with_window(heads, kv, hd):
    _run(heads, kv, hd, 40, [(0, 1), (38, 1), (39, 1), (40, 1), (41, 1), (500, 1)], 2)
    _run(heads, kv, hd, 1, [(0, 1), (77, 1)], 1)


@pytest.mark.parametrize("heads,kv,hd", LAYOUTS)
def test_prefill_portions(heads, kv, hd):
    _run(heads, kv, hd, None, [(0, 2), (0, 64), (0, 65), (7, 130), (300, 17), (63, 2)])


@pytest.mark.parametrize("heads,kv,hd", [(12, 2, 128), (5, 5, 48)])
def test_prefill_with_window(heads, kv, hd):
    _run(heads, kv, hd, 40, [(0, 100), (90, 70), (39, 3)])
    _run(heads, kv, hd, 200, [(10, 260)])


@pytest.mark.parametrize("tc", [True, False], ids=["tcgen05", "mma.sync"])
@pytest.mark.parametrize("heads,kv,hd", [(12, 2, 128), (14, 2, 64)])
def test_prefill_long(heads, kv, hd, tc, monkeypatch):
    """Several query tiles and many key tiles per segment, through the tensor-memory kernel (128 queries x 128 keys per
    tile, keys two tiles ahead) and through the mma.sync kernel: contexts that end inside a tile, a window that drops
    whole tiles, a portion that starts in the middle of a page."""
    from infer_b200 import fast_ops
    monkeypatch.setattr(fast_ops, "ATTENTION_TC", tc)
    _run(heads, kv, hd, None, [(0, 700), (1000, 300), (130, 129), (5, 2)])
    _run(heads, kv, hd, 300, [(0, 650), (900, 140)])


@pytest.mark.parametrize("split", [2, 3, 4])
@pytest.mark.parametrize("heads,kv,hd", [(12, 2, 128), (14, 2, 64)])
def test_prefill_with_shared_query_tiles(heads, kv, hd, split):
    """The keys of a query tile on several CTAs that meet in the workspace: query tiles with 1 to 17 key tiles (those
    with fewer than eight stay whole, nine go two ways, twelve and more up to four ways), a portion behind a long
    context, a two-token segment with twelve key tiles, one-token segments beside them, and a window that cuts the
    first key tile of a part; twice, so that the counters must have come back to zero; the same bits whoever arrives
    last."""
    from infer_b200 import fast_ops
    segs = [(0, 1100), (1900, 200), (1, 1), (1530, 2), (500, 1)]
    first = _run(heads, kv, hd, None, segs, 2, seed=5, tc_split=split)
    again = _run(heads, kv, hd, None, segs, 2, seed=5, tc_split=split)
    assert torch.equal(first, again)
    assert int(fast_ops.device_state(DEV)._counters.abs().sum()) == 0
    whole = _run(heads, kv, hd, None, segs, 2, seed=5, tc_split=1)
    assert (first - whole).abs().max() < 1e-2
    # as the engine calls it: the scratch is laid out over the segments of two or more tokens only
    packed = _run(heads, kv, hd, None, segs, 2, seed=5, tc_split=split, count_decode=True)
    assert torch.equal(first, packed)
    _run(heads, kv, hd, 1200, [(700, 900), (2000, 130)], seed=6, tc_split=split)


def test_prefill_split_follows_the_shape():
    from infer_b200.fast_ops import prefill_split
    assert prefill_split(148, 12, 1, 512, 4096, None) == 3         # a portion behind a long context: 48 long CTAs -> 144
    assert prefill_split(148, 12, 1, 512, 8192, None) == 3
    assert prefill_split(148, 12, 1, 1024, 1024, None) > 1         # 96 CTAs; the one query tile with 8 key tiles is shared
    assert prefill_split(148, 12, 1, 2048, 2048, None) == 1        # 192 CTAs already: more starts cost more than they even out
    assert prefill_split(148, 28, 1, 2048, 2048, None) == 1
    assert prefill_split(148, 12, 4, 300, 600, None) == 1          # too few key tiles to share
    assert prefill_split(148, 12, 1, 128, 4096, 256) == 1          # a window of three key tiles
    assert prefill_split(148, 12, 0, 1, 4096, None) == 1           # decode only


@pytest.mark.parametrize("heads,kv,hd", [(12, 2, 128), (4, 4, 16)])
def test_mixed_step(heads, kv, hd):
    _run(heads, kv, hd, None, [(100, 1), (0, 40), (517, 1), (30, 5), (0, 1)], 2)


def test_slice_counts_give_the_same_result():
    a = _run(12, 2, 128, None, [(2047, 1), (700, 1)], 1, seed=3)
    for s in (2, 4, 8):
        b = _run(12, 2, 128, None, [(2047, 1), (700, 1)], s, seed=3)
        assert (a - b).abs().max() < 1e-2


def test_spike_at_a_far_key():
    """One key far back carries nearly all the weight (first, middle, last position of a long context)."""
    from infer_b200 import fast_ops
    hd, n = 64, 1500
    for spike in (0, 777, n - 1):
        table, kc, vc, ks, vs = _paged_setup(torch.bfloat16, 1, 1, hd, 16, [n], n_pages=100, seed=spike)
        q = torch.randn(1, hd).bfloat16()
        pg, off = int(table[0, spike // 16]), spike % 16
        kc[pg, 0, off] = (q[0].float() * 3.0).bfloat16()
        out = fast_ops.attention_fast(q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                      torch.tensor([n - 1], dtype=torch.int32, device=DEV), 1, 1, hd, None, 1 / math.sqrt(hd), True, 1, n, n_splits=4)
        assert (out.cpu().float() - vs[0][spike].view(1, -1)).abs().max() < 0.25


def test_refused_shapes_fall_back():
    from infer_b200 import fast_ops
    assert not fast_ops.attention_supported(4, 4, 256, 16)
    assert not fast_ops.attention_supported(4, 4, 24, 16)
    assert not fast_ops.attention_supported(4, 4, 64, 32)
    assert not fast_ops.attention_supported(34, 2, 64, 16)


@pytest.mark.parametrize("heads,kv,hd", [(12, 2, 128), (14, 2, 64), (8, 1, 32), (3, 1, 96)])
@pytest.mark.parametrize("window", [None, 40])
@pytest.mark.parametrize("splits", [1, 8, None, (8, 3)])
def test_fused_decode_equals_rotate_store_then_attend(heads, kv, hd, window, splits):
    """The one-kernel decode path (rotation, cache write, attention) against the plain rotate-and-store kernel
    followed by the separate attention kernel: same output, and the same cache contents afterwards."""
    from infer_b200 import fast_ops, ops
    from infer_b200.parts.rotary import rotary_tables
    ctxs = [0, 1, 15, 16, 17, 255, 700, 33]
    S = len(ctxs)
    lens = [c + 1 for c in ctxs]
    table, kc, vc, ks, vs = _paged_setup(torch.bfloat16, heads, kv, hd, 16, lens, n_pages=sum(-(-n // 16) for n in lens) + 3, seed=5)
    g = torch.Generator().manual_seed(9)
    qkv = torch.randn(S, (heads + 2 * kv) * hd, generator=g).bfloat16().to(DEV)
    cos, sin = (t.to(DEV) for t in rotary_tables(hd, 10000.0, 1024))
    seg_start = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    pos0 = torch.tensor(ctxs, dtype=torch.int32, device=DEV)
    seg = torch.arange(S, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    k1, v1 = kc.clone().to(DEV), vc.clone().to(DEV)
    q = ops.rope_kv_write(qkv, cos, sin, pos0, seg, table.to(DEV), k1, v1, heads, kv, hd, True)
    ref = fast_ops.attention_fast(q, k1, v1, table.to(DEV), seg_start, pos0, heads, kv, hd, window, scale, True, 1, max(lens), n_splits=1)
    k2, v2 = kc.clone().to(DEV), vc.clone().to(DEV)
    st = fast_ops.device_state(DEV)
    st.status.zero_()
    splits, clusters = splits if isinstance(splits, tuple) else (splits, 1)
    got = fast_ops.attention_decode_fused(qkv, cos, sin, k2, v2, table.to(DEV), seg_start, pos0, heads, kv, hd, window, scale,
                                          max(lens), True, splits, n_clusters=clusters)
    assert got is not None and st.status.item() == 0
    assert not torch.isnan(got.float()).any()
    assert (got.float() - ref.float()).abs().max() < 1e-2
    same = lambda a, b: torch.equal(torch.nan_to_num(a.float(), nan=7.0), torch.nan_to_num(b.float(), nan=7.0))
    assert same(k1, k2) and same(v1, v2), "the fused kernel must leave the cache exactly as the separate kernel does"
