"""Host-side decisions of the kernels' launchers, which need no GPU: how the tcgen05 matrix product maps a shape onto
tiles and K slices (the planner is a host function of the compiled library) and how the decode attention cuts the key
range into slices and clusters. The shapes are those of the 1.5B model's layer on a GPU of 148 SMs."""
import types

import pytest

SMS = 148


def _plan(M, N, K, sms=SMS):
    from infer_b200 import fast_ops
    from infer_b200.csrc.build import BuildError
    try:
        return fast_ops.gemm_plan(M, N, K, sms)
    except BuildError as e:                                      # no nvcc on this machine: the planner cannot be built
        pytest.skip(f"the library that holds the planner cannot be compiled here: {str(e)[:80]}")


def test_few_tokens_take_the_swapped_mapping_with_cluster_slices():
    for M, bn in ((1, 16), (16, 16), (17, 32), (33, 64), (64, 64), (65, 128), (128, 128)):
        swap, got_bn, splits, ws, counters = _plan(M, 1536, 8960)
        assert (swap, got_bn) == (1, bn)
        assert splits == 8 and ws == 0 and counters == 0          # 12 tiles: 8 slices as a cluster, no scratch
    # enough tiles to fill the GPU: no slices at all
    assert _plan(64, 17920, 1536) == (1, 64, 1, 0, 0)
    # a slice keeps at least two k-blocks
    assert _plan(8, 1536, 320)[2] == 2


def test_middling_token_counts_take_the_plain_mapping():
    assert _plan(129, 1536, 8960)[:2] == (0, 128)
    # 24 tiles: 4 slices of K as a cluster (8 would leave a third of the CTAs to a second round), no scratch
    assert _plan(256, 1536, 8960) == (0, 128, 4, 0, 0)
    assert _plan(768, 1536, 8960) == (0, 128, 2, 0, 0)             # 72 tiles in two slices: 144 CTAs run at once
    assert _plan(512, 1536, 8960) == (0, 768, 4, 0, 0)             # 24 wide tiles in four slices instead of 48 in two
    # very few tiles: up to 16 slices through the workspace, with one counter per tile
    swap, bn, splits, ws, counters = _plan(200, 300, 4096)
    assert (swap, bn, splits, counters) == (0, 128, 16, 6) and ws == 16 * 6 * 128 * 128


def test_many_tokens_take_the_persistent_kernel_with_the_width_that_fills_the_sms():
    assert _plan(2048, 17920, 1536) == (0, 512, 1, 0, 0)          # 128 x 256 tiles: 1120 of them
    assert _plan(2048, 2048, 1536) == (0, 512, 1, 0, 0)           # 128 tiles in one round; narrower would need two
    assert _plan(2048, 1536, 8960) == (0, 352, 1, 0, 0)           # 16 x 9 tiles of 176 columns = 144 CTAs
    assert _plan(2048, 1536, 1536) == (0, 352, 1, 0, 0)
    assert _plan(3000, 3584, 3584)[1] in (352, 384, 512)
    # a long K on few tiles: 128 x 256 tiles with K slices as a cluster (5 x 14 tiles x 2 slices = 140 CTAs)
    assert _plan(540, 3584, 18944) == (0, 768, 2, 0, 0)
    assert _plan(512, 3584, 18944) == (0, 768, 2, 0, 0)
    assert _plan(512, 4608, 3584)[1] == 352                        # 56 k-blocks: the slices' exchange would not pay


def test_refused_shapes():
    assert _plan(8, 1536, 100) is None                            # K not a multiple of 8
    assert _plan(0, 1536, 1536) is None


def test_decode_attention_slices_and_clusters():
    from infer_b200 import fast_ops
    st = types.SimpleNamespace(sm_count=SMS)
    assert fast_ops._decode_splits(st, 8, 2, 2048) == (8, 1)      # the serving shape: 128 CTAs, one cluster each
    assert fast_ops._decode_splits(st, 64, 2, 2048) == (1, 1)     # 128 CTAs for 148 SMs: a second slice would not pay for its merge
    assert fast_ops._decode_splits(st, 48, 2, 2048) == (2, 1)     # 96: two slices
    assert fast_ops._decode_splits(st, 1, 2, 100) == (1, 1)       # 7 pages: not worth cutting
    assert fast_ops._decode_splits(st, 8, 2, 8192) == (8, 1)      # the second level does not pay yet
    n, c = fast_ops._decode_splits(st, 1, 2, 30000)
    assert n == 8 and 1 < c <= fast_ops.ATTENTION_MAX_CLUSTERS
    assert 2 * 8 * c <= 2 * SMS and (30000 // 16) // (8 * c) >= fast_ops.ATTENTION_CLUSTER_PAGES
    assert fast_ops._decode_splits(st, 8, 2, 30000) == (8, 2)     # 128 CTAs already: at most two per SM
    assert fast_ops._decode_scratch(st, 8, 2, 128, 1) == (None, None)


def test_every_plan_that_the_no_alloc_entry_point_accepts_fits_its_array():
    """ib_gemm_tc_static hands its built-in array (8 MiB: 4096 counters, then partial tiles) to the kernel exactly
    when the plan sums K slices through global memory, and refuses when the plan's figures exceed the array. So for
    every shape the plan's figures must be the kernel's true need (slices x tiles x 128 x bn floats, one counter per
    tile), and the plans that add their slices in shared memory must state no need at all. Swept over the products
    of the 1.5B, 7B and 14B layer sizes for 17..4096 rows, and a few odd shapes."""
    room_floats = ((8 << 20) - 4096 * 4) // 4
    widths = [(1536, 2048), (1536, 1536), (1536, 17920), (8960, 1536),            # (K, N) of q/k/v, o, gate/up, down
              (3584, 4608), (3584, 3584), (3584, 37888), (18944, 3584),
              (5120, 7168), (5120, 5120), (5120, 27648), (13824, 5120),
              (4096, 136), (1536, 300), (1024, 256), (16384, 768)]
    rows = list(range(17, 130)) + list(range(130, 1025, 37)) + [1024, 2048, 3000, 4096]
    reached = 0
    for K, N in widths:
        for M in rows:
            plan = _plan(M, N, K)
            assert plan is not None
            swap, bn, splits, ws, counters = plan
            if ws == 0:
                assert counters == 0
                # no scratch: one slice, or slices that form a cluster (at most 8; plain mapping 2, 4 or 8)
                assert splits == 1 or (splits <= 8 and (swap or splits in (2, 4, 8)))
                continue
            assert not swap and bn == 128 and splits > 1
            tiles = -(-M // 128) * -(-N // bn)
            assert ws == splits * tiles * 128 * bn and counters == tiles
            if ws <= room_floats and counters <= 4096:
                reached += 1                                          # accepted: it fits by the same comparison
    assert reached > 0
