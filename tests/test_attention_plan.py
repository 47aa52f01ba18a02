"""The host-side planning of attention work: items, chunks, the decode kernel's split.  No GPU."""

import numpy as np
import pytest

from distengine_b200.kernels.attention_plan import build_plan, choose_chunk, choose_decode_split

SMS = 148          # the planners are told the device's number of SMs; the tests plan for this many


def _covered(items, group, rows_per_tile):
    """(seq, row) -> sorted list of key ranges, from the items of a plan."""
    out = {}
    for seq, row0, begin, end, *_ in items.tolist():
        if begin >= end:
            continue
        out.setdefault((seq, row0), []).append((begin, end))
    return {k: sorted(v) for k, v in out.items()}


@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("chunk,cap", [(0, None), (64, None), (128, 6), (None, None)])
def test_every_row_tile_gets_its_keys_exactly_once(window, chunk, cap):
    qlen = np.array([130, 1, 1, 21, 2], dtype=np.int32)
    pos0 = np.array([0, 0, 76, 279, 31], dtype=np.int32)
    group, kv_heads, rows = 3, 2, 16
    plan = build_plan(qlen, pos0, group, kv_heads, rows, window, chunk, cap, sm_count=SMS)
    ranges = _covered(plan.items, group, rows)
    for seq in range(len(qlen)):
        rows_total = int(qlen[seq]) * group
        for row0 in range(0, rows_total, rows):
            last_row = min(row0 + rows, rows_total) - 1
            hi = int(pos0[seq]) + last_row // group + 1
            lo = max(0, int(pos0[seq]) + row0 // group - window + 1) if window else 0
            got = ranges[(seq, row0)]
            # chunks are disjoint, in order, and reach from at most lo to exactly hi
            assert got[0][0] <= lo and got[-1][1] == hi
            for (b0, e0), (b1, e1) in zip(got, got[1:]):
                assert e0 == b1
    if cap is not None:
        tiles = sum(-(-int(q) * group // rows) for q in qlen)
        assert plan.items.shape[0] == tiles * cap           # a fixed number of items per tile


def test_items_carry_their_tile_and_start_longest_first():
    qlen = np.array([64, 8, 300], dtype=np.int32)
    pos0 = np.array([0, 500, 0], dtype=np.int32)
    plan = build_plan(qlen, pos0, 2, 1, 16, 0, chunk=0)
    keys = plan.items[:, 3] - plan.items[:, 2]
    assert (np.diff(keys) <= 0).all()                       # falling number of keys
    assert sorted(plan.items[:, 7].tolist()) == list(range(plan.items.shape[0]))
    split = build_plan(qlen, pos0, 2, 1, 16, 0, chunk=128, sort=False)
    for tile in np.unique(split.items[:, 7]):
        mine = split.items[split.items[:, 7] == tile]
        live = mine[mine[:, 3] > mine[:, 2]]
        assert (mine[:, 6] == len(live)).all()              # chunks that hold keys
        if len(live) > 1:
            assert (live[:, 4] == live[0, 5] + np.arange(len(live))).all()   # partial slots in a row


def test_capped_plan_refuses_a_range_that_needs_more_chunks():
    with pytest.raises(ValueError, match="capped"):
        build_plan(np.array([1], dtype=np.int32), np.array([999], dtype=np.int32), 1, 1, 16, 0,
                   chunk=64, chunks_cap=4)


@pytest.mark.parametrize("tiles,kv_heads,span", [(8, 4, 1024), (1, 4, 1024), (64, 4, 1024), (8, 4, 64),
                                                 (1, 4, 32768), (8, 4, 32768), (256, 8, 2048),
                                                 (1, 1, 1), (3, 5, 100000)])
@pytest.mark.parametrize("per_sm", [4, 3, 2])
def test_decode_split_covers_the_span_with_whole_tiles_of_keys(tiles, kv_heads, span, per_sm):
    cluster, clusters, chunk = choose_decode_split(tiles, kv_heads, span, per_sm=per_sm, sm_count=SMS)
    assert 1 <= cluster <= 8 and clusters >= 1
    # one round of blocks over the SMs, unless even single blocks do not fit in one
    assert cluster == 1 or tiles * kv_heads * cluster <= per_sm * SMS
    assert chunk % 64 == 0 and chunk >= 64
    assert cluster * clusters * chunk >= span                # every key has an item
    assert chunk <= 2048 + 63                                # no block walks more than that
    if cluster > 1:
        assert span >= 64 * cluster // 2                     # no cluster of blocks without keys


def test_decode_split_takes_sizes_between_the_powers_of_two():
    # 64 tiles of one kv head each... 8 kv heads, three blocks an SM: 6 blocks a cluster fit, 8 not
    assert choose_decode_split(8, 8, 4096, per_sm=3, sm_count=SMS)[0] == 6
    assert choose_decode_split(8, 8, 4096, per_sm=4, sm_count=SMS)[0] == 8
    assert choose_decode_split(8, 4, 520, per_sm=4, sm_count=SMS)[0] == 8
    assert choose_decode_split(64, 4, 520, per_sm=4, sm_count=SMS)[0] == 2
    assert choose_decode_split(20, 4, 520, per_sm=4, sm_count=SMS)[0] == 4       # short ranges: powers of two


def test_clusters_of_eight_only_while_a_fifth_of_the_places_stays_free():
    # 4 kv heads, 4 blocks an SM: 592 places; clusters of 8 up to 473 blocks (14 sequences: 448)
    for sequences, want in ((8, 8), (12, 8), (14, 8), (15, 4), (16, 4), (18, 4), (32, 4), (37, 4),
                            (38, 2), (64, 2)):
        assert choose_decode_split(sequences, 4, 640, per_sm=4, sm_count=SMS)[0] == want, sequences


def test_chunk_choice_fills_the_gpu_or_leaves_ranges_whole():
    assert choose_chunk(1000, 4, 4096, sm_count=SMS) == 0                  # enough tiles: no split
    c = choose_chunk(8, 4, 4096, sm_count=SMS)
    assert c in (2048, 1024, 512, 256, 128, 64) and 8 * 4 * -(-4096 // c) >= 2 * SMS
