"""Cuts a step's attention into work items on the host.

A work item is a tile of query rows of one sequence (rows are (token, query head within its kv
head's group), token-major) together with a range of key positions.  Prompt portions get one item
per tile, covering all keys up to the tile's last position.  When a step has too few tiles to fill
the GPU (decoded tokens over long contexts), a tile's key range is cut into chunks at absolute
multiples of ``chunk``; each chunk writes a partial result and a combine item names the chunks of
the tile.  An item is (seq, row0, kv_begin, kv_end, partial slot or -1, the tile's first partial slot,
the tile's number of chunks that hold keys, the tile's index): ``struct WorkItem`` in the kernels;
a combine item is ``CombineItem``.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np

CHUNKS = (2048, 1024, 512, 256, 128, 64)


@dataclass
class AttentionPlan:
    items: np.ndarray          # int32 [num_items, 8]
    combine: np.ndarray        # int32 [num_combine, 4]
    num_partials: int          # partial slots used (each: kv_heads x rows_per_tile rows)
    rows_per_tile: int
    chunk: int                 # 0: nothing is split


def _tiles(seq_qlen: np.ndarray, seq_pos0: np.ndarray, group: int, rows_per_tile: int,
           window: int):
    """(seq, row0, lo, hi) of every tile, vectorised over sequences."""
    rows_total = seq_qlen.astype(np.int64) * group
    tiles_per_seq = (rows_total + rows_per_tile - 1) // rows_per_tile
    total = int(tiles_per_seq.sum())
    seq = np.repeat(np.arange(len(seq_qlen), dtype=np.int64), tiles_per_seq)
    first = np.cumsum(tiles_per_seq) - tiles_per_seq
    row0 = (np.arange(total, dtype=np.int64) - np.repeat(first, tiles_per_seq)) * rows_per_tile
    last_row = np.minimum(row0 + rows_per_tile, rows_total[seq]) - 1
    pos0 = seq_pos0.astype(np.int64)[seq]
    hi = pos0 + last_row // group + 1
    if window > 0:
        lo = np.maximum(0, pos0 + row0 // group - window + 1)
    else:
        lo = np.zeros(total, dtype=np.int64)
    return seq, row0, lo, hi


def _longest_first(items: np.ndarray, lo: np.ndarray) -> np.ndarray:
    """Items by falling number of keys: blocks start in this order, so the long ones of a causal
    prompt do not start last and leave the other SMs idle at the end.  (Partial slots and combine
    items name slots, not item indices, so the order is free.)"""
    if len(items) < 2:
        return items
    keys = items[:, 3].astype(np.int64) - np.maximum(items[:, 2].astype(np.int64), lo)
    return items[np.argsort(-keys, kind="stable")]


def choose_chunk(num_tiles: int, kv_heads: int, longest: int, blocks_per_sm: int = 2, *,
                 sm_count: int) -> int:
    """The largest chunk that still gives every one of the device's ``sm_count`` SMs
    ``blocks_per_sm`` blocks (as many as the kernel has resident at once); 0: do not split."""
    wanted = blocks_per_sm * sm_count
    if num_tiles * kv_heads >= wanted:
        return 0
    for chunk in CHUNKS:
        if num_tiles * kv_heads * ((longest + chunk - 1) // chunk) >= wanted:
            return chunk
    return CHUNKS[-1]


def choose_decode_split(num_tiles: int, kv_heads: int, span: int, max_cluster: int = 8,
                        per_sm: int = 4, *, sm_count: int) -> tuple[int, int, int]:
    """How the one-launch decode kernel cuts key ranges of up to ``span`` keys:
    (blocks a cluster, clusters a tile, chunk length).  The chunks of a cluster merge through
    shared memory; several clusters a tile merge through global memory, which costs a few
    microseconds, so a tile gets more than one cluster only when ranges are long and the step
    would otherwise leave most of the GPU idle.  ``per_sm``: blocks of the kernel an SM holds;
    ``sm_count``: SMs of the device."""
    blocks = max(num_tiles * kv_heads, 1)
    tiles_of_keys = max((span + 63) // 64, 1)
    cluster = 1
    # one round of blocks over the SMs at most, and no block without a whole tile of 64 keys
    per_sm = int(os.environ.get("DISTENGINE_B200_DECODE_BLOCKS_PER_SM", str(per_sm)))
    # (clusters of 8 are placed 8 blocks at a time and need a fifth of the places free: measured on
    # B200, 520 keys, 4 kv heads: 448 blocks in clusters of 8 a step of 0.96 ms against 0.98 in
    # clusters of 4, 512 blocks 1.06 against 1.02, 576 blocks 1.15 against 1.08)
    places = per_sm * sm_count
    while (cluster < max_cluster and cluster * 2 <= tiles_of_keys
           and blocks * cluster * 2 <= (places if cluster * 2 <= 4 else places * 4 // 5)):
        cluster *= 2
    # where the next power of two would not fit in one round, a size in between may; it pays for
    # long ranges only (measured: 4,096 keys at head size 128, 6 blocks a cluster against 8 in two
    # rounds, 61 against 76 us; 520 keys at batch 20, 7 against 4, 3 % slower a step)
    while (cluster < max_cluster and blocks * (cluster + 1) <= per_sm * sm_count
           and span >= (cluster + 1) * 512):
        cluster += 1
    clusters = (span + cluster * 2048 - 1) // (cluster * 2048)          # 2048 keys a block at most
    while (blocks * cluster * clusters < 2 * sm_count
           and span >= cluster * (clusters + 1) * 256):                   # 256 keys a block at least
        clusters += 1
    per_block = (span + cluster * clusters - 1) // (cluster * clusters)
    chunk = max((per_block + 63) // 64 * 64, 64)
    return cluster, clusters, chunk


def build_plan(seq_qlen: np.ndarray, seq_pos0: np.ndarray, group: int, kv_heads: int,
               rows_per_tile: int, window: int = 0, chunk: "int | None" = None,
               chunks_cap: "int | None" = None, sort: bool = True,
               sm_count: "int | None" = None) -> AttentionPlan:
    """``chunk`` None: chosen from the step's shape and the device's ``sm_count``.  ``chunks_cap`` (with a given chunk): every
    tile gets exactly that many items and one combine item, padded with empty ones, so that the
    arrays' shapes depend on the number of tiles only (what a replayed CUDA graph needs).
    ``sort`` false keeps the items in the order of the tiles and their chunks."""
    seq, row0, lo, hi = _tiles(seq_qlen, seq_pos0, group, rows_per_tile, window)
    total = len(seq)
    if chunk is None:
        longest = int((hi - lo).max()) if total else 0
        if sm_count is None:
            raise ValueError("build_plan chooses the chunk itself only when it is told the "
                             "device's number of SMs")
        chunk = choose_chunk(total, kv_heads, longest, sm_count=sm_count)
    if chunk == 0 or total == 0:
        items = np.zeros((total, 8), dtype=np.int32)
        items[:, 0], items[:, 1], items[:, 2], items[:, 3], items[:, 4] = seq, row0, 0, hi, -1
        items[:, 6], items[:, 7] = 1, np.arange(total)
        return AttentionPlan(_longest_first(items, lo) if sort else items,
                             np.zeros((0, 4), dtype=np.int32), 0, rows_per_tile, 0)

    c0 = lo // chunk
    c1 = (hi - 1) // chunk
    count = c1 - c0 + 1
    if chunks_cap is None:
        split = count > 1
        n_items = np.where(split, count, 1)
    else:
        if int(count.max()) > chunks_cap:
            raise ValueError(f"a key range needs {int(count.max())} chunks of {chunk}, the plan "
                             f"was capped at {chunks_cap}")
        split = np.ones(total, dtype=bool)
        n_items = np.full(total, chunks_cap, dtype=np.int64)
    item_first = np.cumsum(n_items) - n_items
    num_items = int(n_items.sum())
    owner = np.repeat(np.arange(total, dtype=np.int64), n_items)
    k = np.arange(num_items, dtype=np.int64) - item_first[owner]        # chunk index within tile
    c = c0[owner] + k
    begin = np.where(split[owner], c * chunk, 0)
    end = np.where(split[owner], np.minimum(hi[owner], (c + 1) * chunk), hi[owner])
    live = k < count[owner]
    begin = np.where(live, begin, 0)
    end = np.where(live, end, 0)

    # partial slots: consecutive for the chunks of one tile
    n_part = np.where(split, n_items, 0)
    part_first = np.cumsum(n_part) - n_part
    partial = np.where(split[owner], part_first[owner] + k, -1)

    items = np.zeros((num_items, 8), dtype=np.int32)
    items[:, 0], items[:, 1], items[:, 2], items[:, 3], items[:, 4] = (
        seq[owner], row0[owner], begin, end, partial)
    # the tile of an item: its first partial slot, how many of its items hold keys, its index
    items[:, 5], items[:, 6], items[:, 7] = part_first[owner], count[owner], owner
    sel = np.nonzero(split)[0]
    combine = np.zeros((len(sel), 4), dtype=np.int32)
    combine[:, 0], combine[:, 1], combine[:, 2] = seq[sel], row0[sel], part_first[sel]
    combine[:, 3] = count[sel]
    if sort:
        items = _longest_first(items, lo[owner])
    return AttentionPlan(items, combine, int(n_part.sum()), rows_per_tile, chunk)
