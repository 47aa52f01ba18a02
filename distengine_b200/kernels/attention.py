"""Attention over the paged cache: picks the kernel for a dtype and head size, plans a step's work
items on the host and launches them.

* bfloat16 with a head size that is a multiple of 16: the tensor-core kernel
  (``csrc/attention_mma.cu``, compiled for that head size at first use).  Sequences with many query
  rows in the step use its wide tile (64 rows), sequences with at most 16 rows (decoded tokens)
  its narrow tile (16 rows, the keys of a tile split over the warps).
* float32, or any other even head size up to 256: the CUDA-core kernel in float32 arithmetic
  (``csrc/attention_simt.cu``), 8 rows a tile.

Long key ranges of a step with few tiles are cut into chunks; ``de_attn_combine`` merges the
partial results (``attention_plan``).  In float32 the chunk length is fixed (``F32_CHUNK`` keys,
at absolute multiples of it) whatever else the step holds: a row's keys are then always summed in
the same order - tiles of 32 keys in ascending order within a chunk, chunks in ascending order -
so its result does not depend, bit for bit, on how the tokens were cut into steps or on what
shares the batch.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

import os

from . import library
from .attention_plan import build_plan, choose_chunk, choose_decode_split
from .ops import _check, _i32, _need, _ptr, _stream, _tag

MAX_HEAD_DIM = 256
F32_CHUNK = 128          # keys in a chunk of the float32 path (a fixed order of summation)
_status_fallback: "torch.Tensor | None" = None
NARROW_ROWS = 16


def check_head_dim(head_dim: int) -> None:
    if head_dim <= 0 or head_dim > MAX_HEAD_DIM or head_dim % 2 != 0:
        raise ValueError(f"attention kernels take even head sizes up to {MAX_HEAD_DIM}, "
                         f"got {head_dim}")


def uses_tensor_cores(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0


@dataclass
class _Shape:
    name: str            # suffix of the step arrays of this tile shape
    rows: int            # query rows in a tile
    code: int            # the kernel's shape argument (-1: the CUDA-core kernel)


class AttentionLauncher:
    """Plans and runs the attention of all layers that share one shape of heads."""

    def __init__(self, dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int,
                 scale: float, window: "int | None",
                 device: "torch.device | None" = None) -> None:
        check_head_dim(head_dim)
        if heads % kv_heads != 0:
            raise ValueError(f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        self.dtype, self.heads, self.kv_heads, self.head_dim = dtype, heads, kv_heads, head_dim
        self.scale, self.window = float(scale), int(window or 0)
        self.group = heads // kv_heads
        self.tensor_cores = uses_tensor_cores(dtype, head_dim)
        if self.tensor_cores:
            # wide tiles are 128 rows where the kernel gives a warp two row tiles (head size <= 64)
            self.shapes = [_Shape("wide", 128 if head_dim <= 64 else 64, 0),
                           _Shape("narrow", NARROW_ROWS, 1)]
            self.module = ("attention_mma", (f"HEAD_DIM={head_dim}",))
            self.decode_module = ("attention_decode", (f"HEAD_DIM={head_dim}",))
            # prompt portions at head sizes 64 and 128: the tcgen05 kernel (tensor-memory
            # accumulators, TMA page loads) takes the wide tiles, two row tiles of 128 a block at
            # head size 64 and one at 128; DISTENGINE_B200_ATTENTION=mma keeps the mma.sync one
            self.tcgen05_module = ("attention_tcgen05", (f"HEAD_DIM={head_dim}",))
            if (head_dim in (64, 128)
                    and os.environ.get("DISTENGINE_B200_ATTENTION", "tcgen05") != "mma"):
                self.shapes[0] = _Shape("wide", 256 if head_dim == 64 else 128, 2)
        else:
            self.shapes = [_Shape("rows8", 8, -1)]
            self.module = ("attention_simt", ())
        self.fixed_chunk = F32_CHUNK if dtype == torch.float32 else None
        # steps of decoded tokens only: rotation, cache write, attention and merge in one launch;
        # DISTENGINE_B200_DECODE_ATTENTION=split keeps them apart
        self.fused_decode = (self.tensor_cores and os.environ.get(
            "DISTENGINE_B200_DECODE_ATTENTION", "fused") != "split")
        self._decode_blocks_per_sm: "int | None" = None     # asked of the kernel at first use
        self._device = device
        self._sm_count: "int | None" = None                 # asked of the device at first use
        self.key = (f"attention/{'mma' if self.tensor_cores else 'simt'}/{self.group}/"
                    f"{kv_heads}/{head_dim}/{self.window}")

    def _blocks_per_sm(self) -> int:
        """Blocks an SM holds at once: one of the tcgen05 kernel (it takes nearly all shared
        memory), about two of the others; key ranges are only cut when there are fewer tiles."""
        return 1 if any(shape.code == 2 for shape in self.shapes) else 2

    def sm_count(self) -> int:
        """SMs of the device the layer runs on (the current one if none was named)."""
        if self._sm_count is None:
            device = self._device if self._device is not None else torch.cuda.current_device()
            self._sm_count = int(torch.cuda.get_device_properties(device).multi_processor_count)
        return self._sm_count

    def modules(self) -> list[tuple[str, tuple[str, ...]]]:
        """The kernel libraries this launcher calls (to compile them side by side up front)."""
        extra = [self.decode_module] if self.fused_decode else []
        if any(shape.code == 2 for shape in self.shapes):
            extra.append(self.tcgen05_module)
        return [self.module, ("attention_simt", ())] + extra

    # ------------------------------------------------------------------ host side
    def _split(self, seq_qlen: np.ndarray) -> list[np.ndarray]:
        """The step's sequences divided over the tile shapes (zero rows where not taken)."""
        if len(self.shapes) == 1:
            return [seq_qlen]
        narrow = seq_qlen.astype(np.int64) * self.group <= NARROW_ROWS
        # with many query heads per kv head even one token fills more than a narrow tile; such
        # sequences still take narrow tiles while they bring a single token
        narrow |= seq_qlen == 1
        return [np.where(narrow, 0, seq_qlen).astype(np.int32),
                np.where(narrow, seq_qlen, 0).astype(np.int32)]

    def _prepare_decode(self, prep, force_split: "tuple[int, int, int] | None") -> None:
        """A step in which every sequence brings one token: the work list of the one-launch
        decode kernel (``csrc/attention_decode.cu``)."""
        host = prep.host
        rows = NARROW_ROWS
        tiles = len(host.seq_qlen) * ((self.group + rows - 1) // rows)
        if prep.graph_shape is not None:
            span = int(prep.graph_shape["context_cap"])
        else:
            span = int(host.seq_pos0.max()) + 1
        if self.window:
            span = min(span, self.window)
        if self._decode_blocks_per_sm is None:
            lib = library.load(*self.decode_module)
            self._decode_blocks_per_sm = min(int(lib.de_attn_decode_blocks_per_sm(self.group)) or 4, 4)
        cluster, clusters, chunk = force_split or choose_decode_split(
            tiles, self.kv_heads, span, int(os.environ.get("DISTENGINE_B200_DECODE_CLUSTER", "8")),
            self._decode_blocks_per_sm, sm_count=self.sm_count())
        if force_split is None:
            # the number of items is fixed by the cap (a replayed graph needs that); the chunk
            # length follows the step's longest range, so that the items share it evenly
            longest = int(host.seq_pos0.max()) + 1
            if self.window:
                longest = min(longest, self.window)
            per_item = (longest + cluster * clusters - 1) // (cluster * clusters)
            chunk = max((per_item + 63) // 64 * 64, 64)
        # chunks lie at absolute multiples of `chunk`: a window that starts inside one reaches
        # into one chunk more
        cap = clusters * cluster
        if self.window and force_split is None:
            need = (span + chunk - 1) // chunk + 1
            cap = (need + cluster - 1) // cluster * cluster
        plan = build_plan(host.seq_qlen, host.seq_pos0, self.group, self.kv_heads, rows,
                          self.window, chunk, cap, sort=False)
        # the kernel derives the partial slots itself; their fields carry the token's position
        # and the sequence's slot instead
        items = plan.items
        items[:, 4] = host.seq_pos0[items[:, 0]]
        items[:, 5] = host.seq_slot[items[:, 0]]
        prep.add(f"{self.key}/decode/items", items)
        prep.notes[self.key] = ()
        prep.notes[self.key + "/decode"] = (tiles, cluster, cap)

    def prepare(self, prep, force_chunk: "int | None" = None,
                force_cap: "int | None" = None, force_shape: "str | None" = None,
                force_split: "tuple[int, int, int] | None" = None,
                allow_decode: bool = True) -> None:
        """Add this step's work lists to ``prep`` (once per step for all layers of this shape).
        The ``force_*`` arguments pin the chunk size, the chunk cap and the tile shape, and
        ``allow_decode`` false keeps a step of single tokens on the general kernels; tests use
        them to reach every path at small sizes."""
        if self.key in prep.notes:
            return
        host = prep.host
        one_each = bool(len(host.seq_qlen)) and bool((host.seq_qlen == 1).all())
        if self.fused_decode and one_each and force_shape is None and allow_decode:
            self._prepare_decode(prep, force_split)
            return
        prep.notes[self.key + "/decode"] = None
        notes = {}
        parts = self._split(host.seq_qlen)
        if force_shape is not None:
            parts = [host.seq_qlen if s.name == force_shape else np.zeros_like(host.seq_qlen)
                     for s in self.shapes]
        total_tiles = sum(int(((q.astype(np.int64) * self.group + s.rows - 1) // s.rows).sum())
                          for q, s in zip(parts, self.shapes))
        for qlen, shape in zip(parts, self.shapes):
            if not int(qlen.sum()):                      # no sequence takes this tile shape
                prep.add(f"{self.key}/{shape.name}/items", np.zeros((0, 8), dtype=np.int32))
                prep.add(f"{self.key}/{shape.name}/combine", np.zeros((0, 4), dtype=np.int32))
                notes[shape.name] = 0
                continue
            chunk = chunks_cap = None
            if force_chunk is not None:
                chunk, chunks_cap = force_chunk, force_cap
            elif self.fixed_chunk is not None:
                chunk = self.fixed_chunk
                if prep.graph_shape is not None:
                    cap = int(prep.graph_shape["context_cap"])
                    span = cap if not self.window else min(cap, self.window
                                                           + int(host.seq_qlen.max()))
                    chunks_cap = (span + chunk - 1) // chunk + (1 if self.window else 0)
            elif prep.graph_shape is not None:
                cap = int(prep.graph_shape["context_cap"])
                span = cap if not self.window else min(cap, self.window + int(host.seq_qlen.max()))
                chunk = choose_chunk(total_tiles, self.kv_heads, span, self._blocks_per_sm(),
                                     sm_count=self.sm_count())
                if chunk:
                    chunks_cap = (span + chunk - 1) // chunk + (1 if self.window else 0)
            elif int(qlen.sum()):
                live = qlen > 0
                longest = int((host.seq_pos0[live] + qlen[live]).max())
                if self.window:
                    longest = min(longest, self.window + int(qlen.max()))
                chunk = choose_chunk(total_tiles, self.kv_heads, longest, self._blocks_per_sm(),
                                     sm_count=self.sm_count())
            plan = build_plan(qlen, host.seq_pos0, self.group, self.kv_heads, shape.rows,
                              self.window, chunk, chunks_cap)
            prep.add(f"{self.key}/{shape.name}/items", plan.items)
            prep.add(f"{self.key}/{shape.name}/combine", plan.combine)
            notes[shape.name] = plan.num_partials
        prep.notes[self.key] = tuple(sorted(notes.items()))

    # ------------------------------------------------------------------ device side
    def run(self, q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor,
            v_pages: torch.Tensor, block_table: torch.Tensor, ctx) -> None:
        """q: rows of [heads * d] query features at the front of each row of ``q`` (row stride
        free); out [N, heads * d]; keys and values [pages, kv_heads, page, d]."""
        d = self.head_dim
        _need(q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype
              == self.dtype, "paged attention: q, out and the pages must have the layer's dtype "
              "and contiguous rows")
        _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
              and k_pages.shape[1] == self.kv_heads and k_pages.shape[3] == d
              and v_pages.shape == k_pages.shape,
              "paged attention: pages must be [pages, kv_heads, page, head_dim]")
        _i32(block_table, "block_table")
        partials = dict(ctx.notes[self.key])
        for shape in self.shapes:
            items = ctx.arrays[f"{self.key}/{shape.name}/items"]
            combine = ctx.arrays[f"{self.key}/{shape.name}/combine"]
            if items.shape[0] == 0:
                continue
            num_partials = partials[shape.name]
            acc = ml = None
            if num_partials:
                rows = num_partials * self.kv_heads * shape.rows
                acc = ctx.buffer(f"attention.partial_acc.{shape.name}", (rows * d,), torch.float32)
                ml = ctx.buffer(f"attention.partial_ml.{shape.name}", (rows * 2,), torch.float32)
            module = self.tcgen05_module if shape.code == 2 else self.module
            launch_items(shape.code, module, q, out, k_pages, v_pages, block_table,
                         ctx.seq_slot, ctx.seq_qstart, ctx.seq_qlen, ctx.seq_pos0, items, combine,
                         shape.rows, acc, ml, self.heads, self.kv_heads, d, self.scale, self.window,
                         getattr(ctx, "status", None))


    def decode_step(self, ctx) -> bool:
        """Whether ``run_decode`` takes this step (it then also rotates and stores k and v)."""
        return ctx.notes.get(self.key + "/decode") is not None

    def run_decode(self, qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor,
                   v_pages: torch.Tensor, block_table: torch.Tensor,
                   inv_freq: "torch.Tensor | None", rotary_dim: int, writes: bool, ctx) -> None:
        """A step of decoded tokens in one launch.  ``qkv``: rows [q heads | k heads | v heads]
        as the product left them; q and k are rotated inside, k and v stored in the pages
        (``writes``), the chunks of a split key range merged inside the kernel."""
        d = self.head_dim
        _need(qkv.stride(1) == 1 and out.stride(1) == 1 and qkv.dtype == out.dtype
              == k_pages.dtype == self.dtype and qkv.shape[1] == (self.heads + 2 * self.kv_heads) * d,
              "decode attention: qkv, out and the pages must have the layer's dtype, and qkv rows "
              "hold q, k and v")
        _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
              and k_pages.shape[1] == self.kv_heads and k_pages.shape[3] == d
              and v_pages.shape == k_pages.shape,
              "decode attention: pages must be [pages, kv_heads, page, head_dim]")
        _i32(block_table, "block_table")
        items = ctx.arrays[f"{self.key}/decode/items"]
        for name, t in (("seq_slot", ctx.seq_slot), ("seq_qstart", ctx.seq_qstart),
                        ("seq_pos0", ctx.seq_pos0), ("items", items)):
            _i32(t, name)
        tiles, cluster, cap = ctx.notes[self.key + "/decode"]
        _need(items.shape[0] == tiles * cap, "decode attention: the plan's size")
        acc = ml = None
        if cap > cluster:                         # several clusters a tile: partial results
            rows = tiles * (cap // cluster) * self.kv_heads * NARROW_ROWS
            acc = ctx.buffer("attention.partial_acc.decode", (rows * d,), torch.float32)
            ml = ctx.buffer("attention.partial_ml.decode", (rows * 2,), torch.float32)
        counters = ctx.buffer("attention.counters", (max(tiles, 1) * self.kv_heads,), torch.int32,
                              zero=True)
        if inv_freq is not None:
            _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
                  and inv_freq.shape[0] * 2 == rotary_dim, "decode attention: inv_freq must be "
                  "float32 [rotary_dim / 2]")
        lib = library.load(*self.decode_module)
        _check(lib.de_attn_decode(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), k_pages.data_ptr(),
            v_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), k_pages.shape[0],
            ctx.seq_slot.data_ptr(), ctx.seq_qstart.data_ptr(), ctx.seq_pos0.data_ptr(),
            items.data_ptr(), items.shape[0], cap, cluster, _ptr(acc), _ptr(ml),
            counters.data_ptr(), _ptr(inv_freq), int(rotary_dim) if inv_freq is not None else 0,
            1 if writes else 0, self.heads, self.kv_heads, d, k_pages.shape[2],
            float(self.scale), self.window, ctx.status.data_ptr(), _stream()), "decode attention")


def launch_items(code: int, module, q, out, k_pages, v_pages, block_table, seq_slot, seq_qstart,
                 seq_qlen, seq_pos0, items, combine, tile_rows, partial_acc, partial_ml, heads,
                 kv_heads, head_dim, scale, window, status=None) -> None:
    """One launch of a kernel over ``items`` and, if any range was split, the merge."""
    for name, t in (("seq_slot", seq_slot), ("seq_qstart", seq_qstart), ("seq_qlen", seq_qlen),
                    ("seq_pos0", seq_pos0), ("items", items)):
        _i32(t, name)
    lib = library.load(*module)
    if code in (0, 1):
        _need(lib.de_attn_mma_rows(code) == tile_rows,
              "paged attention: the plan's tile height is not the kernel's")
    elif code == 2:
        _need(lib.de_attn_tcgen05_rows() == tile_rows,
              "paged attention: the plan's tile height is not the kernel's")
    common = (q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_pages.data_ptr(),
              v_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0),
              k_pages.shape[0], seq_slot.data_ptr(), seq_qstart.data_ptr(), seq_qlen.data_ptr(),
              seq_pos0.data_ptr(), items.data_ptr(), items.shape[0], _ptr(partial_acc),
              _ptr(partial_ml), heads, kv_heads, head_dim, k_pages.shape[2], float(scale),
              int(window or 0))
    global _status_fallback
    if status is None:
        if _status_fallback is None or _status_fallback.device != q.device:
            _status_fallback = torch.zeros(1, dtype=torch.int32, device=q.device)
        status = _status_fallback
    if code < 0:
        _check(lib.de_attn_simt(_tag(q.dtype), *common, status.data_ptr(), _stream()),
               "paged attention")
    elif code == 2:
        _check(lib.de_attn_tcgen05(*common, status.data_ptr(), _stream()),
               "paged attention (tcgen05)")
    else:
        _check(lib.de_attn_mma(code, *common, status.data_ptr(), _stream()),
               "paged attention (tensor cores)")
    if combine is not None and combine.shape[0] > 0:
        _i32(combine, "combine")
        merge = library.load("attention_simt")
        _check(merge.de_attn_combine(_tag(q.dtype), out.data_ptr(), out.stride(0),
                                     seq_qstart.data_ptr(), seq_qlen.data_ptr(),
                                     combine.data_ptr(), combine.shape[0], partial_acc.data_ptr(),
                                     partial_ml.data_ptr(), heads, kv_heads, head_dim, tile_rows,
                                     _stream()), "attention combine")
