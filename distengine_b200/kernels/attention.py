"""Launches attention over the paged cache: picks the kernel for a dtype and head size, and runs
a plan of work items (``attention_plan``) plus the merge of split key ranges."""

from __future__ import annotations

import torch

from . import library
from .ops import _check, _i32, _need, _ptr, _stream, _tag

MAX_HEAD_DIM = 256


def check_head_dim(head_dim: int) -> None:
    if head_dim <= 0 or head_dim > MAX_HEAD_DIM or head_dim % 2 != 0:
        raise ValueError(f"attention kernels take even head sizes up to {MAX_HEAD_DIM}, "
                         f"got {head_dim}")


def rows_per_tile(dtype: torch.dtype, head_dim: int) -> int:
    """Query rows in one work item of the kernel that serves this dtype and head size."""
    check_head_dim(head_dim)
    return 8


def paged_attention(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor,
                    v_pages: torch.Tensor, block_table: torch.Tensor, seq_slot: torch.Tensor,
                    seq_qstart: torch.Tensor, seq_qlen: torch.Tensor, seq_pos0: torch.Tensor,
                    items: torch.Tensor, combine: "torch.Tensor | None", num_partials: int,
                    tile_rows: int, partial_acc: "torch.Tensor | None",
                    partial_ml: "torch.Tensor | None", heads: int, kv_heads: int, head_dim: int,
                    scale: float, window: "int | None") -> None:
    """q: [N, >= heads * d] rows (row stride free, heads first); out [N, heads * d]."""
    check_head_dim(head_dim)
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype,
          "paged_attention: q, out and the pages must share a dtype and have contiguous rows")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and k_pages.shape[1] == kv_heads and k_pages.shape[3] == head_dim
          and v_pages.shape == k_pages.shape,
          "paged_attention: pages must be [pages, kv_heads, page, head_dim]")
    _need(heads % kv_heads == 0, "paged_attention: heads must be a multiple of kv_heads")
    for name, t in (("block_table", block_table), ("seq_slot", seq_slot),
                    ("seq_qstart", seq_qstart), ("seq_qlen", seq_qlen), ("seq_pos0", seq_pos0),
                    ("items", items)):
        _i32(t, name)
    num_items = items.shape[0]
    if num_partials > 0:
        need = num_partials * kv_heads * tile_rows
        _need(partial_acc is not None and partial_ml is not None
              and partial_acc.dtype == torch.float32 and partial_ml.dtype == torch.float32
              and partial_acc.numel() >= need * head_dim and partial_ml.numel() >= need * 2,
              "paged_attention: scratch for partial results is too small")
    lib = library.load("attention_simt")
    _check(lib.de_attn_simt(_tag(q.dtype), q.data_ptr(), q.stride(0), out.data_ptr(),
                            out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                            block_table.data_ptr(), block_table.stride(0), k_pages.shape[0],
                            seq_slot.data_ptr(), seq_qstart.data_ptr(), seq_qlen.data_ptr(),
                            seq_pos0.data_ptr(), items.data_ptr(), num_items, _ptr(partial_acc),
                            _ptr(partial_ml), heads, kv_heads, head_dim, k_pages.shape[2],
                            float(scale), int(window or 0), _stream()), "paged_attention")
    if combine is not None and combine.shape[0] > 0:
        _i32(combine, "combine")
        _check(lib.de_attn_combine(_tag(q.dtype), out.data_ptr(), out.stride(0),
                                   seq_qstart.data_ptr(), seq_qlen.data_ptr(), combine.data_ptr(),
                                   combine.shape[0], partial_acc.data_ptr(), partial_ml.data_ptr(),
                                   heads, kv_heads, head_dim, tile_rows, _stream()),
               "attention combine")
