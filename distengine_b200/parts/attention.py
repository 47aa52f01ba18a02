"""Grouped-query attention over the paged cache.

q, k, v are one product against the stacked matrix [(heads + 2 kv_heads) * d, width] (the
reference runs three, src/layers/attention.py:120-136); q and k are rotated and k, v stored in the
pages by one kernel (:138-141); attention reads the pages through the block table
(``kernels.attention``); then the output product (:155).  Heads, kv heads, head size, scale and
window are constructor arguments; the position encoding is a part of its own.
"""

from __future__ import annotations

import torch

from ..config.model import PartSpec
from ..kernels import ops
from ..kernels.attention import AttentionLauncher
from .base import (Mixer, PagedKVSpec, build_position_encoding, compute_matrix, register_mixer)
from .context import CacheBinding, NormAhead, StepContext, StepPrep, UnscaledRows


class PagedAttention(Mixer):
    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int, scale: float,
                 window: "int | None", position: PartSpec, dtype: torch.dtype,
                 device: torch.device) -> None:
        super().__init__(dtype, device)
        if heads % kv_heads != 0:
            raise ValueError(f"attention: heads ({heads}) must be a multiple of kv_heads "
                             f"({kv_heads})")            # src/layers/attention.py:18-19
        if window is not None and window <= 0:
            raise ValueError(f"attention: window must be positive or None, got {window}")
        self.width, self.heads, self.kv_heads, self.head_dim = width, heads, kv_heads, head_dim
        self.scale, self.window = float(scale), window
        self.position = build_position_encoding(position, dtype, device)
        self.kernels = AttentionLauncher(dtype, heads, kv_heads, head_dim, scale, window, device)
        self.w_qkv: "torch.Tensor | None" = None
        self.w_o: "torch.Tensor | None" = None

    # ------------------------------------------------------------------ weights
    def tensors(self):
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        return {"q_proj.weight": ((q, self.width), "matrix"),
                "k_proj.weight": ((kv, self.width), "matrix"),
                "v_proj.weight": ((kv, self.width), "matrix"),
                "o_proj.weight": ((self.width, q), "matrix")}

    def load(self, tensors):
        stacked = torch.cat((tensors["q_proj.weight"], tensors["k_proj.weight"],
                             tensors["v_proj.weight"]), dim=0)
        self.w_qkv = compute_matrix(stacked, self.dtype, self.device)
        self.w_o = compute_matrix(tensors["o_proj.weight"], self.dtype, self.device)

    # ------------------------------------------------------------------ cache
    def cache_spec(self):
        return PagedKVSpec(self.kv_heads, self.head_dim, self.window)

    # ------------------------------------------------------------------ step
    @property
    def prepare_key(self) -> str:
        """Layers with the same key share one plan of a step's attention work."""
        return self.kernels.key

    def prepare(self, prep: StepPrep) -> None:
        self.kernels.prepare(prep)

    def takes_unscaled(self, n_rows: int) -> bool:
        return ops.norm_ride_parts(n_rows, self.w_qkv, self.dtype) > 0

    def ahead_parts(self, n_rows: int) -> int:
        return ops.norm_ride_parts(n_rows, self.w_o, self.dtype)

    def forward(self, x: "torch.Tensor | UnscaledRows", ctx: StepContext,
                cache: "CacheBinding | None",
                ahead: "NormAhead | None" = None) -> "torch.Tensor | None":
        if cache is None or cache.kind != "paged":
            raise ValueError("attention needs a paged key/value cache")
        before = None
        if isinstance(x, UnscaledRows):
            before, x = x, x.rows
        n, d = x.shape[0], self.head_dim
        qkv = ctx.buffer("attention.qkv", (n, (self.heads + 2 * self.kv_heads) * d))
        ops.linear(x, self.w_qkv, out=qkv, status=ctx.status, before=before)
        self.position.apply(qkv[:, : self.heads * d].view(n, self.heads, d),
                            qkv[:, self.heads * d: (self.heads + self.kv_heads) * d]
                            .view(n, self.kv_heads, d), ctx)
        inv_freq, rotary_dim = self.position.rotation_table()
        out = ctx.buffer("attention.context", (n, self.heads * d))
        if self.kernels.decode_step(ctx):
            # decoded tokens only: rotation, cache write, attention and merge are one kernel
            self.kernels.run_decode(qkv, out, cache.k_pages, cache.v_pages, cache.block_table,
                                    inv_freq, rotary_dim, cache.writes, ctx)
        else:
            ops.rope_kv_write(qkv, ctx.positions, ctx.token_slot, inv_freq, rotary_dim,
                              self.heads, self.kv_heads, d, cache.k_pages, cache.v_pages,
                              cache.block_table, cache.writes, ctx.status)
            self.kernels.run(qkv, out, cache.k_pages, cache.v_pages, cache.block_table, ctx)
        if ahead is not None:          # the product joins the residual and does the next norm's work
            ops.linear(out, self.w_o, out=ahead.rows, status=ctx.status, after=ahead)
            return None
        branch = ctx.buffer("attention.out", (n, self.width))
        ops.linear(out, self.w_o, out=branch, status=ctx.status)
        return branch


register_mixer("attention", PagedAttention)
