"""What a part sees of one step: the ragged batch's arrays, its cache binding, scratch buffers.

A step holds N tokens of S sequences.  Tokens of a sequence are consecutive and in order.
Device arrays (int32):

    token_ids[N]  positions[N]  token_slot[N]  token_seq[N]
    seq_slot[S]   seq_qstart[S] (first token's index)  seq_qlen[S]  seq_pos0[S] (its position)
    logit_rows[R] (token indices whose logits are wanted)

``host`` has the same arrays as numpy, for parts that plan on the host.  The reference builds its
per-step tensors in the same spirit, once per step for all layers
(src/distengine/paged_kv_cache.py:263-293, src/distengine/model_runner.py:79-110).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Any

import numpy as np
import torch


class Workspace:
    """Named device buffers that live across steps, so a step allocates nothing once warm and a
    captured CUDA graph finds its buffers at the same addresses."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self._buffers: dict[str, torch.Tensor] = {}
        # views handed out before, by (name, shape, dtype): a step asks for the same ones again
        self._views: dict[tuple, torch.Tensor] = {}
        self.generation = 0          # grows whenever a buffer moves: captured graphs are stale then

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype,
            zero: bool = False) -> torch.Tensor:
        """``zero``: the buffer is zero when it is made (or made anew, larger); its users leave it
        zero after every use (counters that a kernel resets itself)."""
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        count = 1
        for s in shape:
            count *= int(s)
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < count:
            grow = count if buf is None or buf.dtype != dtype else max(count, 2 * buf.numel())
            make = torch.zeros if zero else torch.empty
            buf = make(max(grow, 1), dtype=dtype, device=self.device)
            self._buffers[name] = buf
            self.generation += 1
            self._views = {k: v for k, v in self._views.items() if k[0] != name}
        if len(self._views) > 4096:              # steps of ever new shapes: start over
            self._views.clear()
        view = self._views[key] = buf[:count].view(shape)
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class StepPrep:
    """Host side of a step before upload: the batch's numpy arrays plus arrays that parts add."""

    def __init__(self, host: SimpleNamespace, graph_shape: "dict[str, Any] | None" = None) -> None:
        self.host = host
        self.extra: dict[str, np.ndarray] = {}
        self.notes: dict[str, Any] = {}
        # set when the step is being shaped for a replayed CUDA graph: parts must then produce
        # arrays whose shapes depend on the batch's shape only (see kernels.attention_plan)
        self.graph_shape = graph_shape

    def add(self, name: str, array: np.ndarray) -> None:
        if name not in self.extra:
            self.extra[name] = np.ascontiguousarray(array, dtype=np.int32)

    def has(self, name: str) -> bool:
        return name in self.extra


@dataclass
class CacheBinding:
    """The cache of one run of a layer.  Paged keys/values: ``k_pages``/``v_pages``
    [pages, kv_heads, page, head_dim] and the group's ``block_table`` [slots, max_pages] (int32,
    -1 where a request holds no page).  Fixed-size state: ``state`` [slots, *shape].  ``writes``
    false: this run reads the cache that an earlier run of the plan wrote."""
    kind: str                                   # "paged" | "state"
    writes: bool = True
    k_pages: "torch.Tensor | None" = None
    v_pages: "torch.Tensor | None" = None
    block_table: "torch.Tensor | None" = None
    page_size: int = 0
    window: "int | None" = None
    state: "torch.Tensor | None" = None


@dataclass
class StepContext:
    device: torch.device
    dtype: torch.dtype
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_slot: torch.Tensor
    token_seq: torch.Tensor
    seq_slot: torch.Tensor
    seq_qstart: torch.Tensor
    seq_qlen: torch.Tensor
    seq_pos0: torch.Tensor
    logit_rows: torch.Tensor
    host: SimpleNamespace
    arrays: dict[str, torch.Tensor]
    notes: dict[str, Any]
    workspace: Workspace
    status: torch.Tensor                         # int32 [1]; a kernel sets it when it skips work
    extras: dict[str, Any] = field(default_factory=dict)

    def buffer(self, name: str, shape: tuple[int, ...], dtype: "torch.dtype | None" = None,
               zero: bool = False) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype or self.dtype, zero)


@dataclass
class UnscaledRows:
    """A norm's output but for the rows' factors: ``rows`` [N, width] is residual * norm weight in
    the activation dtype, and row m's factor is rsqrt(sum(parts[m]) / width + eps).  A factor is a
    scalar of its row, so a matrix product may take ``rows`` as they are and apply it to its
    float32 sums (``kernels.ops.linear(..., before=)``)."""
    rows: torch.Tensor
    parts: torch.Tensor                         # float32 [N, count]: shares of the sums of squares
    width: int
    eps: float


@dataclass
class NormAhead:
    """A norm's work handed to the product that runs before it: that product adds its result to
    ``resid`` and writes ``rows`` and ``parts`` as ``UnscaledRows`` describes them
    (``kernels.ops.linear(..., after=)``), so the norm needs no kernel of its own."""
    norm: Any                                   # the norm part whose work this is
    resid: torch.Tensor                         # float32 [N, width]
    weight: torch.Tensor                        # the norm's weight [width]
    eps: float
    rows: torch.Tensor                          # [N, width], activation dtype
    parts: torch.Tensor                         # float32 [N, count]

    def result(self) -> UnscaledRows:
        return UnscaledRows(self.rows, self.parts, self.resid.shape[1], self.eps)


class ResidualStream:
    """The residual stream in float32 and the branch output that has not been added yet.

    A norm folds ``pending`` into ``resid`` in the same kernel that normalises, so the sum is
    formed in 32-bit and costs no pass over memory of its own.  ``ahead``: the last product
    already added its result and did the next norm's work (``NormAhead``); that norm hands out
    its result instead of running."""

    def __init__(self, resid: torch.Tensor) -> None:
        self.resid = resid                      # float32 [N, width]
        self.pending: "torch.Tensor | None" = None
        self.ahead: "NormAhead | None" = None
