"""Interfaces and registries of the parts a layer is put together from.

A part knows its own sizes and constants (constructor arguments, from a ``PartSpec``), the tensors
it needs from the weight file (by local name) and how to run on the tokens of a step.  It does not
know which model it is in.  Kinds are looked up in four registries - mixers, feed-forwards, norms,
position encodings - plus one for block arrangements; a new kind is one ``register_*`` call, from
anywhere (a test registers a toy mixer without touching this package).

The reference has the same separation of primitives whose constants are constructor parameters
(src/layers/, src/models/llama.py:44-64) but one fixed block and no registries.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from ..config.model import PartSpec
from .context import CacheBinding, NormAhead, ResidualStream, StepContext, StepPrep


# ----------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values in pages: [pages, kv_heads, page, head_dim] each.  ``window`` None: every
    key is kept; a number: only the last ``window`` keys are needed, older pages are given back."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one tensor ``shape`` per live request (slot)."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ----------------------------------------------------------------------------- interfaces
class Part:
    """Base of all parts."""

    # False for a part whose forward depends on the step's host arrays (Python control flow over
    # sequences): its steps are then never captured into a CUDA graph
    graph_safe = True

    def __init__(self, dtype: torch.dtype, device: torch.device) -> None:
        self.dtype = dtype
        self.device = device

    def tensors(self) -> dict[str, tuple[tuple[int, ...], str]]:
        """local tensor name -> (shape, "matrix" | "vector").  Matrices are drawn N(0, 0.02) in
        the random-weights mode, vectors are norm weights."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Take the tensors (host, stored dtype) by local name; pack and move them to the device."""

    def prepare(self, prep: StepPrep) -> None:
        """Called once per step before the step's arrays go to the device: a part may add int32
        arrays of its own (work lists) with ``prep.add``."""


class Norm(Part):
    def forward(self, stream: ResidualStream, ctx: StepContext,
                rows: "torch.Tensor | None" = None) -> torch.Tensor:
        """Fold the stream's pending branch output into the residual and return the normalised
        rows [N, width] (or the rows picked by ``rows``) in the activation dtype."""
        raise NotImplementedError

    def ahead(self, stream: ResidualStream, ctx: StepContext, count: int) -> "NormAhead | None":
        """Optional: buffers with which the product before this norm does the norm's work
        (``NormAhead``; ``count`` shares of a row's sum of squares), or None if this norm must
        run itself."""
        return None


class NormRider:
    """Optional abilities of a mixer or feed-forward whose first and last operations are matrix
    products that can carry the norms around the part.  The defaults say no."""

    def takes_unscaled(self, n_rows: int) -> bool:
        """Whether ``forward`` accepts ``UnscaledRows`` in place of x for a step of n_rows."""
        return False

    def ahead_parts(self, n_rows: int) -> int:
        """Not 0: ``forward`` accepts ``ahead=NormAhead`` - its last product then adds the
        part's output to the residual itself, does the following norm's work and leaves this many
        shares of each row's sum of squares; ``forward`` returns None."""
        return 0


class PositionEncoding(Part):
    def rotation_table(self) -> "tuple[torch.Tensor | None, int]":
        """(inverse frequencies float32 [rotary_dim / 2] on the device, rotary_dim) for encodings
        that rotate q and k by position, which the fused rotate-and-store kernel applies; (None, 0)
        for encodings that do not."""
        return None, 0

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx: StepContext) -> None:
        """Hook for encodings that are not a rotation: change q [N, heads, d] and k [N, kv_heads,
        d] in place before k is stored.  The default does nothing."""


class Mixer(Part, NormRider):
    def cache_spec(self) -> "PagedKVSpec | StateSpec | None":
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext,
                cache: "CacheBinding | None") -> torch.Tensor:
        """x [N, width] (normalised) -> branch output [N, width]."""
        raise NotImplementedError


class FeedForward(Part, NormRider):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """Arrangement of a mixer, a feed-forward and their norms around the residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self) -> dict[str, Part]:
        """role -> part; the roles are the keys of ``LayerSpec.prefixes``."""
        return {"mixer": self.mixer, "feed_forward": self.feed_forward,
                "mixer_norm": self.mixer_norm, "feed_forward_norm": self.feed_forward_norm}

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: "CacheBinding | None",
                following: "tuple[Norm, Part] | None" = None) -> None:
        """``following``: the norm and the part that read the stream after this block (the next
        block's, if the model knows them), for arrangements that hand a norm's work to the
        product before it."""
        raise NotImplementedError


# ----------------------------------------------------------------------------- registries
PartFactory = Callable[..., Part]

MIXERS: dict[str, PartFactory] = {}
FEED_FORWARDS: dict[str, PartFactory] = {}
NORMS: dict[str, PartFactory] = {}
POSITION_ENCODINGS: dict[str, PartFactory] = {}
BLOCKS: dict[str, Callable[..., Block]] = {}


def _register(table: dict[str, Any], what: str, kind: str, factory: Any) -> None:
    if kind in table:
        raise ValueError(f"{what} kind '{kind}' is already registered")
    table[kind] = factory


def register_mixer(kind: str, factory: PartFactory) -> None:
    _register(MIXERS, "mixer", kind, factory)


def register_feed_forward(kind: str, factory: PartFactory) -> None:
    _register(FEED_FORWARDS, "feed-forward", kind, factory)


def register_norm(kind: str, factory: PartFactory) -> None:
    _register(NORMS, "norm", kind, factory)


def register_position_encoding(kind: str, factory: PartFactory) -> None:
    _register(POSITION_ENCODINGS, "position encoding", kind, factory)


def register_block(kind: str, factory: Callable[..., Block]) -> None:
    _register(BLOCKS, "block", kind, factory)


def _build(table: dict[str, PartFactory], what: str, spec: PartSpec, dtype: torch.dtype,
           device: torch.device) -> Part:
    if spec.kind not in table:
        raise ValueError(f"unknown {what} kind '{spec.kind}'; registered: {sorted(table)}")
    return table[spec.kind](dtype=dtype, device=device, **spec.params)


def build_mixer(spec: PartSpec, dtype: torch.dtype, device: torch.device) -> Mixer:
    return _build(MIXERS, "mixer", spec, dtype, device)          # type: ignore[return-value]


def build_feed_forward(spec: PartSpec, dtype: torch.dtype, device: torch.device) -> FeedForward:
    return _build(FEED_FORWARDS, "feed-forward", spec, dtype, device)  # type: ignore[return-value]


def build_norm(spec: PartSpec, dtype: torch.dtype, device: torch.device) -> Norm:
    return _build(NORMS, "norm", spec, dtype, device)            # type: ignore[return-value]


def build_position_encoding(spec: PartSpec, dtype: torch.dtype,
                            device: torch.device) -> PositionEncoding:
    return _build(POSITION_ENCODINGS, "position encoding", spec, dtype,
                  device)                                        # type: ignore[return-value]


def build_block(kind: str, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                feed_forward_norm: Norm) -> Block:
    if kind not in BLOCKS:
        raise ValueError(f"unknown block kind '{kind}'; registered: {sorted(BLOCKS)}")
    return BLOCKS[kind](mixer, feed_forward, mixer_norm, feed_forward_norm)


def compute_matrix(tensor: torch.Tensor, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A matrix operand in the compute dtype on the device."""
    return tensor.to(device=device, dtype=dtype).contiguous()


def stored_vector(tensor: torch.Tensor, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A small vector: float32 in the float32 path, else as stored (float32 or bfloat16)."""
    if dtype == torch.float32 or tensor.dtype not in (torch.float32, torch.bfloat16):
        tensor = tensor.to(torch.float32 if dtype == torch.float32 else torch.bfloat16)
    return tensor.to(device).contiguous()
