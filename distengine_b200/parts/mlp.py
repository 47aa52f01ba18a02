"""Dense gated feed-forward (SwiGLU): down( silu(gate(x)) * up(x) ), no biases
(src/models/llama.py:13-29, src/layers/activation.py:6-9).  gate and up are one product against
the stacked matrix [2 inner, width]; the reference runs two and concatenates (llama.py:23-26).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, compute_matrix, register_feed_forward
from .context import NormAhead, StepContext, UnscaledRows


class GatedMLP(FeedForward):
    def __init__(self, width: int, inner: int, activation: str, dtype: torch.dtype,
                 device: torch.device) -> None:
        super().__init__(dtype, device)
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation '{activation}' is not implemented; 'silu' is")
        self.width, self.inner = width, inner
        self.w_gate_up: "torch.Tensor | None" = None
        self.w_down: "torch.Tensor | None" = None

    def tensors(self):
        return {"gate_proj.weight": ((self.inner, self.width), "matrix"),
                "up_proj.weight": ((self.inner, self.width), "matrix"),
                "down_proj.weight": ((self.width, self.inner), "matrix")}

    def load(self, tensors):
        stacked = torch.cat((tensors["gate_proj.weight"], tensors["up_proj.weight"]), dim=0)
        self.w_gate_up = compute_matrix(stacked, self.dtype, self.device)
        self.w_down = compute_matrix(tensors["down_proj.weight"], self.dtype, self.device)

    def takes_unscaled(self, n_rows: int) -> bool:
        return ops.norm_ride_parts(n_rows, self.w_gate_up, self.dtype) > 0

    def ahead_parts(self, n_rows: int) -> int:
        return ops.norm_ride_parts(n_rows, self.w_down, self.dtype)

    def forward(self, x: "torch.Tensor | UnscaledRows", ctx: StepContext,
                ahead: "NormAhead | None" = None) -> "torch.Tensor | None":
        before = None
        if isinstance(x, UnscaledRows):
            before, x = x, x.rows
        n = x.shape[0]
        act = ctx.buffer("mlp.act", (n, self.inner))
        scratch = None
        if before is None and ops.gated_needs_scratch(x, self.w_gate_up):
            scratch = ctx.buffer("mlp.gate_up", (n, 2 * self.inner))
        ops.linear_gated(x, self.w_gate_up, act, scratch, status=ctx.status, before=before)
        if ahead is not None:          # the product joins the residual and does the next norm's work
            ops.linear(act, self.w_down, out=ahead.rows, status=ctx.status, after=ahead)
            return None
        out = ctx.buffer("mlp.out", (n, self.width))
        ops.linear(act, self.w_down, out=out, status=ctx.status)
        return out


register_feed_forward("gated_mlp", GatedMLP)
