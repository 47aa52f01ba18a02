"""RMS norm with the residual sum folded in.

Formula (src/layers/layernorm.py:12-23): float32 mean of squares, x * rsqrt(mean + eps), cast to
the activation dtype, then times the weight.  The block's residual sums
(src/models/llama.py:74-89) happen in the same kernel, in 32-bit.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, register_norm, stored_vector
from .context import NormAhead, ResidualStream, StepContext


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype, device)
        self.width, self.eps = width, eps
        self.weight: "torch.Tensor | None" = None

    def tensors(self):
        return {"weight": ((self.width,), "vector")}

    def load(self, tensors):
        self.weight = stored_vector(tensors["weight"], self.dtype, self.device)

    def ahead(self, stream: ResidualStream, ctx: StepContext, count: int):
        if self.weight.dtype != torch.bfloat16 or stream.pending is not None:
            return None
        n = stream.resid.shape[0]
        return NormAhead(self, stream.resid, self.weight, self.eps,
                         ctx.buffer("norm.out", (n, self.width)),
                         ctx.buffer("norm.parts", (n, count), torch.float32))

    def forward(self, stream: ResidualStream, ctx: StepContext, rows=None,
                out_name: str = "norm.out") -> torch.Tensor:
        if stream.ahead is not None:
            raise RuntimeError("this norm's work was handed to the product before it: its "
                               "result is stream.ahead.result()")
        n_out = stream.resid.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (n_out, self.width))
        ops.add_rmsnorm(stream.resid, stream.pending, self.weight, self.eps, out, rows)
        if rows is None:
            stream.pending = None              # it is part of the residual now
        return out


register_norm("rmsnorm", RMSNorm)
