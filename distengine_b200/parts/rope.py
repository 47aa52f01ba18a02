"""Rotary position encoding, default kind.

inv_freq[i] = 1 / theta^(2i / rotary_dim) in float32 (src/layers/rotary_embedding.py:14-15); the
angle float(position) * inv_freq[i], its cosine and sine are float32 and are formed inside the
kernel that also stores k and v (``kernels.ops.rope_kv_write``); pairing is half-split, feature j
with j + rotary_dim / 2 (:45-54).  ``rotary_dim`` below the head size leaves the upper features
unrotated; ``NoPositionEncoding`` rotates nothing.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding


class RotaryPositionEncoding(PositionEncoding):
    def __init__(self, rotary_dim: int, theta: float, dtype: torch.dtype,
                 device: torch.device) -> None:
        super().__init__(dtype, device)
        if rotary_dim <= 0 or rotary_dim % 2 != 0:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        self.rotary_dim, self.theta = rotary_dim, float(theta)
        indices = torch.arange(0, rotary_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (indices / rotary_dim))).to(device)

    def rotation_table(self):
        return self.inv_freq, self.rotary_dim


class NoPositionEncoding(PositionEncoding):
    def __init__(self, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype, device)


register_position_encoding("rope", RotaryPositionEncoding)
register_position_encoding("none", NoPositionEncoding)
