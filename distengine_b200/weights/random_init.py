"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

Matrices, the embedding table and the output matrix are N(0, 0.02) as the reference initialises
them (src/layers/linear.py:12, src/layers/embed_head.py:10,20); norm weights are ones
(src/layers/layernorm.py:9) or, on request, U(0.5, 1.5) so that a test sees whether the norm's
weight is applied.  Values are drawn in float32 from one seeded generator in the order of the
tensor names, then stored in the asked dtype, so a folder is reproducible from (configuration,
seed, norm_init, dtype) alone.
"""

from __future__ import annotations

import json
import os
from typing import Any, Mapping

import torch

from ..registry import resolve
from .safetensors_io import save_tensors


def random_tensors(expected: dict[str, tuple[int, ...]], vectors: set[str], seed: int,
                   norm_init: str = "ones", std: float = 0.02,
                   dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    if norm_init not in ("ones", "uniform"):
        raise ValueError("norm_init must be 'ones' or 'uniform'")
    generator = torch.Generator(device="cpu")
    generator.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name, shape in expected.items():
        if name in vectors:
            if norm_init == "ones":
                value = torch.ones(shape, dtype=torch.float32)
            else:
                value = torch.rand(shape, generator=generator, dtype=torch.float32) + 0.5
        else:
            value = torch.randn(shape, generator=generator, dtype=torch.float32) * std
        out[name] = value.to(dtype)
    return out


def write_random_model(config_json: Mapping[str, Any], out_dir: str, seed: int,
                       dtype: "str | torch.dtype" = torch.float32,
                       norm_init: str = "ones") -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns ``out_dir``."""
    from ..config.engine import parse_dtype
    from ..models.decoder import expected_tensors

    store = parse_dtype(dtype)
    _, config = resolve(config_json)
    expected, vectors, optional = expected_tensors(config)
    names = {name: shape for name, shape in expected.items() if name not in optional}
    tensors = random_tensors(names, vectors, seed, norm_init=norm_init, dtype=store)
    os.makedirs(out_dir, exist_ok=True)
    text = dict(config.to_json())
    text["torch_dtype"] = "bfloat16" if store == torch.bfloat16 else "float32"
    with open(os.path.join(out_dir, "config.json"), "w") as handle:
        json.dump(text, handle, indent=2)
    save_tensors(os.path.join(out_dir, "model.safetensors"), tensors)
    return out_dir
