"""From a model folder to a model on the device: config.json picks the architecture, the weights
are read by name and checked against what the built parts expect."""

from __future__ import annotations

import torch

from ..config.engine import parse_dtype
from ..kernels.ops import require_device
from ..registry import read_config
from ..weights.loader import load_checked


def load_model(model_dir: str, dtype: "str | torch.dtype" = torch.bfloat16,
               device: "str | torch.device" = "cuda:0"):
    dtype = parse_dtype(dtype)
    device = require_device(device)
    architecture, config = read_config(model_dir)
    model = architecture.build_model(config, dtype, device)
    expected, _, optional = model.expected_tensors()
    tensors = load_checked(model_dir, expected, optional, dtype)
    model.load(tensors)
    return model
