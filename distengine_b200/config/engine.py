"""Settings of the engine itself (not of the model).

The reference scatters these as keyword arguments: ``num_blocks`` and ``block_size``
(src/distengine/worker.py:533-534, src/Modal/run_benchmark.py:93-94), ``decode_batch_size``
(src/distengine/coordinator.py:47).  Names are kept where the reference has them.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def parse_dtype(name: "str | torch.dtype") -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[name.lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got '{name}'") from None


@dataclass
class EngineConfig:
    dtype: torch.dtype = torch.bfloat16
    block_size: int = 16                 # tokens in one page of the cache
    num_blocks: int | None = None        # pages in every cache group's pool; None: from memory_fraction
    memory_fraction: float = 0.8         # share of free device memory given to the pools
    decode_batch_size: int = 64          # most requests that are live at a time (slots)
    max_batch_tokens: int = 2048         # token budget of one step
    max_model_len: int | None = None     # longest request; None: the model's max positions
    use_graphs: bool = True              # replay decode steps as CUDA graphs
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        self.dtype = parse_dtype(self.dtype)
        for name in ("block_size", "decode_batch_size", "max_batch_tokens"):
            value = getattr(self, name)
            if type(value) is not int or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if self.num_blocks is not None and (type(self.num_blocks) is not int
                                            or self.num_blocks <= 0):
            raise ValueError("num_blocks must be a positive integer")
        if 64 % self.block_size != 0:
            raise ValueError("block_size must divide 64 (1, 2, 4, 8, 16, 32 or 64)")
