"""Weights by tensor name, with one error that lists everything that is wrong.

The names on disk are the reference's module paths (``model.embed_tokens.weight``,
``model.layers.{i}.self_attn.q_proj.weight`` ... ``lm_head.weight``; structure at
src/models/llama.py:17-19,44-64,96,126,201 and src/layers/attention.py:95-98).  The reference loads
with ``load_state_dict(strict=True)`` (src/utils/load_model.py:18), which also refuses missing and
unexpected names and wrong shapes; here all of them are collected into one ``WeightMismatchError``,
together with tensors of the wrong class of dtype (integers or booleans where a matrix or a norm
weight is expected, floating point where an integer table is), which a strict load refuses too.

Dtypes: a tensor stays as it is stored (bfloat16 stays bfloat16, a tensor stored in 32-bit stays
32-bit, float16 becomes bfloat16, integer tables become int32).  What a matrix product multiplies is
converted to the compute dtype by the part that packs it (``Part.load``); small vectors are used as
stored.  With ``dtype=float32`` every floating tensor is widened to float32: the true 32-bit path.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .safetensors_io import open_model_files

# tensors that a file may hold and no model needs (buffers that some exporters write)
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


@dataclass
class WeightMismatchError(Exception):
    missing: list[str] = field(default_factory=list)
    unexpected: list[str] = field(default_factory=list)
    wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]] = field(default_factory=list)
    wrong_dtype: list[tuple[str, str, str]] = field(default_factory=list)   # name, wanted, stored
    where: str = ""

    def __str__(self) -> str:
        lines = [f"weights in {self.where or 'the model folder'} do not fit the configuration:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{name}: expected {list(want)}, file has {list(got)}"
                for name, want, got in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{name}: expected {want}, file has {got}"
                for name, want, got in self.wrong_dtype))
        return "\n".join(lines)


def stored_dtype_policy(tensor: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The dtype a loaded tensor is kept in (see the module's header)."""
    if tensor.dtype.is_floating_point:
        if dtype == torch.float32:
            return tensor.to(torch.float32)
        if tensor.dtype in (torch.float32, torch.bfloat16):
            return tensor
        if tensor.dtype == torch.float64:
            return tensor.to(torch.float32)
        return tensor.to(torch.bfloat16)
    if tensor.dtype == torch.bool:
        return tensor
    return tensor.to(torch.int32)


def load_checked(model_dir: str, expected: dict[str, tuple[int, ...]],
                 optional: set[str] = frozenset(), dtype: torch.dtype = torch.bfloat16,
                 integer: set[str] = frozenset()) -> dict[str, torch.Tensor]:
    """Every tensor of ``expected`` (name -> shape) from the folder's safetensors files.

    ``optional`` names may be absent (a tied output matrix).  ``integer`` names are integer
    tables; every other tensor must be stored in a floating-point dtype.  Raises
    ``WeightMismatchError`` with all missing and unexpected names, wrong shapes and wrong dtypes
    at once.  Tensors come back on the host.
    """
    found: dict[str, torch.Tensor] = {}
    error = WeightMismatchError(where=model_dir)
    for handle in open_model_files(model_dir):
        for name in handle.names():
            if name.endswith(IGNORED_SUFFIXES):
                continue
            if name not in expected:
                error.unexpected.append(name)
                continue
            shape = handle.shape(name)
            if tuple(shape) != tuple(expected[name]):
                error.wrong_shape.append((name, tuple(expected[name]), tuple(shape)))
                continue
            stored = handle.dtype(name)
            if name in integer:
                if stored.is_floating_point or stored == torch.bool:
                    error.wrong_dtype.append((name, "an integer dtype", str(stored)))
                    continue
            elif not stored.is_floating_point:
                error.wrong_dtype.append((name, "a floating-point dtype", str(stored)))
                continue
            found[name] = stored_dtype_policy(handle.tensor(name), dtype)
    wrong = {name for name, _, _ in error.wrong_shape} | {name for name, _, _ in error.wrong_dtype}
    error.missing = [name for name in expected
                     if name not in found and name not in wrong and name not in optional]
    if error.missing or error.unexpected or error.wrong_shape or error.wrong_dtype:
        error.missing.sort()
        error.unexpected.sort()
        raise error
    return found
