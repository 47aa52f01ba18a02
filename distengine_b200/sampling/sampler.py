"""Sampling the next token of each finished portion: greedy and temperature.

Greedy is the reference's only sampler: arg-max over the vocabulary
(src/layers/sampler.py:5-8); the lowest id wins a tie.  Temperature sampling draws from
softmax(logits / T), computed in 32-bit, by the Gumbel-max rule with counter-based uniforms of
(seed, position of the sampled token, token id): a request's draws depend on its own seed and
position only, not on the batch it shares or on how its prompt was cut.  Temperature 0 is greedy.
Both run in one kernel over the step's logits rows; the sampled ids come back in one small copy,
and with them the status word in which the step's kernels record work that they had to skip.
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops


def pack_sampling(temperatures: list[float], seeds: list[int], positions: list[int]):
    """int32 arrays that carry float32 temperatures, int64 seeds and int32 positions to the
    device inside the step's upload, or None when every row is greedy."""
    if not any(t > 0.0 for t in temperatures):
        return None
    t = np.asarray(temperatures, dtype=np.float32).view(np.int32)
    s = np.asarray([np.int64(x) for x in seeds], dtype=np.int64).view(np.int32)
    p = np.asarray(positions, dtype=np.int32)
    return {"sampling/temperature": t, "sampling/seed": s, "sampling/position": p}


class Sampler:
    """Two launches may be outstanding (the engine starts the next step before it has read this
    step's ids): the ids travel to the host through two pinned buffers in turn.

    ``status`` (int32 [1]) lies directly before ``ids`` in one device buffer, so that one copy
    brings both to the host: a step runner that is given it as its status word has its kernels'
    complaints read at every step without a synchronisation of their own (``last_status``)."""

    def __init__(self, device: torch.device, max_rows: int) -> None:
        self.device = device
        self.max_rows = max_rows
        self._buffer = torch.zeros(max_rows + 1, dtype=torch.int32, device=device)
        self.status = self._buffer[:1]
        self.ids = self._buffer[1:]
        self.host_ids = [torch.zeros(max_rows + 1, dtype=torch.int32).pin_memory()
                         for _ in range(2)]
        self._done = [torch.cuda.Event(), torch.cuda.Event()]
        self._turn = 0
        self._last = (0, 0)
        self.last_status = 0

    def launch(self, logits: torch.Tensor,
               arrays: "dict[str, torch.Tensor] | None") -> "tuple[int, int]":
        """Start sampling the rows of ``logits`` [R, V] and the copy of the ids to the host;
        returns a ticket for ``wait``.  The ids also stay on the device (``self.ids[:R]``) until
        the next launch, for a step that is started before the host has seen them."""
        rows = logits.shape[0]
        self._turn ^= 1
        turn = self._turn
        self._last = (turn, rows)
        if rows == 0:
            return self._last
        if rows > self.max_rows:
            raise ValueError(f"the sampler was made for {self.max_rows} rows a step, got {rows}")
        out = self.ids[:rows]
        if arrays and "sampling/temperature" in arrays:
            ops.sample_rows(logits, out, arrays["sampling/temperature"].view(torch.float32),
                            arrays["sampling/seed"].view(torch.int64),
                            arrays["sampling/position"])
        else:
            ops.sample_rows(logits, out)
        self.host_ids[turn][: rows + 1].copy_(self._buffer[: rows + 1], non_blocking=True)
        self._done[turn].record()
        return self._last

    def wait(self, ticket: "tuple[int, int] | None" = None) -> list[int]:
        """The ids of a launch (the last one by default); synchronises with it."""
        turn, rows = ticket or self._last
        if rows == 0:
            return []
        self._done[turn].synchronize()
        values = self.host_ids[turn][: rows + 1].tolist()
        self.last_status = values[0]
        return values[1:]

    def sample(self, logits: torch.Tensor, arrays: "dict[str, torch.Tensor] | None") -> list[int]:
        """Token ids for the rows of ``logits`` [R, V]; synchronises to bring them to the host."""
        return self.wait(self.launch(logits, arrays))
