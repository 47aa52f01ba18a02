"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the model through
the registry and drives the same ``StepRunner``, ``CacheManager`` and kernels that generation uses.

Input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 [wanted, vocab].
After every step a line ``done <step>`` is printed and flushed.  Requests named in ``end`` give
back what they hold after the step.

The reference has no such program; its relatives are ``generate_greedy_cached`` (feeds a prompt,
then its own samples: src/utils/generation.py:34-39) and ``replay_workload`` (replays timed
arrivals: src/distengine/workload.py:233-324).
"""

from __future__ import annotations

import json
import os
import sys
from typing import IO

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.engine import parse_dtype
from ..models.loading import load_model
from .step import StepEntry, StepRunner

LIVE_REQUESTS = 8          # slots; a trace holds up to four live requests


def build_runner(model_dir: str, dtype: "str | torch.dtype", max_tokens: int,
                 page_size: int = 16, device: str = "cuda:0",
                 poison_freed_pages: bool = False, use_graphs: bool = False,
                 live_requests: int = LIVE_REQUESTS) -> StepRunner:
    """Model, cache for ``max_tokens`` tokens (in pages of ``page_size``) and the step runner.
    ``use_graphs``: steps of single tokens are replayed as CUDA graphs, as the engine does;
    ``live_requests``: slots, the most requests that are live at a time."""
    dtype = parse_dtype(dtype)
    model = load_model(model_dir, dtype, device)
    if max_tokens <= 0:
        raise ValueError("--max-tokens must be positive")
    num_pages = (max_tokens + page_size - 1) // page_size
    max_len = min(model.config.max_positions, num_pages * page_size)
    cache = CacheManager(model.cache_specs(), [e.reads_cache_of for e in model.plan], page_size,
                         num_pages, live_requests, max_len, dtype, model.device,
                         poison_freed_pages=poison_freed_pages)
    return StepRunner(model, cache, use_graphs=use_graphs)


def replay(runner: StepRunner, lines: IO[str], out_dir: str, log: IO[str] = sys.stdout) -> None:
    os.makedirs(out_dir, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(str(e["id"]), [int(t) for t in e["tokens"]],
                             [int(w) for w in e.get("want", [])])
                   for e in record.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            wanted = sum(len(e.want) for e in entries)
            runner.check_status()
            if wanted:
                host = logits.to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                host.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for request_id in record.get("end", []):
            runner.release(str(request_id))
        print(f"done {step}", file=log, flush=True)
