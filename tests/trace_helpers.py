"""Builds replay traces (the JSON steps that bin/trace_run reads) for the ways of cutting that the
tests compare, and collects the logits a replay wrote."""

from __future__ import annotations

import io
import json
import os

import numpy as np


def _round64(n: int) -> int:
    return (n + 63) // 64 * 64


def schedule_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole: one step, every position wanted."""
    steps = []
    for rid, tokens in requests.items():
        steps.append({"step": len(steps), "end": [rid],
                      "entries": [{"id": rid, "tokens": tokens,
                                   "want": list(range(len(tokens)))}]})
    return steps


def schedule_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(len(tokens) - tail, 1)
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": tokens[:head],
                                   "want": list(range(head))}]})
        for i in range(head, len(tokens)):
            steps.append({"step": len(steps), "end": [rid] if i == len(tokens) - 1 else [],
                          "entries": [{"id": rid, "tokens": [tokens[i]], "want": [0]}]})
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def schedule_portions(requests: dict[str, list[int]],
                      sizes=(7, 2, 13, 1, 30, 17, 2, 3, 64, 5)) -> list[dict]:
    """Portions of changing size, down to two tokens and one."""
    steps = []
    for rid, tokens in requests.items():
        at, k = 0, 0
        while at < len(tokens):
            size = min(sizes[k % len(sizes)], len(tokens) - at)
            k += 1
            steps.append({"step": len(steps), "end": [rid] if at + size == len(tokens) else [],
                          "entries": [{"id": rid, "tokens": tokens[at: at + size],
                                       "want": list(range(size))}]})
            at += size
    return steps


def schedule_mixed(requests: dict[str, list[int]], max_tokens: int, seed: int = 0,
                   max_live: int = 4, decode_tail: int = 12) -> list[dict]:
    """Up to ``max_live`` live requests: portions of some beside single tokens of others, requests
    now and then left out of a step; a request is admitted only while the live ones, each rounded
    up to 64 tokens, fit into ``max_tokens`` - so pages are used again as requests end."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}                 # id -> tokens fed so far
    steps: list[dict] = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, tokens = waiting[0]
            held = sum(_round64(len(requests[r])) for r in live)
            if held + _round64(len(tokens)) > max_tokens:
                if not live:
                    raise ValueError(f"request '{rid}' alone exceeds max_tokens")
                break
            live[rid] = 0
            waiting.pop(0)
        entries, ended = [], []
        for rid in list(live):
            tokens, at = requests[rid], live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            left = len(tokens) - at
            if left <= decode_tail:
                size = 1
            else:
                size = int(min(rng.choice([2, 3, 5, 8, 16, 21, 33]), left - decode_tail))
            want = list(range(size)) if rng.random() < 0.8 else [size - 1]
            entries.append({"id": rid, "tokens": tokens[at: at + size], "want": want})
            live[rid] = at + size
            if live[rid] == len(tokens):
                ended.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def trace_text(steps: list[dict]) -> str:
    return "".join(json.dumps(s) + "\n" for s in steps)


def collect(steps: list[dict], out_dir: str, vocab: int) -> dict[tuple[str, int], np.ndarray]:
    """(request, position) -> logits row, from the files a replay wrote."""
    fed: dict[str, int] = {}
    rows: dict[tuple[str, int], np.ndarray] = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        data = None
        if wanted:
            data = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4")
            assert data.size == wanted * vocab, (s["step"], data.size, wanted, vocab)
            data = data.reshape(wanted, vocab)
        k = 0
        for e in s["entries"]:
            at = fed.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], at + w)] = data[k]
                k += 1
            fed[e["id"]] = at + len(e["tokens"])
        for rid in s["end"]:
            fed.pop(rid, None)
    return rows


def replay_in_process(runner, steps: list[dict], out_dir: str) -> None:
    from distengine_b200.engine.replay import replay
    replay(runner, io.StringIO(trace_text(steps)), out_dir, log=io.StringIO())
