"""Replay of the same requests cut in every way, in 32-bit and in bfloat16, against the plain
implementation: whole; most in one step and the last 32 tokens one by one; portions of changing
size down to two tokens; mixed with other requests on so few pages that they are used again."""

import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_llama as plain
import tiny_configs
import trace_helpers as th
from gpu_helpers import assert_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
LENGTHS = [70, 33, 100, 5, 64, 17, 90, 48, 1, 2]

_cache: dict = {}


def _model(name, model_root):
    if name not in _cache:
        folder = tiny_configs.make_folder(name, model_root)
        config, weights = plain.load_model_folder(folder)
        limit = config["max_position_embeddings"]
        requests = {f"r{i}": tiny_configs.prompt_tokens(name, min(n, limit), i)
                    for i, n in enumerate(LENGTHS)}
        reference = {}
        for dtype in DTYPES.values():
            reference[dtype] = {rid: plain.plain_forward(config, weights, t, dtype).numpy()
                                for rid, t in requests.items()}
        _cache[name] = (folder, config, requests, reference)
    return _cache[name]


def _schedules(requests):
    return {
        "whole": (th.schedule_whole(requests), 128),
        "tail": (th.schedule_tail(requests, 32), 128),
        "portions": (th.schedule_portions(requests), 128),
        "mixed": (th.schedule_mixed(requests, 320, seed=3), 320),
        "mixed_tight": (th.schedule_mixed(requests, 192, seed=11, decode_tail=32), 192),
    }


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed", "mixed_tight"])
def test_replay_matches_plain(name, dtype_name, schedule, model_root):
    from distengine_b200.engine.replay import build_runner
    folder, config, requests, reference = _model(name, model_root)
    dtype = DTYPES[dtype_name]
    steps, max_tokens = _schedules(requests)[schedule]
    runner = build_runner(folder, dtype_name, max_tokens,
                          page_size=tiny_configs.ALL[name]["page_size"],
                          poison_freed_pages=True)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, config["vocab_size"])
    assert rows
    runner.cache.check_invariants()
    assert not runner.cache.live and runner.cache.num_free_pages() == runner.cache.num_pages
    for rid in requests:
        positions = sorted(p for r, p in rows if r == rid)
        got = np.stack([rows[(rid, p)] for p in positions])
        assert_close(got, reference[dtype][rid][positions], dtype, f"{name} {schedule} {rid}")


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_trace_run_program(dtype_name, model_root):
    """The program itself, as a user calls it: standard input, files, 'done' lines, exit 0."""
    folder, config, requests, reference = _model("tiny_a", model_root)
    steps, max_tokens = _schedules(requests)["mixed"]
    with tempfile.TemporaryDirectory() as out:
        proc = subprocess.run(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype",
             dtype_name, "--out", out, "--max-tokens", str(max_tokens)],
            input=th.trace_text(steps), capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
        assert done == [f"done {s['step']}" for s in steps]
        rows = th.collect(steps, out, config["vocab_size"])
    dtype = DTYPES[dtype_name]
    for (rid, pos), got in rows.items():
        assert_close(got, reference[dtype][rid][pos], dtype, f"trace_run {rid}@{pos}")


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_cuts_agree_with_each_other(dtype_name, model_root):
    """Logits at a position do not depend on the cut beyond rounding: in float32 the ways of
    cutting agree far more closely with each other than the bound against the plain
    implementation asks."""
    from distengine_b200.engine.replay import build_runner
    folder, config, requests, _ = _model("tiny_b", model_root)
    results = {}
    for schedule in ("whole", "tail", "portions", "mixed"):
        steps, max_tokens = _schedules(requests)[schedule]
        runner = build_runner(folder, dtype_name, max_tokens, page_size=8)
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            results[schedule] = th.collect(steps, out, config["vocab_size"])
    base = results["whole"]
    for schedule, rows in results.items():
        for key, got in rows.items():
            assert_close(got, base[key], DTYPES[dtype_name], f"{schedule} against whole {key}")


@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
def test_persistent_decode_kernel_matches_plain(name, model_root):
    """The optional single-kernel decode step (csrc/decode_fused.cu): steps of single tokens go
    through it, everything else through the kernels of the parts; same logits."""
    from distengine_b200.engine.replay import build_runner
    folder, config, requests, reference = _model(name, model_root)
    dtype = torch.bfloat16
    used = 0
    for schedule in ("tail", "mixed"):
        steps, max_tokens = _schedules(requests)[schedule]
        runner = build_runner(folder, "bfloat16", max_tokens,
                              page_size=tiny_configs.ALL[name]["page_size"],
                              poison_freed_pages=True, use_fused=True)
        assert runner.fused is not None
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            rows = th.collect(steps, out, config["vocab_size"])
        used += runner.fused_steps
        for rid in requests:
            positions = sorted(p for r, p in rows if r == rid)
            got = np.stack([rows[(rid, p)] for p in positions])
            assert_close(got, reference[dtype][rid][positions], dtype, f"{name} fused {schedule} {rid}")
    assert used > 50
