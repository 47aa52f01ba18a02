"""Generation through the entry points against the plain implementation: greedy and temperature,
the reference's request sets (3 and 4 requests of different lengths), few pages with preemption,
the command line."""

import os
import subprocess
import sys

import pytest
import torch

import plain_llama as plain
import tiny_configs
from gpu_helpers import BF16_MAX_REL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_cache: dict = {}


def _setup(name, model_root):
    if name not in _cache:
        spec = tiny_configs.ALL[name]
        folder = tiny_configs.make_folder(name, model_root)
        config, weights = plain.load_model_folder(folder)
        prompts = [tiny_configs.prompt_tokens(name, n, i) for i, n in enumerate(spec["prompts"])]
        _cache[name] = (spec, folder, config, weights, prompts)
    return _cache[name]


def _engine(folder, spec, dtype, capacity_tokens=1024, budget=2048, seqs=4):
    from distengine_b200 import Engine, EngineConfig
    return Engine(folder, EngineConfig(dtype=dtype, block_size=spec["page_size"],
                                       num_blocks=capacity_tokens // spec["page_size"],
                                       decode_batch_size=seqs, max_batch_tokens=budget))


def _check_against_plain(config, weights, prompt, got, temperature, seed, dtype):
    """Equal tokens; in bfloat16 a different token is accepted only where the plain logits of the
    two candidates lie closer together than the bfloat16 bound (a near tie).  The comparison goes
    on after such a token: the plain path is always fed the engine's own tokens, so every later
    token is still checked against the logits of the sequence the engine really has."""
    tokens = list(prompt)
    for i, token in enumerate(got):
        logits = plain.plain_forward(config, weights, tokens, dtype)[-1]
        want = plain.plain_temperature_sample(logits, temperature, seed, len(tokens))
        if token != want:
            assert dtype == torch.bfloat16, f"token {i}: got {token}, the plain path gives {want}"
            assert temperature == 0.0
            gap = (logits[want] - logits[token]).item()
            assert 0 <= gap <= BF16_MAX_REL * logits.abs().max().item(), (i, token, want, gap)
        tokens.append(token)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_entry_point(name, dtype, model_root):
    spec, folder, config, weights, prompts = _setup(name, model_root)
    engine = _engine(folder, spec, dtype)
    got = engine.generate(prompts, spec["max_new_tokens"])
    assert [len(g) for g in got] == [spec["max_new_tokens"]] * len(prompts)
    for prompt, g in zip(prompts, got):
        _check_against_plain(config, weights, prompt, g, 0.0, 0, dtype)
    engine.cache.check_invariants()
    assert engine.cache.num_free_pages() == engine.cache.num_pages and not engine.has_pending()


@pytest.mark.parametrize("name,count", [("tiny_a", 24), ("tiny_d", 12)])
def test_many_requests_decode_together(name, count, model_root):
    """24 (12) requests at once in bfloat16: their decode steps are replayed graphs whose
    products are the kernels for 17 to 32 (9 to 16) tokens, with the norms in their epilogues."""
    spec, folder, config, weights, _ = _setup(name, model_root)
    prompts = [tiny_configs.prompt_tokens(name, 3 + (7 * i) % 40, 50 + i) for i in range(count)]
    engine = _engine(folder, spec, torch.bfloat16, capacity_tokens=4096, seqs=count)
    got = engine.generate(prompts, 10)
    assert [len(g) for g in got] == [10] * count
    for prompt, g in zip(prompts, got):
        _check_against_plain(config, weights, prompt, g, 0.0, 0, torch.bfloat16)
    engine.cache.check_invariants()
    assert engine.cache.num_free_pages() == engine.cache.num_pages and not engine.has_pending()


def test_temperature_generation_is_seeded_and_matches_plain(model_root):
    spec, folder, config, weights, prompts = _setup("tiny_b", model_root)
    engine = _engine(folder, spec, torch.float32)
    got = engine.generate(prompts, spec["max_new_tokens"], -1, spec["temperature"], seed=5)
    for i, (prompt, g) in enumerate(zip(prompts, got)):
        _check_against_plain(config, weights, prompt, g, spec["temperature"], 5 + i, torch.float32)
    # the same seeds give the same tokens whatever the batching: one request at a time, tiny budget
    alone = _engine(folder, spec, torch.float32, budget=7, seqs=1)
    again = alone.generate(prompts, spec["max_new_tokens"], -1, spec["temperature"], seed=5)
    assert again == got
    other = engine.generate(prompts, spec["max_new_tokens"], -1, spec["temperature"], seed=6)
    assert other != got


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_few_pages_preempt_and_still_give_the_same_tokens(dtype, model_root):
    spec, folder, config, weights, _ = _setup("tiny_a", model_root)
    prompts = [tiny_configs.prompt_tokens("tiny_a", n, 10 + i) for i, n in enumerate([20, 22, 24])]
    roomy = _engine(folder, spec, dtype).generate(prompts, 24)
    tight = _engine(folder, spec, dtype, capacity_tokens=96, budget=16, seqs=3)
    got = tight.generate(prompts, 24)
    assert tight.scheduler.num_preemptions >= 1
    if dtype == torch.float32:
        assert got == roomy
    for prompt, g in zip(prompts, got):
        _check_against_plain(config, weights, prompt, g, 0.0, 0, dtype)
    tight.cache.check_invariants()
    assert tight.cache.num_free_pages() == tight.cache.num_pages


def test_submit_step_interface_and_eos(model_root):
    spec, folder, config, weights, prompts = _setup("tiny_a", model_root)
    engine = _engine(folder, spec, torch.float32)
    first = plain.plain_generate(config, weights, prompts[1], 3)
    engine.submit("x", prompts[1], 8, eos_token_id=first[2])
    engine.submit("y", prompts[0], 2, eos_token_id=-1)
    with pytest.raises(ValueError):
        engine.submit("x", prompts[0], 2, -1)
    seen = []
    while engine.has_pending():
        seen += engine.step()
    records = {r["request_id"]: r for r in engine.drain_completed()}
    assert {r["request_id"] for r in seen} == {"x", "y"} and engine.drain_completed() == []
    assert records["x"] == {"request_id": "x", "prompt_token_ids": prompts[1],
                            "generated_token_ids": first, "status": "FINISHED", "reason": "eos"}
    assert records["y"]["reason"] == "length" and len(records["y"]["generated_token_ids"]) == 2


def test_a_step_started_ahead_is_taken_back_when_a_request_ends(model_root):
    """The engine starts the next decode step before it has seen this step's tokens.  A request
    that ends on an end-of-sequence token makes that step void for everyone: the others must go
    on from the right length and give the tokens they give alone."""
    spec, folder, config, weights, prompts = _setup("tiny_a", model_root)
    engine = _engine(folder, spec, torch.float32)
    alone = [plain.plain_generate(config, weights, p, 12) for p in prompts[:3]]
    # request 0 ends when it produces its 5th token; the token must not occur earlier in its output
    eos = alone[0][4]
    cut = alone[0].index(eos) + 1
    engine.submit("a", prompts[0], 12, eos_token_id=eos)
    engine.submit("b", prompts[1], 12, eos_token_id=-1)
    engine.submit("c", prompts[2], 12, eos_token_id=-1)
    launched_ahead = 0
    while engine.has_pending():
        engine.step()
        launched_ahead += engine._flying is not None
    records = {r["request_id"]: r for r in engine.drain_completed()}
    assert launched_ahead > 0
    assert records["a"]["generated_token_ids"] == alone[0][:cut] and records["a"]["reason"] == "eos"
    assert records["b"]["generated_token_ids"] == alone[1]
    assert records["c"]["generated_token_ids"] == alone[2]
    engine.cache.check_invariants()
    assert engine.cache.num_free_pages() == engine.cache.num_pages


def test_generate_greedy_function(model_root):
    from distengine_b200 import generate_greedy
    spec, folder, config, weights, prompts = _setup("tiny_a", model_root)
    out = generate_greedy(folder, torch.tensor([prompts[2]]), 5, -1, dtype="float32",
                          block_size=16, num_blocks=16)
    want = prompts[2] + plain.plain_generate(config, weights, prompts[2], 5)
    assert out.tolist() == [want]
    with pytest.raises(ValueError):
        generate_greedy(folder, torch.tensor(prompts[2]), 5, -1)


def test_command_line(model_root):
    spec, folder, config, weights, prompts = _setup("tiny_a", model_root)
    proc = subprocess.run(
        [sys.executable, "-m", "distengine_b200", "generate", "--model", folder, "--dtype",
         "float32", "--prompt-ids", " ".join(map(str, prompts[0])), "--prompt-ids",
         ",".join(map(str, prompts[1])), "--max-new-tokens", "4", "--num-blocks", "32"],
        capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("Generated token IDs:")]
    want = [plain.plain_generate(config, weights, p, 4) for p in prompts[:2]]
    assert lines == [f"Generated token IDs: {w}" for w in want]


def test_command_line_bench(model_root, tmp_path):
    """The request-level benchmark: the reference's smoke request set through the engine, twice;
    every request completes with its four tokens, the figures are consistent with one another, and
    an existing output folder is refused."""
    import json
    spec, folder, config, weights, prompts = _setup("tiny_a", model_root)
    out = tmp_path / "bench-out"
    command = [sys.executable, "-m", "distengine_b200", "bench", "--model", folder, "--dtype",
               "float32", "--repeats", "2", "--output", str(out), "--num-blocks", "64",
               "--block-size", str(spec["page_size"])]
    proc = subprocess.run(command, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert f"Saved {out / 'baseline.json'}" in proc.stdout
    report = json.loads((out / "baseline.json").read_text())
    assert report["executed_repeats"] == 2 and len(report["runs"]) == 2
    assert report["workload"]["prompt_lengths"] == [1, 8, 16]
    for run in report["runs"]:
        assert run["completed"] == 6 and run["output_tokens"] == 24
        assert run["completed_output_tokens_per_s"] == pytest.approx(24 / run["elapsed_s"])
        for row in run["per_request"].values():
            assert row["output_tokens"] == 4
            assert 0 < row["ttft_s"] <= row["e2e_s"] and row["tpot_s"] >= 0
        assert run["latencies"]["e2e_s"]["p50"] <= run["latencies"]["e2e_s"]["p99"]
    assert report["aggregate"]["request_throughput_rps"]["mean"] > 0
    again = subprocess.run(command, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert again.returncode != 0 and "Choose a new output directory" in again.stderr


def test_no_cpu_path():
    from distengine_b200.kernels import KernelsUnavailable
    from distengine_b200.models import load_model
    with pytest.raises(KernelsUnavailable):
        load_model("/nonexistent", "float32", "cpu")
