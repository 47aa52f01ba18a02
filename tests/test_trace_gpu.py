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


LONG = dict(architectures=["LlamaForCausalLM"], vocab_size=211, hidden_size=120,
            intermediate_size=136, num_hidden_layers=2, num_attention_heads=6,
            num_key_value_heads=1, head_dim=48, rms_norm_eps=1e-5, rope_theta=1.0e6,
            max_position_embeddings=6144, tie_word_embeddings=True)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_long_context_then_decoding(dtype_name, model_root):
    """4,500 tokens of context, fed in portions, then 24 tokens one by one: the decode steps cut
    the key range into so many chunks that one thread-block cluster does not cover them (its
    partial results are merged through global memory), prompt portions read thousands of keys
    through the block table, and the pages of a second, short request lie in between."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.kernels.attention_plan import choose_decode_split
    from distengine_b200.weights import write_random_model
    dtype = DTYPES[dtype_name]
    folder = write_random_model(LONG, f"{model_root}/long-context", seed=21, norm_init="uniform")
    config, weights = plain.load_model_folder(folder)
    rng = np.random.default_rng(8)
    requests = {"long": [int(t) for t in rng.integers(0, 211, size=4524)],
                "short": [int(t) for t in rng.integers(0, 211, size=40)]}
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert choose_decode_split(1, 1, 4608, sm_count=sms)[1] > 1          # more than one cluster a tile
    want = {rid: plain.plain_forward(config, weights, ids, dtype).numpy()
            for rid, ids in requests.items()}
    steps, at = [], 0
    long_ids, short_ids = requests["long"], requests["short"]
    for i, size in enumerate([1024, 20, 1500, 700, 1256]):        # 4,500 tokens in portions
        entries = [{"id": "long", "tokens": long_ids[at: at + size], "want": [size - 1]}]
        if i == 1:
            entries.append({"id": "short", "tokens": short_ids[:30], "want": [29]})
        steps.append({"step": len(steps), "entries": entries, "end": []})
        at += size
    for i in range(24):                                             # then token by token
        entries = [{"id": "long", "tokens": [long_ids[at]], "want": [0]}]
        if i < 10:
            entries.append({"id": "short", "tokens": [short_ids[30 + i]], "want": [0]})
        steps.append({"step": len(steps), "entries": entries,
                      "end": ["short"] if i == 9 else (["long"] if i == 23 else [])})
        at += 1
    runner = build_runner(folder, dtype_name, 4608 + 64, page_size=32, poison_freed_pages=True)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, 211)
    assert len(rows) == 5 + 1 + 24 + 10
    for (rid, pos), got in rows.items():
        assert_close(got, want[rid][pos], dtype, f"long context {rid}@{pos}")
    runner.cache.check_invariants()
    assert not runner.cache.live and runner.cache.num_free_pages() == runner.cache.num_pages


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


@pytest.mark.parametrize("name", ["tiny_b", "tiny_c"])
def test_float32_cuts_agree_bit_for_bit(name, model_root):
    """In float32 the logits at a position are the same bits however the tokens were cut into
    steps and whatever else was in the batch, with and without CUDA graphs: every kernel of the
    32-bit path sums a row's terms in an order that depends on the row alone (the matrix product
    over k in ascending order, the attention over tiles of 32 keys at absolute positions within
    chunks of a fixed length, chunks in ascending order).  One request is 1,300 tokens long, so
    that its key ranges span three chunks."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.kernels.attention import F32_CHUNK
    from distengine_b200.weights import write_random_model
    spec = tiny_configs.ALL[name]
    shape = dict(spec["config"], max_position_embeddings=2048)
    folder = write_random_model(shape, f"{model_root}/{name}-2048-positions", spec["seed"],
                                dtype="float32", norm_init=spec["norm_init"])
    vocab = shape["vocab_size"]
    requests = {f"r{i}": tiny_configs.prompt_tokens(name, n, i)
                for i, n in enumerate([70, 2 * F32_CHUNK + 276, 33, 100, 5])}
    cuts = {
        "whole": (th.schedule_whole(requests), 1408),
        "tail": (th.schedule_tail(requests, 32), 1408),
        "portions": (th.schedule_portions(requests, sizes=(7, 2, 130, 1, 300, 17, 2, 3, 64, 5)),
                     1408),
        "mixed": (th.schedule_mixed(requests, 1600, seed=3), 1600),
    }
    results = {}
    for schedule, graphs in (("whole", False), ("tail", False), ("tail", True), ("portions", False),
                             ("mixed", False), ("mixed", True)):
        steps, max_tokens = cuts[schedule]
        runner = build_runner(folder, "float32", max_tokens, page_size=spec["page_size"],
                              use_graphs=graphs)
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            results[(schedule, graphs)] = th.collect(steps, out, vocab)
        if graphs:
            assert runner.graph_replays > 0
    base = results[("whole", False)]
    for key, rows in results.items():
        assert rows
        for place, got in rows.items():
            assert np.array_equal(got, base[place]), f"{key} differs from whole at {place}"


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_bfloat16_engine_against_the_reference_run_in_bfloat16(name, model_root):
    """Anchors the bfloat16 path on the reference itself and not only on the plain
    implementation's rounding model: the logits that the reference's own modules gave when cast
    to bfloat16 on the CPU (tests/golden, made by make_golden.py) against the engine's, for the
    sequence whole and with its last 32 tokens fed one by one.  The engine adds the residual
    stream in float32 where the reference adds in bfloat16; the bound is the bfloat16 bound."""
    from distengine_b200.engine.replay import build_runner
    folder = tiny_configs.make_folder(name, model_root, dtype="float32")
    golden = np.load(os.path.join(ROOT, "tests", "golden", f"{name}.npz"))
    ids = [int(t) for t in golden["token_ids"]]
    requests = {"g": ids}
    for steps in (th.schedule_whole(requests), th.schedule_tail(requests, 32)):
        runner = build_runner(folder, "bfloat16", 128,
                              page_size=tiny_configs.ALL[name]["page_size"])
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            rows = th.collect(steps, out, golden["logits"].shape[1])
        got = np.stack([rows[("g", p)] for p in range(len(ids))])
        assert_close(got, golden["logits_bf16"], torch.bfloat16, f"{name} against the reference "
                     "in bfloat16")


def test_bfloat16_cuts_agree_with_each_other(model_root):
    """bfloat16 steps of different shapes take different kernels (tile shapes, products), so the
    cuts agree within the bfloat16 bound, not bit for bit."""
    from distengine_b200.engine.replay import build_runner
    folder, config, requests, _ = _model("tiny_b", model_root)
    results = {}
    for schedule in ("whole", "tail", "portions", "mixed"):
        steps, max_tokens = _schedules(requests)[schedule]
        runner = build_runner(folder, "bfloat16", max_tokens, page_size=8)
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            results[schedule] = th.collect(steps, out, config["vocab_size"])
    base = results["whole"]
    for schedule, rows in results.items():
        for key, got in rows.items():
            assert_close(got, base[key], torch.bfloat16, f"{schedule} against whole {key}")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["tail", "mixed", "mixed_tight"])
def test_replay_with_graphs_matches_plain(name, dtype_name, schedule, model_root):
    """The same traces with steps of single tokens replayed as CUDA graphs, as the engine runs
    them: graphed and ungraphed decode steps are both under every cut."""
    from distengine_b200.engine.replay import build_runner
    folder, config, requests, reference = _model(name, model_root)
    dtype = DTYPES[dtype_name]
    steps, max_tokens = _schedules(requests)[schedule]
    runner = build_runner(folder, dtype_name, max_tokens,
                          page_size=tiny_configs.ALL[name]["page_size"],
                          poison_freed_pages=True, use_graphs=True)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, config["vocab_size"])
    assert runner.graph_replays > 0
    runner.cache.check_invariants()
    for rid in requests:
        positions = sorted(p for r, p in rows if r == rid)
        got = np.stack([rows[(rid, p)] for p in positions])
        assert_close(got, reference[dtype][rid][positions], dtype,
                     f"{name} graphs {schedule} {rid}")


@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_steps_with_prompt_portions_of_a_shape_seen_before_are_replayed(name, dtype_name,
                                                                        model_root):
    """A step with prompt portions is replayed as a CUDA graph once its shape (the portions'
    lengths, the cap on positions, the wanted rows) has come a few times: eight prompts of 70
    tokens, one a step, on pages that are used again; then seven steps of two new prompts each
    (40 and 9 tokens); then a prompt of 105 tokens in seven portions of 15.  Every logit row
    against the plain implementation; in 32-bit also bit for bit against the same trace without
    graphs."""
    from distengine_b200.engine.replay import build_runner
    folder, config, _, _ = _model(name, model_root)
    dtype = DTYPES[dtype_name]
    prompts, steps = {}, []

    def step(entries, end):
        steps.append({"step": len(steps), "entries": entries, "end": end})

    for i in range(8):
        prompts[f"a{i}"] = tiny_configs.prompt_tokens(name, 70, 20 + i)
        step([{"id": f"a{i}", "tokens": prompts[f"a{i}"], "want": [0, 35, 69]}], [f"a{i}"])
    for i in range(7):
        prompts[f"b{i}"] = tiny_configs.prompt_tokens(name, 40, 40 + i)
        prompts[f"c{i}"] = tiny_configs.prompt_tokens(name, 9, 60 + i)
        step([{"id": f"b{i}", "tokens": prompts[f"b{i}"], "want": [39]},
              {"id": f"c{i}", "tokens": prompts[f"c{i}"], "want": [0, 8]}], [f"b{i}", f"c{i}"])
    prompts["d"] = tiny_configs.prompt_tokens(name, 105, 80)
    for part in range(7):
        step([{"id": "d", "tokens": prompts["d"][15 * part: 15 * part + 15], "want": [14]}],
             ["d"] if part == 6 else [])
    results = {}
    for graphs in (True, False):
        runner = build_runner(folder, dtype_name, 128,
                              page_size=tiny_configs.ALL[name]["page_size"],
                              poison_freed_pages=True, use_graphs=graphs)
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            results[graphs] = th.collect(steps, out, config["vocab_size"])
        runner.cache.check_invariants()
        if graphs:
            # a shape's first three steps run as they are, the fourth shaped for replay, the
            # fifth is captured and replayed
            assert runner.graph_replays == 4 + 3 + 3
    weights = plain.load_model_folder(folder)[1]
    for (rid, position), got in results[True].items():
        want = plain.plain_forward(config, weights, prompts[rid], dtype).numpy()[position]
        assert_close(got[None], want[None], dtype, f"{name} graphed portions {rid} {position}")
        if dtype_name == "float32":
            assert np.array_equal(got, results[False][(rid, position)]), (rid, position)


@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "portions", "mixed_tight"])
def test_replay_at_head_sizes_64_and_128(name, dtype_name, schedule, model_root):
    """The head sizes of the full-size Llama models: in bfloat16 their prompt portions go through
    the tensor-memory attention kernel (two row tiles a block at 64, one at 128)."""
    from distengine_b200.engine.replay import build_runner
    folder, config, requests, reference = _model(name, model_root)
    dtype = DTYPES[dtype_name]
    steps, max_tokens = _schedules(requests)[schedule]
    runner = build_runner(folder, dtype_name, max_tokens,
                          page_size=tiny_configs.ALL[name]["page_size"], poison_freed_pages=True)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, config["vocab_size"])
    assert rows
    runner.cache.check_invariants()
    for rid in requests:
        positions = sorted(p for r, p in rows if r == rid)
        got = np.stack([rows[(rid, p)] for p in positions])
        assert_close(got, reference[dtype][rid][positions], dtype, f"{name} {schedule} {rid}")


WIDE = dict(architectures=["LlamaForCausalLM"], vocab_size=203, hidden_size=2048,
            intermediate_size=1024, num_hidden_layers=2, num_attention_heads=32,
            num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0,
            max_position_embeddings=4096, tie_word_embeddings=False)


def test_a_prompt_of_2048_tokens_at_full_width():
    """Layers as wide as the benchmark's, two of them, a prompt of 2,100 tokens fed whole and
    then cut in two ways, then eight tokens one by one: the portions' products are the tcgen05
    kernels at the sizes they were made for, the single tokens' the weight-streaming ones with
    the norms in their epilogues; logits against the plain implementation at a few positions."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.weights import write_random_model
    with tempfile.TemporaryDirectory() as root:
        folder = write_random_model(WIDE, f"{root}/wide", seed=5, norm_init="uniform")
        config, weights = plain.load_model_folder(folder)
        rng = np.random.default_rng(4)
        ids = [int(t) for t in rng.integers(0, 203, size=2108)]
        want = plain.plain_forward(config, weights, ids, torch.bfloat16).numpy()
        places = [0, 1, 777, 2047, 2048, 2099] + list(range(2100, 2108))
        for cuts in ([2100], [2048, 52], [1030, 1070]):
            cuts = cuts + [1] * 8
            runner = build_runner(folder, "bfloat16", 2176, page_size=64)
            steps, at = [], 0
            for size in cuts:
                asked = [p - at for p in places if at <= p < at + size]
                steps.append({"step": len(steps), "entries": [
                    {"id": "w", "tokens": ids[at: at + size], "want": asked}], "end": []})
                at += size
            with tempfile.TemporaryDirectory() as out:
                th.replay_in_process(runner, steps, out)
                rows = th.collect(steps, out, 203)
            assert sorted(p for _, p in rows) == places
            for (_, pos), got in rows.items():
                assert_close(got, want[pos], torch.bfloat16,
                             f"wide model, cuts {cuts[:2]}, position {pos}")
