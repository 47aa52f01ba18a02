"""The benchmark's own layer sizes (TinyLlama-1.1B: width 2,048, 32 query and 4 key/value heads of
64, inner width 5,632, vocabulary 32,000), with 4 of its 22 layers so that the plain implementation
on the CPU stays within minutes, against the plain implementation:

* float32, the four ways of cutting, through the replay;
* bfloat16 decode steps replayed as CUDA graphs at batch 8 and batch 64, from 500-token prompts
  across the 512-position boundary at which the graph's key-range cap (and with it the graph and
  the plan of the decode attention) changes: logits of every request at every step;
* the same through ``Engine`` (graphs on, the GPU one step ahead of the host): logits at every
  generated position and the tokens;
* a context of 4,200 tokens, then graphed decode steps whose key ranges take several clusters a
  tile.

The reference checks its outputs at full model size too, token for token
(src/utils/benchmark.py:187-207,365-400)."""

import tempfile

import numpy as np
import pytest
import torch

import plain_llama as plain
import trace_helpers as th
from gpu_helpers import BF16_MAX_REL, assert_close

pytestmark = pytest.mark.gpu

LAYERS, LAYERS_OF_MODEL = 4, 22
SHAPE = dict(architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=2048,
             intermediate_size=5632, num_hidden_layers=LAYERS, num_attention_heads=32,
             num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0,
             max_position_embeddings=2048, tie_word_embeddings=False)
VOCAB = SHAPE["vocab_size"]
_models: dict = {}
_plain: dict = {}


def _model(model_root, max_positions=2048):
    if max_positions not in _models:
        from distengine_b200.weights import write_random_model
        shape = dict(SHAPE, max_position_embeddings=max_positions)
        folder = write_random_model(shape, f"{model_root}/full-width-{max_positions}", seed=0,
                                    dtype="bfloat16")
        _models[max_positions] = (folder,) + plain.load_model_folder(folder)
    return _models[max_positions]


def _plain_rows(model_root, tokens, dtype, rows, max_positions=2048):
    """Plain logits of ``tokens`` at ``rows``; one forward per distinct (sequence, dtype)."""
    _, config, weights = _model(model_root, max_positions)
    key = (tuple(tokens), dtype, tuple(rows))
    if key not in _plain:
        _plain[key] = plain.plain_forward(config, weights, tokens, dtype, rows=list(rows)).numpy()
    return _plain[key]


def _tokens(seed, n):
    return [int(t) for t in np.random.default_rng(seed).integers(0, VOCAB, size=n)]


@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_float32_cuts_at_the_benchmark_width(schedule, model_root):
    """True 32-bit at real width: the float32 matrix product with k = 5,632 inside a model, the
    CUDA-core attention at 32 and 4 heads, every cut."""
    from distengine_b200.engine.replay import build_runner
    folder, config, weights = _model(model_root)
    requests = {f"q{i}": _tokens(100 + i, n) for i, n in enumerate([210, 97, 45, 33])}
    steps, max_tokens = {
        "whole": (th.schedule_whole(requests), 256),
        "tail": (th.schedule_tail(requests, 32), 256),
        "portions": (th.schedule_portions(requests), 256),
        "mixed": (th.schedule_mixed(requests, 384, seed=5), 384),
    }[schedule]
    runner = build_runner(folder, "float32", max_tokens, page_size=16, poison_freed_pages=True)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, VOCAB)
    runner.cache.check_invariants()
    for rid, tokens in requests.items():
        positions = sorted(p for r, p in rows if r == rid)
        assert positions
        want = _plain_rows(model_root, tokens, torch.float32, range(len(tokens)))
        got = np.stack([rows[(rid, p)] for p in positions])
        assert_close(got, want[positions], torch.float32, f"{LAYERS} of {LAYERS_OF_MODEL} "
                     f"layers, float32 {schedule} {rid}")


def _decode_trace(requests, prompt_len, batch_budget=2048):
    """Prompts in steps of up to ``batch_budget`` tokens (no logits), then every request one token
    a step, logits wanted, until the tokens run out."""
    steps, batch, used = [], [], 0
    for rid, tokens in requests.items():
        if used + prompt_len > batch_budget and batch:
            steps.append({"step": len(steps), "entries": batch, "end": []})
            batch, used = [], 0
        batch.append({"id": rid, "tokens": tokens[:prompt_len], "want": []})
        used += prompt_len
    steps.append({"step": len(steps), "entries": batch, "end": []})
    total = len(next(iter(requests.values())))
    for at in range(prompt_len, total):
        steps.append({"step": len(steps), "end": list(requests) if at == total - 1 else [],
                      "entries": [{"id": rid, "tokens": [tokens[at]], "want": [0]}
                                  for rid, tokens in requests.items()]})
    return steps


@pytest.mark.parametrize("batch", [8, 64])
def test_graphed_decode_steps_at_the_benchmark_width(batch, model_root):
    """bfloat16, CUDA graphs on: ``batch`` requests (four distinct token sequences, the others
    their copies under other names, slots and pages) with 500 tokens in the cache decode 24 tokens
    each, from position 500 to 523: the graph for a cap of 512 positions, then a new one for
    1,024.  Batch 64 is the library's products with norm kernels of their own, batch 8 the
    weight-streaming products that carry the norms."""
    from distengine_b200.engine.replay import build_runner
    folder, config, weights = _model(model_root)
    prompt_len, new = 500, 24
    distinct = [_tokens(200 + i, prompt_len + new) for i in range(4)]
    requests = {f"g{i}": distinct[i % 4] for i in range(batch)}
    steps = _decode_trace(requests, prompt_len)
    runner = build_runner(folder, "bfloat16", batch * 576, page_size=16, use_graphs=True,
                          live_requests=batch)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, VOCAB)
    # (a graph's key begins with the sequences' token counts; steps of the prompts, which repeat
    # too, may have graphs of their own)
    decode_graphs = [key for key in runner._graphs
                     if (np.frombuffer(key[0], dtype=np.int32) == 1).all()]
    assert runner.graph_replays >= new - 4 and len(decode_graphs) == 2
    positions = list(range(prompt_len, prompt_len + new))
    for rid, tokens in requests.items():
        want = _plain_rows(model_root, tokens, torch.bfloat16, positions)
        got = np.stack([rows[(rid, p)] for p in positions])
        assert_close(got, want, torch.bfloat16, f"{LAYERS} of {LAYERS_OF_MODEL} layers, graphed "
                     f"decode at batch {batch}, {rid}")


@pytest.mark.parametrize("batch", [8, 64])
def test_engine_at_the_benchmark_width(batch, model_root):
    """``Engine.generate`` in bfloat16 with graphs on and the GPU a step ahead of the host:
    ``batch`` requests (copies of four prompts of 500 tokens) generate 20 tokens each.  Checked
    are the logits at every generated position against the plain model fed the engine's own
    tokens, and that every token is the plain model's choice or nearly tied with it."""
    from distengine_b200 import Engine, EngineConfig
    folder, config, weights = _model(model_root)
    prompt_len, new = 500, 20
    prompts = [_tokens(300 + i % 4, prompt_len) for i in range(batch)]
    engine = Engine(folder, EngineConfig(dtype="bfloat16", block_size=16,
                                         num_blocks=batch * 36, decode_batch_size=batch,
                                         max_batch_tokens=2048))
    seen: dict = {}

    def keep(places, logits):
        host = logits.float().cpu().numpy()
        for row, place in enumerate(places):
            seen[place] = host[row].copy()

    engine.on_logits = keep
    ids = [f"e{i}" for i in range(batch)]
    for rid, prompt in zip(ids, prompts):
        engine.submit(rid, prompt, new, -1)
    results = {}
    while engine.has_pending():
        for record in engine.step():
            results[record["request_id"]] = record["generated_token_ids"]
    assert engine.runner.graph_replays > 0
    engine.cache.check_invariants()
    positions = list(range(prompt_len - 1, prompt_len + new - 1))
    for rid, prompt in zip(ids, prompts):
        generated = results[rid]
        assert len(generated) == new
        want = _plain_rows(model_root, prompt + generated[:-1], torch.bfloat16, positions)
        got = np.stack([seen[(rid, p)] for p in positions])
        assert_close(got, want, torch.bfloat16, f"{LAYERS} of {LAYERS_OF_MODEL} layers, engine "
                     f"at batch {batch}, {rid}")
        for i, token in enumerate(generated):
            best = int(want[i].argmax())
            gap = float(want[i][best] - want[i][token])
            assert gap <= BF16_MAX_REL * float(np.abs(want[i]).max()), (rid, i, token, best, gap)


def test_graphed_decode_over_several_clusters_at_the_benchmark_width(model_root):
    """One request with 4,200 tokens of context (the same layers with a longer position limit),
    then 6 graphed decode steps: each key range is cut over several thread-block clusters a tile,
    whose partial results are merged through global memory inside the replayed graph."""
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.kernels.attention_plan import choose_decode_split
    folder, config, weights = _model(model_root, max_positions=8192)
    context, new = 4200, 6
    tokens = _tokens(400, context + new)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert choose_decode_split(1, 4, 4608, sm_count=sms)[1] > 1
    steps, at = [], 0
    for size in (2048, 2048, 104):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": "long", "tokens": tokens[at: at + size], "want": [size - 1]}]})
        at += size
    for i in range(new):
        steps.append({"step": len(steps), "end": ["long"] if i == new - 1 else [], "entries": [
            {"id": "long", "tokens": [tokens[at + i]], "want": [0]}]})
    runner = build_runner(folder, "bfloat16", 4608, page_size=16, use_graphs=True)
    with tempfile.TemporaryDirectory() as out:
        th.replay_in_process(runner, steps, out)
        rows = th.collect(steps, out, VOCAB)
    assert runner.graph_replays >= new - 2
    positions = sorted(p for _, p in rows)
    want = _plain_rows(model_root, tokens, torch.bfloat16, positions, max_positions=8192)
    got = np.stack([rows[("long", p)] for p in positions])
    assert_close(got, want, torch.bfloat16, f"{LAYERS} of {LAYERS_OF_MODEL} layers, long context")
