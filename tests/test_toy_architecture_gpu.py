"""A mixer with state of its own, defined here, is registered, built and stepped without a change
to the framework's files; and the layer order is data: a layer named twice, a run that reads
another run's cache, layers of different kinds in one model.

The toy mixer is a causal running mean: out_t = W * mean(x_0 .. x_t).  Its per-request state of
fixed size is the running sum of its inputs (one vector per request, in a slot).  It is a test
fixture only."""

import tempfile
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama as plain
import trace_helpers as th
from gpu_helpers import assert_close

pytestmark = pytest.mark.gpu
_registered = False


def _register():
    global _registered
    if _registered:
        return
    _registered = True
    from distengine_b200.config.model import LayerSpec, ModelConfig, PartSpec, PlanEntry
    from distengine_b200.models.decoder import DecoderModel
    from distengine_b200.parts import Mixer, StateSpec, register_mixer
    from distengine_b200.parts.base import compute_matrix
    from distengine_b200.registry import register_architecture

    class RunningMean(Mixer):
        graph_safe = False        # its forward walks the step's host arrays

        def __init__(self, width, dtype, device):
            super().__init__(dtype, device)
            self.width = width

        def tensors(self):
            return {"mix.weight": ((self.width, self.width), "matrix")}

        def load(self, tensors):
            self.w = compute_matrix(tensors["mix.weight"], self.dtype, self.device)

        def cache_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, x, ctx, cache):
            assert cache.kind == "state" and cache.state.shape[1:] == (self.width,)
            out = torch.empty_like(x)
            host = ctx.host
            for s in range(ctx.n_seqs):
                lo, n = int(host.seq_qstart[s]), int(host.seq_qlen[s])
                slot, pos0 = int(host.seq_slot[s]), int(host.seq_pos0[s])
                sums = cache.state[slot] + torch.cumsum(x[lo: lo + n].float(), dim=0)
                counts = torch.arange(pos0 + 1, pos0 + n + 1, device=x.device)[:, None]
                mean = (sums / counts).to(self.dtype)
                out[lo: lo + n] = (mean.float() @ self.w.float().t()).to(self.dtype)
                cache.state[slot] = sums[-1]
            return out

    register_mixer("toy_running_mean", RunningMean)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        data: tuple = ()

        @staticmethod
        def from_json(data):
            return ToyConfig(architecture="ToyForCausalLM", data=tuple(sorted(
                (k, tuple(v) if isinstance(v, list) else v) for k, v in data.items())))

        def get(self, key):
            return dict(self.data)[key]

        def to_json(self):
            out = {k: list(v) if isinstance(v, tuple) else v for k, v in self.data}
            out["architectures"] = ["ToyForCausalLM"]
            return out

        width = property(lambda self: self.get("width"))
        vocabulary = property(lambda self: self.get("vocab"))
        max_positions = property(lambda self: self.get("max_positions"))
        tied_output = property(lambda self: True)

        def layer_specs(self):
            w, eps = self.width, self.get("eps")
            norm = PartSpec.of("rmsnorm", width=w, eps=eps)
            ffn = PartSpec.of("gated_mlp", width=w, inner=self.get("inner"), activation="silu")
            attn = PartSpec.of("attention", width=w, heads=self.get("heads"),
                               kv_heads=self.get("kv_heads"), head_dim=self.get("head_dim"),
                               scale=self.get("head_dim") ** -0.5,
                               window=dict(self.data).get("window"),
                               position=PartSpec.of("rope", rotary_dim=self.get("head_dim"),
                                                    theta=self.get("theta")))
            toy = PartSpec.of("toy_running_mean", width=w)
            specs = []
            for i, kind in enumerate(self.get("kinds")):
                p = f"layers.{i}."
                specs.append(LayerSpec("prenorm", attn if kind == "attention" else toy, ffn, norm,
                                       (("mixer", p + "mixer."), ("feed_forward", p + "ffn."),
                                        ("mixer_norm", p + "norm1."),
                                        ("feed_forward_norm", p + "norm2."))))
            return specs

        def plan(self):
            return [PlanEntry(layer, None if reads < 0 else reads)
                    for layer, reads in self.get("plan")]

        def final_norm(self):
            return PartSpec.of("rmsnorm", width=self.width, eps=self.get("eps"))

        def tensor_names(self):
            return {"embedding": "embed.weight", "final_norm": "norm.", "output": "head.weight"}

    register_architecture("ToyForCausalLM", ToyConfig.from_json,
                          lambda config, dtype, device: DecoderModel(config, dtype, device))


TOY = dict(architectures=["ToyForCausalLM"], width=40, vocab=97, max_positions=256, eps=1e-5,
           inner=56, heads=2, kv_heads=1, head_dim=20, theta=1000.0,
           kinds=["attention", "toy", "attention"],
           # layer 0, the toy layer, layer 0 again (a cache of its own), layer 2 reading the cache
           # that the first run of layer 0 wrote, the toy layer again (a state of its own)
           plan=[[0, -1], [1, -1], [0, -1], [2, 0], [1, -1]])


def _plain_toy(config, w, ids, dtype):
    """The toy model, whole sequence, from the plain parts."""
    T = len(ids)
    pos = torch.arange(T)
    x = plain._rnd(w["embed.weight"], dtype)[torch.tensor(ids)]
    kv = {}

    def attn(h, p, entry, reads):
        d, nh, nkv = config["head_dim"], config["heads"], config["kv_heads"]
        q = plain.plain_rope(plain.plain_linear(h, w[p + "q_proj.weight"], dtype).view(T, nh, d),
                             pos, config["theta"], dtype)
        if reads is None:
            k = plain.plain_rope(plain.plain_linear(h, w[p + "k_proj.weight"], dtype)
                                 .view(T, nkv, d), pos, config["theta"], dtype)
            v = plain.plain_linear(h, w[p + "v_proj.weight"], dtype).view(T, nkv, d)
            kv[entry] = (k, v)
        else:
            k, v = kv[reads]
        ctx = plain.plain_attention(q, k, v, pos, config.get("window"), dtype)
        return plain.plain_linear(ctx.reshape(T, nh * d), w[p + "o_proj.weight"], dtype)

    def toy(h, p):
        mean = plain._rnd(torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None], dtype)
        return plain._rnd(mean @ plain._rnd(w[p + "mix.weight"], dtype).t(), dtype)

    for entry, (layer, reads) in enumerate(config["plan"]):
        p = f"layers.{layer}."
        h = plain.plain_rmsnorm(x, w[p + "norm1.weight"], config["eps"], dtype)
        if config["kinds"][layer] == "attention":
            x = x + attn(h, p + "mixer.", entry, None if reads < 0 else reads)
        else:
            x = x + toy(h, p + "mixer.")
        h = plain.plain_rmsnorm(x, w[p + "norm2.weight"], config["eps"], dtype)
        x = x + plain.plain_mlp(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                                w[p + "ffn.down_proj.weight"], dtype)
    x = plain.plain_rmsnorm(x, w["norm.weight"], config["eps"], dtype)
    return plain.plain_linear(x, w["embed.weight"], dtype, keep_f32=True)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_toy_architecture_is_built_and_stepped(dtype_name, model_root):
    _register()
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.weights import write_random_model
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype_name]
    folder = write_random_model(TOY, f"{model_root}/toy", seed=4, norm_init="uniform")
    config, weights = plain.load_model_folder(folder)
    rng = np.random.default_rng(0)
    requests = {f"t{i}": [int(t) for t in rng.integers(0, 97, size=n)]
                for i, n in enumerate([50, 9, 77, 30, 64])}
    want = {rid: _plain_toy(config, weights, ids, dtype).numpy() for rid, ids in requests.items()}
    # (the last 32 tokens one by one: steps of single tokens, where the run that reads another
    # run's cache goes through the one-launch decode attention)
    for steps, max_tokens in ((th.schedule_whole(requests), 128),
                              (th.schedule_tail(requests, 32), 128),
                              (th.schedule_portions(requests), 128),
                              (th.schedule_mixed(requests, 256, seed=1), 256)):
        runner = build_runner(folder, dtype_name, max_tokens, page_size=16,
                              poison_freed_pages=True)
        model = runner.model
        # a cache for each run that writes; the reading run has none of its own
        specs = model.cache_specs()
        assert [type(s).__name__ for s in specs] == ["PagedKVSpec", "StateSpec", "PagedKVSpec",
                                                     "NoneType", "StateSpec"]
        assert runner.cache.paged[0].k.shape[0] == 2 and runner.cache.states[0].state.shape[0] == 2
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            rows = th.collect(steps, out, 97)
        for (rid, pos), got in rows.items():
            assert_close(got, want[rid][pos], dtype, f"toy {rid}@{pos}")
        runner.cache.check_invariants()


def test_a_plan_that_reads_a_cache_of_another_shape_is_refused():
    _register()
    from distengine_b200.registry import resolve
    bad = dict(TOY, plan=[[0, -1], [1, -1], [2, 1]])      # attention reading the toy's state
    arch, config = resolve(bad)
    with pytest.raises(ValueError, match="cannot read the cache"):
        arch.build_model(config, torch.float32, "cuda:0").cache_specs()
    with pytest.raises(ValueError, match="does not run before"):
        arch.build_model(resolve(dict(TOY, plan=[[0, 1], [1, -1]]))[1], torch.float32, "cuda:0")


def _plain_toy_generate(config, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(_plain_toy(config, weights, tokens, torch.float32)[-1].argmax()))
    return tokens[len(prompt):]


def test_a_step_taken_back_gives_state_and_window_pages_back(model_root):
    """Through ``Engine``: a windowed attention layer (window 6, pages of 4) and the running-mean
    layer, three requests, one of which ends on an end-of-sequence token.  The engine has then
    already launched the next step for all three; that step is void.  The running sums it
    advanced must be what they were, and the page that its window would have passed must still
    be there for the token that is fed again.  The second request's prompt takes eight lengths in
    turn, so that the void step meets every alignment of window and page.  Freed pages hold
    NaN."""
    _register()
    from distengine_b200 import Engine, EngineConfig
    from distengine_b200.weights import write_random_model
    toy = dict(TOY, kinds=["attention", "toy"], plan=[[0, -1], [1, -1]], window=6,
               max_positions=128)
    folder = write_random_model(toy, f"{model_root}/toy-window", seed=6, norm_init="uniform")
    config, weights = plain.load_model_folder(folder)
    rng = np.random.default_rng(3)
    first = [int(t) for t in rng.integers(0, 97, size=9)]
    third = [int(t) for t in rng.integers(0, 97, size=5)]
    alone_first = _plain_toy_generate(config, weights, first, 8)
    # the first request ends on a token that it has not produced before
    cut = max(i for i in range(len(alone_first)) if alone_first[i] not in alone_first[:i])
    taken_back = 0
    for length in range(6, 14):
        second = [int(t) for t in rng.integers(0, 97, size=length)]
        alone = [_plain_toy_generate(config, weights, p, 14) for p in (second, third)]
        engine = Engine(folder, EngineConfig(dtype="float32", block_size=4, num_blocks=48,
                                             decode_batch_size=4))
        engine.cache.poison = True
        for group in engine.cache.paged:
            group.k.fill_(float("nan"))
            group.v.fill_(float("nan"))
        voided = []
        take_back = engine._take_back
        engine._take_back = lambda prepared: (voided.append(1), take_back(prepared))[1]
        engine.submit("a", first, 14, eos_token_id=alone_first[cut])
        engine.submit("b", second, 14, eos_token_id=-1)
        engine.submit("c", third, 14, eos_token_id=-1)
        while engine.has_pending():
            engine.step()
        records = {r["request_id"]: r for r in engine.drain_completed()}
        taken_back += len(voided)
        assert records["a"]["generated_token_ids"] == alone_first[: cut + 1], length
        assert records["b"]["generated_token_ids"] == alone[0], length
        assert records["c"]["generated_token_ids"] == alone[1], length
        engine.cache.check_invariants()
        assert engine.cache.num_free_pages() == engine.cache.num_pages
    assert taken_back == 8
