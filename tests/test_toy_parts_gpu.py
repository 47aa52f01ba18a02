"""Parts of other kinds than the Llama ones, defined here and registered from outside the package:
a feed-forward that routes every token to one of several experts, and a position encoding that is
no rotation (it goes through the ``apply`` hook).  One model mixes them with the package's own
parts, layer by layer.  They are test fixtures only: they show that the framework's files need no
change for a new kind of part, not a model of anyone's."""

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
WAVE = 0.37          # the toy position encoding's frequency


def _register():
    global _registered
    if _registered:
        return
    _registered = True
    from distengine_b200.config.model import LayerSpec, ModelConfig, PartSpec, PlanEntry
    from distengine_b200.models.decoder import DecoderModel
    from distengine_b200.parts import (FeedForward, PositionEncoding, register_feed_forward,
                                       register_position_encoding)
    from distengine_b200.parts.base import compute_matrix
    from distengine_b200.registry import register_architecture

    class RoutedExperts(FeedForward):
        """out = p_e * W_e x with e = the expert of the largest router logit and p_e its softmax
        probability; router logits in float32."""

        def __init__(self, width, experts, dtype, device):
            super().__init__(dtype, device)
            self.width, self.experts = width, experts

        def tensors(self):
            out = {"router.weight": ((self.experts, self.width), "matrix")}
            for e in range(self.experts):
                out[f"experts.{e}.weight"] = ((self.width, self.width), "matrix")
            return out

        def load(self, tensors):
            self.router = tensors["router.weight"].to(self.device, torch.float32)
            self.w = torch.stack([compute_matrix(tensors[f"experts.{e}.weight"], self.dtype,
                                                 self.device) for e in range(self.experts)])

        def forward(self, x, ctx):
            logits = x.float() @ self.router.t()
            prob = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            picked = self.w[choice].float()                                   # [N, width, width]
            out = torch.bmm(picked, x.float()[:, :, None])[:, :, 0].to(self.dtype)
            gate = prob.gather(1, choice[:, None])
            return (out.float() * gate).to(self.dtype)

    class WavePositions(PositionEncoding):
        """Adds sin(f pos) to the first feature of every q head and cos(f pos) to the first
        feature of every k head, before k is stored: scores then depend on both positions."""

        def __init__(self, frequency, dtype, device):
            super().__init__(dtype, device)
            self.frequency = frequency

        def apply(self, q, k, ctx):
            angle = ctx.positions.float() * self.frequency
            q[:, :, 0] = (q[:, :, 0].float() + torch.sin(angle)[:, None]).to(q.dtype)
            k[:, :, 0] = (k[:, :, 0].float() + torch.cos(angle)[:, None]).to(k.dtype)

    register_feed_forward("toy_routed_experts", RoutedExperts)
    register_position_encoding("toy_wave", WavePositions)

    @dataclass(frozen=True)
    class MixConfig(ModelConfig):
        data: tuple = ()

        @staticmethod
        def from_json(data):
            return MixConfig(architecture="ToyMixForCausalLM", data=tuple(sorted(data.items())))

        def get(self, key):
            return dict(self.data)[key]

        def to_json(self):
            out = dict(self.data)
            out["architectures"] = ["ToyMixForCausalLM"]
            return out

        width = property(lambda self: self.get("width"))
        vocabulary = property(lambda self: self.get("vocab"))
        max_positions = property(lambda self: self.get("max_positions"))
        tied_output = property(lambda self: False)

        def layer_specs(self):
            w, eps, d = self.width, self.get("eps"), self.get("head_dim")
            norm = PartSpec.of("rmsnorm", width=w, eps=eps)

            def attention(position):
                return PartSpec.of("attention", width=w, heads=self.get("heads"),
                                   kv_heads=self.get("kv_heads"), head_dim=d, scale=d ** -0.5,
                                   window=None, position=position)
            kinds = [
                # layer 0: attention with the toy positions, routed experts
                (attention(PartSpec.of("toy_wave", frequency=WAVE)),
                 PartSpec.of("toy_routed_experts", width=w, experts=self.get("experts"))),
                # layer 1: the package's own rotation and gated feed-forward
                (attention(PartSpec.of("rope", rotary_dim=d, theta=self.get("theta"))),
                 PartSpec.of("gated_mlp", width=w, inner=self.get("inner"), activation="silu")),
                # layer 2: no position encoding at all, routed experts
                (attention(PartSpec.of("none")),
                 PartSpec.of("toy_routed_experts", width=w, experts=self.get("experts"))),
            ]
            return [LayerSpec("prenorm", mixer, ffn, norm,
                              (("mixer", f"layers.{i}.mixer."), ("feed_forward", f"layers.{i}.ffn."),
                               ("mixer_norm", f"layers.{i}.norm1."),
                               ("feed_forward_norm", f"layers.{i}.norm2.")))
                    for i, (mixer, ffn) in enumerate(kinds)]

        def plan(self):
            return [PlanEntry(i, None) for i in range(3)]

        def final_norm(self):
            return PartSpec.of("rmsnorm", width=self.width, eps=self.get("eps"))

        def tensor_names(self):
            return {"embedding": "embed.weight", "final_norm": "norm.", "output": "head.weight"}

    register_architecture("ToyMixForCausalLM", MixConfig.from_json,
                          lambda config, dtype, device: DecoderModel(config, dtype, device))


MIX = dict(architectures=["ToyMixForCausalLM"], width=48, vocab=89, max_positions=256, eps=2e-5,
           inner=72, heads=3, kv_heads=1, head_dim=16, theta=500.0, experts=3)


def _plain_mix(config, w, ids):
    """The model above, whole sequence, float32, from the plain parts."""
    T = len(ids)
    pos = torch.arange(T)
    d, nh, nkv = config["head_dim"], config["heads"], config["kv_heads"]
    x = w["embed.weight"][torch.tensor(ids)]

    def attention(h, p, kind):
        q = plain.plain_linear(h, w[p + "q_proj.weight"]).view(T, nh, d)
        k = plain.plain_linear(h, w[p + "k_proj.weight"]).view(T, nkv, d)
        v = plain.plain_linear(h, w[p + "v_proj.weight"]).view(T, nkv, d)
        if kind == "rope":
            q, k = plain.plain_rope(q, pos, config["theta"]), plain.plain_rope(k, pos, config["theta"])
        elif kind == "wave":
            q, k = q.clone(), k.clone()
            q[:, :, 0] += torch.sin(pos.float() * WAVE)[:, None]
            k[:, :, 0] += torch.cos(pos.float() * WAVE)[:, None]
        ctx = plain.plain_attention(q, k, v, pos)
        return plain.plain_linear(ctx.reshape(T, nh * d), w[p + "o_proj.weight"])

    def routed(h, p):
        logits = h @ w[p + "router.weight"].t()
        prob = torch.softmax(logits, dim=-1)
        choice = logits.argmax(dim=-1)
        out = torch.stack([w[p + f"experts.{int(e)}.weight"] @ h[t] for t, e in enumerate(choice)])
        return out * prob.gather(1, choice[:, None])

    for i, (kind, ffn) in enumerate([("wave", "routed"), ("rope", "mlp"), ("none", "routed")]):
        p = f"layers.{i}."
        h = plain.plain_rmsnorm(x, w[p + "norm1.weight"], config["eps"])
        x = x + attention(h, p + "mixer.", kind)
        h = plain.plain_rmsnorm(x, w[p + "norm2.weight"], config["eps"])
        if ffn == "routed":
            x = x + routed(h, p + "ffn.")
        else:
            x = x + plain.plain_mlp(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                                    w[p + "ffn.down_proj.weight"])
    x = plain.plain_rmsnorm(x, w["norm.weight"], config["eps"])
    return plain.plain_linear(x, w["head.weight"], keep_f32=True)


def test_routed_feed_forward_and_other_position_encodings_step_through_the_engine(model_root):
    """float32 (a routing decision must not hang on a rounding): whole prompts, portions down to
    two tokens, and mixed steps with few pages all give the plain model's logits, and the experts
    are all in use."""
    _register()
    from distengine_b200.engine.replay import build_runner
    from distengine_b200.weights import write_random_model
    folder = write_random_model(MIX, f"{model_root}/toy_mix", seed=9, norm_init="uniform")
    config, weights = plain.load_model_folder(folder)
    rng = np.random.default_rng(3)
    requests = {f"m{i}": [int(t) for t in rng.integers(0, 89, size=n)]
                for i, n in enumerate([41, 7, 66, 23])}
    want = {rid: _plain_mix(config, weights, ids).numpy() for rid, ids in requests.items()}
    h = plain.plain_rmsnorm(weights["embed.weight"], weights["layers.0.norm2.weight"], config["eps"])
    used = (h @ weights["layers.0.ffn.router.weight"].t()).argmax(dim=-1).unique()
    assert len(used) == MIX["experts"], "the random router should use every expert"
    for steps, max_tokens in ((th.schedule_whole(requests), 192),
                              (th.schedule_tail(requests, 8), 192),
                              (th.schedule_portions(requests), 192),
                              (th.schedule_mixed(requests, 192, seed=2), 192)):
        runner = build_runner(folder, "float32", max_tokens, page_size=16,
                              poison_freed_pages=True)
        with tempfile.TemporaryDirectory() as out:
            th.replay_in_process(runner, steps, out)
            rows = th.collect(steps, out, 89)
        assert rows
        for (rid, pos), got in rows.items():
            assert_close(got, want[rid][pos], torch.float32, f"toy mix {rid}@{pos}")
        runner.cache.check_invariants()
