"""Typed configuration of the Llama dense decoder, read from the architecture's config.json keys.

Keys and their meaning follow what the reference's model reads from ``transformers.LlamaConfig``
(src/models/llama.py:93-129, src/distengine/model_runner.py:25-39): vocab_size, hidden_size,
intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads (absent: the number
of query heads, :101-103), rms_norm_eps, and rope_theta with rope_type "default" (:105-110).

Beyond the reference: ``rope_theta`` is also accepted as a top-level key (Llama config.json files
carry it there); ``head_dim`` is honoured when given (the reference always uses hidden_size //
heads, src/layers/attention.py:90); ``tie_word_embeddings`` is honoured (the reference always has
a separate lm_head, src/models/llama.py:201); ``max_position_embeddings`` bounds a request's length
(the reference never enforces it).  Options the reference ignores and this engine does not compute
(attention_bias, mlp_bias, another hidden_act, scaled RoPE) are refused instead of ignored.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .model import ConfigError, LayerSpec, ModelConfig, PartSpec, positive, require


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_id: int | None = None

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def from_json(data: Mapping[str, Any]) -> "LlamaConfig":
        hidden = positive("hidden_size", require(data, "hidden_size", int))
        heads = positive("num_attention_heads", require(data, "num_attention_heads", int))
        kv_heads = data.get("num_key_value_heads")
        if kv_heads is None:
            kv_heads = heads
        if not isinstance(kv_heads, int) or isinstance(kv_heads, bool) or kv_heads <= 0:
            raise ConfigError(f"config.json: 'num_key_value_heads' must be a positive integer, "
                              f"got {kv_heads!r}")
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads ({heads}) must be a multiple of "
                              f"num_key_value_heads ({kv_heads})")
        head_dim = data.get("head_dim")
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(f"config.json: hidden_size ({hidden}) must be a multiple of "
                                  f"num_attention_heads ({heads}) when 'head_dim' is absent")
            head_dim = hidden // heads
        if not isinstance(head_dim, int) or isinstance(head_dim, bool) or head_dim <= 0:
            raise ConfigError(f"config.json: 'head_dim' must be a positive integer, got {head_dim!r}")
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim ({head_dim}) must be even for rotary "
                              f"position encoding")

        # rotary parameters: nested (what the reference reads) or top-level
        rope = data.get("rope_parameters")
        scaling = data.get("rope_scaling")
        rope_type = "default"
        theta = data.get("rope_theta")
        if isinstance(rope, Mapping):
            rope_type = rope.get("rope_type", rope.get("type", "default"))
            theta = rope.get("rope_theta", theta)
        if isinstance(scaling, Mapping):
            rope_type = scaling.get("rope_type", scaling.get("type", rope_type))
        if rope_type != "default":
            raise ConfigError(f"config.json: rope type '{rope_type}' is not supported; only "
                              f"'default' rotary position encoding is")
        if theta is None:
            raise ConfigError("config.json: key 'rope_theta' is missing (top-level or inside "
                              "'rope_parameters')")
        if isinstance(theta, bool) or not isinstance(theta, (int, float)) or theta <= 0:
            raise ConfigError(f"config.json: 'rope_theta' must be a positive number, got {theta!r}")

        for key in ("attention_bias", "mlp_bias"):
            if data.get(key):
                raise ConfigError(f"config.json: '{key}' = true is not supported (the linear "
                                  f"layers of this architecture have no bias)")
        act = data.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported; only 'silu' is")

        eps = require(data, "rms_norm_eps", float)
        if eps <= 0:
            raise ConfigError(f"config.json: 'rms_norm_eps' must be positive, got {eps}")

        def optional_id(key: str) -> int | None:
            value = data.get(key)
            if isinstance(value, list):
                value = value[0] if value else None
            if value is not None and (isinstance(value, bool) or not isinstance(value, int)):
                raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
            return value

        tied = data.get("tie_word_embeddings", False)
        if not isinstance(tied, bool):
            raise ConfigError(f"config.json: 'tie_word_embeddings' must be true or false, "
                              f"got {tied!r}")
        architectures = data.get("architectures") or ["LlamaForCausalLM"]
        return LlamaConfig(
            architecture=architectures[0],
            vocab_size=positive("vocab_size", require(data, "vocab_size", int)),
            hidden_size=hidden,
            intermediate_size=positive("intermediate_size",
                                       require(data, "intermediate_size", int)),
            num_hidden_layers=positive("num_hidden_layers",
                                       require(data, "num_hidden_layers", int)),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=eps,
            rope_theta=float(theta),
            max_position_embeddings=positive("max_position_embeddings",
                                             require(data, "max_position_embeddings", int)),
            tie_word_embeddings=tied,
            bos_token_id=optional_id("bos_token_id"),
            eos_token_id=optional_id("eos_token_id"),
        )

    def to_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architectures": [self.architecture or "LlamaForCausalLM"],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_parameters": {"rope_type": "default", "rope_theta": self.rope_theta},
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out

    # ------------------------------------------------------------------ the model as data
    @property
    def width(self) -> int:
        return self.hidden_size

    @property
    def vocabulary(self) -> int:
        return self.vocab_size

    @property
    def max_positions(self) -> int:
        return self.max_position_embeddings

    @property
    def tied_output(self) -> bool:
        return self.tie_word_embeddings

    def layer_specs(self) -> list[LayerSpec]:
        """Every layer: pre-norm block, grouped-query attention with rotary position encoding,
        SwiGLU feed-forward, RMS norm (src/models/llama.py:32-89)."""
        norm = PartSpec.of("rmsnorm", width=self.hidden_size, eps=self.rms_norm_eps)
        mixer = PartSpec.of(
            "attention",
            width=self.hidden_size,
            heads=self.num_attention_heads,
            kv_heads=self.num_key_value_heads,
            head_dim=self.head_dim,
            scale=self.head_dim ** -0.5,                     # src/layers/attention.py:22
            window=None,                                     # causal only (:41-58)
            position=PartSpec.of("rope", rotary_dim=self.head_dim, theta=self.rope_theta),
        )
        feed_forward = PartSpec.of("gated_mlp", width=self.hidden_size,
                                   inner=self.intermediate_size, activation="silu")
        specs = []
        for i in range(self.num_hidden_layers):
            base = f"model.layers.{i}."
            specs.append(LayerSpec(
                block="prenorm", mixer=mixer, feed_forward=feed_forward, norm=norm,
                prefixes=(("mixer", base + "self_attn."),
                          ("feed_forward", base + "mlp."),
                          ("mixer_norm", base + "input_layernorm."),
                          ("feed_forward_norm", base + "post_attention_layernorm.")),
            ))
        return specs

    def final_norm(self) -> PartSpec:
        return PartSpec.of("rmsnorm", width=self.hidden_size, eps=self.rms_norm_eps)

    def tensor_names(self) -> dict[str, str]:
        return {"embedding": "model.embed_tokens.weight",
                "final_norm": "model.norm.",
                "output": "lm_head.weight"}
