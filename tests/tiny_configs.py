"""The tiny configurations the tests run on.  They differ in every size and option: layers, width,
heads and groups (grouped-query against plain multi-head), head size, inner width, vocabulary,
rotary base, the norm's eps, the longest position, tied against separate output matrix, how the
norm weights are drawn, page size and seed.  C has sizes that are no power of two and a head size
that is given, not derived."""

from __future__ import annotations

TINY_A = dict(
    config=dict(architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64,
                intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-5, rope_theta=10000.0,
                max_position_embeddings=128, tie_word_embeddings=False),
    seed=0, norm_init="ones", page_size=16,
    prompts=(5, 17, 33), max_new_tokens=8, temperature=0.0,
)

TINY_B = dict(
    config=dict(architectures=["LlamaForCausalLM"], vocab_size=320, hidden_size=96,
                intermediate_size=256, num_hidden_layers=3, num_attention_heads=3,
                num_key_value_heads=3, rms_norm_eps=1e-6, rope_theta=500000.0,
                max_position_embeddings=256, tie_word_embeddings=True),
    seed=1, norm_init="uniform", page_size=8,
    prompts=(1, 9, 40, 70), max_new_tokens=12, temperature=0.8,
)

TINY_C = dict(
    config=dict(architectures=["LlamaForCausalLM"], vocab_size=331, hidden_size=120,
                intermediate_size=200, num_hidden_layers=2, num_attention_heads=6,
                num_key_value_heads=1, head_dim=48, rms_norm_eps=3e-6,
                rope_parameters={"rope_type": "default", "rope_theta": 25000.0},
                max_position_embeddings=512, tie_word_embeddings=False),
    seed=2, norm_init="uniform", page_size=32,
    prompts=(3, 50), max_new_tokens=6, temperature=0.0,
)

# head size 64, grouped-query, a given head size
TINY_D = dict(
    config=dict(architectures=["LlamaForCausalLM"], vocab_size=300, hidden_size=192,
                intermediate_size=328, num_hidden_layers=2, num_attention_heads=6,
                num_key_value_heads=2, head_dim=64, rms_norm_eps=2e-5, rope_theta=50000.0,
                max_position_embeddings=256, tie_word_embeddings=False),
    seed=3, norm_init="uniform", page_size=16,
    prompts=(4, 30), max_new_tokens=6, temperature=0.0,
)

# head size 128 (the Llama-2 and Llama-3 head), three query heads on one key/value head
TINY_E = dict(
    config=dict(architectures=["LlamaForCausalLM"], vocab_size=270, hidden_size=136,
                intermediate_size=232, num_hidden_layers=2, num_attention_heads=3,
                num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                max_position_embeddings=256, tie_word_embeddings=True),
    seed=4, norm_init="uniform", page_size=32,
    prompts=(6, 21), max_new_tokens=6, temperature=0.0,
)

ALL = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D, "tiny_e": TINY_E}


def make_folder(name: str, root: str, dtype: str = "float32") -> str:
    """Write the tiny model ``name`` under ``root`` with the product's random-weights mode."""
    import os
    from distengine_b200.weights import write_random_model
    spec = ALL[name]
    return write_random_model(spec["config"], os.path.join(root, f"{name}-{dtype}"), spec["seed"],
                              dtype=dtype, norm_init=spec["norm_init"])


def prompt_tokens(name: str, length: int, index: int = 0) -> list[int]:
    """Seeded uniform token ids."""
    import numpy as np
    spec = ALL[name]
    rng = np.random.default_rng(1000 * spec["seed"] + 17 * index + length)
    return [int(t) for t in rng.integers(0, spec["config"]["vocab_size"], size=length)]
