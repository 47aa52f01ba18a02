"""Compares the plain implementation (tests/plain_llama.py) with the reference's own model code on
the CPU, once, on tiny random models, and writes the small outputs next to this file.

Run it where the reference project is checked out:

    DISTENGINE_REFERENCE_SRC=<reference>/src python tests/golden/make_golden.py

The reference's ``models.llama.LlamaForCausalLM`` is built from a ``transformers.LlamaConfig`` (it
is only a holder of sizes there, src/models/llama.py:93-129), loaded with this repository's seeded
random weights by state-dict name, and run whole and uncached in float32
(src/utils/generation.py:75-85 does the same per token).  The reference ignores
``tie_word_embeddings`` (src/models/llama.py:201), so a tied model gets a copy of the embedding
table as its ``lm_head.weight``.  Outputs: for every tiny model, token ids and the reference's
logits at all positions.  ``tests/test_plain.py`` checks the plain implementation against them.

The reference has no bfloat16 mode of its own, but its modules run in whatever dtype their
parameters have: the same model cast to bfloat16 (weights, activations and the residual sums all
bfloat16, src/models/llama.py:74-89) is run too and its logits stored as ``logits_bf16``.  The
engine keeps the residual stream and the logits in float32, so it does not reproduce those
roundings; the stored logits anchor how far the engine's bfloat16 path, and the plain
implementation's bfloat16 rounding model, lie from the reference's own arithmetic in that dtype.
"""

from __future__ import annotations

import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import plain_llama  # noqa: E402
import tiny_configs  # noqa: E402


def main() -> None:
    src = os.environ.get("DISTENGINE_REFERENCE_SRC")
    if not src or not os.path.isdir(src):
        raise SystemExit("set DISTENGINE_REFERENCE_SRC to the reference's src folder")
    sys.path.insert(0, src)
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    sys.dont_write_bytecode = True
    from transformers import LlamaConfig
    from models.llama import LlamaForCausalLM

    torch.manual_seed(0)
    with tempfile.TemporaryDirectory() as root:
        for name, spec in tiny_configs.ALL.items():
            cfg = spec["config"]
            if cfg.get("head_dim") and cfg["head_dim"] != cfg["hidden_size"] // cfg[
                    "num_attention_heads"]:
                # the reference derives the head size (src/layers/attention.py:90)
                print(f"{name}: head_dim is given; the reference cannot run it, skipped")
                continue
            folder = tiny_configs.make_folder(name, root)
            config, weights = plain_llama.load_model_folder(folder)
            theta = plain_llama.rope_theta_of(config)
            ref_config = LlamaConfig(
                vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
                intermediate_size=cfg["intermediate_size"],
                num_hidden_layers=cfg["num_hidden_layers"],
                num_attention_heads=cfg["num_attention_heads"],
                num_key_value_heads=cfg["num_key_value_heads"],
                rms_norm_eps=cfg["rms_norm_eps"],
                max_position_embeddings=cfg["max_position_embeddings"],
                rope_parameters={"rope_type": "default", "rope_theta": theta})
            model = LlamaForCausalLM(ref_config).to(torch.float32).eval()
            state = dict(weights)
            if "lm_head.weight" not in state:
                state["lm_head.weight"] = state["model.embed_tokens.weight"].clone()
            model.load_state_dict(state, strict=True)
            length = max(spec["prompts"])
            ids = tiny_configs.prompt_tokens(name, length)
            with torch.inference_mode():
                ref_logits = model(torch.tensor([ids]))[0].to(torch.float32)
                bf16_model = LlamaForCausalLM(ref_config).to(torch.bfloat16).eval()
                bf16_model.load_state_dict({k: v.to(torch.bfloat16) for k, v in state.items()},
                                           strict=True)
                ref_bf16 = bf16_model(torch.tensor([ids]))[0].to(torch.float32)
            plain_bf16 = plain_llama.plain_forward(config, weights, ids, torch.bfloat16)
            err16 = (plain_bf16 - ref_bf16).abs()
            print(f"{name}: bfloat16 rounding model against the reference cast to bfloat16: max "
                  f"{err16.max().item():.3e}, rms {err16.pow(2).mean().sqrt().item():.3e} "
                  f"(max |logit| {ref_bf16.abs().max().item():.3e})")
            plain = plain_llama.plain_forward(config, weights, ids)
            err = (plain - ref_logits).abs().max().item()
            scale = ref_logits.abs().max().item()
            print(f"{name}: {length} tokens, max |plain - reference| = {err:.3e} "
                  f"(max |logit| {scale:.3e})")
            assert err <= 2e-6 * max(1.0, scale), "the plain implementation disagrees"
            np.savez_compressed(os.path.join(HERE, f"{name}.npz"),
                                token_ids=np.asarray(ids, dtype=np.int32),
                                logits=ref_logits.numpy(), logits_bf16=ref_bf16.numpy())


if __name__ == "__main__":
    main()
