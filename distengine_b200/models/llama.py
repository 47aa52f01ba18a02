"""The Llama architecture: ``LlamaConfig`` describes it, the generic decoder runs it.

Registered under the names that its config.json files carry in ``architectures``.
Reference: src/models/llama.py (LlamaForCausalLM), run there for TinyLlama-1.1B-Chat.
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..registry import register_architecture
from .decoder import DecoderModel


def build_llama(config: LlamaConfig, dtype, device) -> DecoderModel:
    return DecoderModel(config, dtype, device)


register_architecture("LlamaForCausalLM", LlamaConfig.from_json, build_llama)
