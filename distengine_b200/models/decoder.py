"""The generic decoder: embedding, the blocks that the configuration's layer specs describe, run in
the order of its plan, final norm, output matrix.  Nothing in here is specific to one
architecture; an architecture is a configuration class (``config/``) plus one registry entry.

Reference counterpart: ``LlamaModel`` / ``LlamaForCausalLM`` (src/models/llama.py:92-217), whose
forward returns logits at all positions (:217); here only the wanted rows reach the output matrix.
"""

from __future__ import annotations

import torch

from ..config.model import LayerSpec, ModelConfig
from ..kernels import ops
from ..parts.base import (Block, PagedKVSpec, StateSpec, build_block, build_feed_forward,
                          build_mixer, build_norm, compute_matrix)
from ..parts.context import CacheBinding, ResidualStream, StepContext, StepPrep


def _layer_parts(spec: LayerSpec, dtype: torch.dtype, device: torch.device) -> Block:
    return build_block(spec.block,
                       build_mixer(spec.mixer, dtype, device),
                       build_feed_forward(spec.feed_forward, dtype, device),
                       build_norm(spec.norm, dtype, device),
                       build_norm(spec.norm, dtype, device))


class DecoderModel:
    def __init__(self, config: ModelConfig, dtype: torch.dtype,
                 device: "torch.device | str") -> None:
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        self.specs = config.layer_specs()
        self.plan = config.plan()
        for index, entry in enumerate(self.plan):
            if not 0 <= entry.layer < len(self.specs):
                raise ValueError(f"plan entry {index} names layer {entry.layer}, the model has "
                                 f"{len(self.specs)}")
            if entry.reads_cache_of is not None and not 0 <= entry.reads_cache_of < index:
                raise ValueError(f"plan entry {index} reads the cache of entry "
                                 f"{entry.reads_cache_of}, which does not run before it")
        self.blocks = [_layer_parts(spec, dtype, self.device) for spec in self.specs]
        self.final_norm = build_norm(config.final_norm(), dtype, self.device)
        self.embedding: "torch.Tensor | None" = None
        self.output: "torch.Tensor | None" = None

    # ------------------------------------------------------------------ weights
    def expected_tensors(self):
        """(name -> shape, names that are vectors, names that may be absent)."""
        names = self.config.tensor_names()
        expected: dict[str, tuple[int, ...]] = {
            names["embedding"]: (self.config.vocabulary, self.config.width)}
        vectors: set[str] = set()
        for spec, block in zip(self.specs, self.blocks):
            for role, part in block.parts().items():
                for local, (shape, kind) in part.tensors().items():
                    full = spec.prefix(role) + local
                    expected[full] = tuple(shape)
                    if kind == "vector":
                        vectors.add(full)
        for local, (shape, kind) in self.final_norm.tensors().items():
            expected[names["final_norm"] + local] = tuple(shape)
            if kind == "vector":
                vectors.add(names["final_norm"] + local)
        expected[names["output"]] = (self.config.vocabulary, self.config.width)
        optional = {names["output"]} if self.config.tied_output else set()
        return expected, vectors, optional

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        names = self.config.tensor_names()
        self.embedding = compute_matrix(tensors[names["embedding"]], self.dtype, self.device)
        for spec, block in zip(self.specs, self.blocks):
            for role, part in block.parts().items():
                prefix = spec.prefix(role)
                part.load({local: tensors[prefix + local] for local in part.tensors()})
        self.final_norm.load({local: tensors[names["final_norm"] + local]
                              for local in self.final_norm.tensors()})
        if names["output"] in tensors:
            self.output = compute_matrix(tensors[names["output"]], self.dtype, self.device)
        else:
            self.output = self.embedding          # tied: one matrix for both ends

    # ------------------------------------------------------------------ cache needs
    def cache_specs(self) -> "list[PagedKVSpec | StateSpec | None]":
        """For every plan entry what its run must be given: a cache of its own (a spec) or, when
        it reads an earlier entry's cache or its mixer keeps nothing, None."""
        out = []
        for entry in self.plan:
            spec = self.blocks[entry.layer].mixer.cache_spec()
            out.append(None if entry.reads_cache_of is not None else spec)
        for index, entry in enumerate(self.plan):
            if entry.reads_cache_of is not None:
                mine = self.blocks[entry.layer].mixer.cache_spec()
                theirs = self.blocks[self.plan[entry.reads_cache_of].layer].mixer.cache_spec()
                if self.plan[entry.reads_cache_of].reads_cache_of is not None or mine != theirs:
                    raise ValueError(f"plan entry {index} cannot read the cache of entry "
                                     f"{entry.reads_cache_of}: it needs {mine}, that entry "
                                     f"keeps {theirs}")
        return out

    # ------------------------------------------------------------------ step
    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for block in self.blocks for part in block.parts().values())

    def prepare(self, prep: StepPrep) -> None:
        for part in self._preparers():
            part.prepare(prep)

    def _preparers(self):
        """The parts whose ``prepare`` does something, one for each distinct plan key (layers of
        the same shape share their work lists); found once."""
        cached = getattr(self, "_preparer_list", None)
        if cached is None:
            from ..parts.base import Part
            cached, seen = [], set()
            for block in self.blocks:
                for part in block.parts().values():
                    if type(part).prepare is Part.prepare:
                        continue
                    key = getattr(part, "prepare_key", None)
                    if key is not None and key in seen:
                        continue
                    seen.add(key)
                    cached.append(part)
            self._preparer_list = cached
        return cached

    def forward(self, ctx: StepContext,
                caches: "list[CacheBinding | None]") -> torch.Tensor:
        """Run the step's tokens through the plan; logits float32 [R, vocabulary] at
        ``ctx.logit_rows``."""
        resid = ctx.buffer("model.residual", (ctx.n_tokens, self.config.width), torch.float32)
        ops.embed_rows(ctx.token_ids, self.embedding, resid)
        stream = ResidualStream(resid)
        for index, entry in enumerate(self.plan):
            # the norm and mixer that read the stream next, for blocks that hand a norm's work to
            # the product before it
            following = None
            if index + 1 < len(self.plan):
                later = self.blocks[self.plan[index + 1].layer]
                following = (later.mixer_norm, later.mixer)
            self.blocks[entry.layer].forward(stream, ctx, caches[index], following=following)
        rows = ctx.logit_rows
        logits = ctx.buffer("model.logits", (rows.shape[0], self.config.vocabulary),
                            torch.float32)
        if rows.shape[0] == 0:
            return logits
        last = self.final_norm.forward(stream, ctx, rows=rows, out_name="model.final_norm")
        ops.linear(last, self.output, out=logits, out_dtype=torch.float32)
        return logits


def expected_tensors(config: ModelConfig):
    """Names and shapes without building anything on a device."""
    model = DecoderModel(config, torch.float32, "meta")
    return model.expected_tensors()
