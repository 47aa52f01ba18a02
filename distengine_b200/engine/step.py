"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step holds prompt portions of any length beside single decoded tokens, cut anywhere.  It runs
only the tokens it is given, as one ragged batch, against the keys and values that earlier steps
left in the pages, and returns float32 logits at the wanted places.  It samples nothing and keeps
no request state beyond the cache's lengths; the scheduler and the trace replay both drive it.

The reference's nearest relative is ``ModelRunner`` (src/distengine/model_runner.py): ``prefill``
runs one whole prompt (:113-173), ``decode_batch`` runs B single tokens (:226-269); a batch there
is never mixed and a prompt never cut.  Kept from it: tokens are validated against the vocabulary
(:72-77), positions continue from the cache's length (src/models/llama.py:177-179), pages for the
whole batch are taken before anything is written or the step does not start (:244-256), and all
per-step index arrays are built once on the host and reused by every layer
(src/distengine/paged_kv_cache.py:263-293).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..parts.context import StepContext, StepPrep, Workspace


@dataclass
class StepEntry:
    request_id: str
    tokens: list[int]
    want: list[int] = field(default_factory=list)      # places among ``tokens``


@dataclass
class PreparedStep:
    """A step whose host half is done (see ``StepRunner.prepare``)."""
    entries: list
    host: SimpleNamespace
    prep: StepPrep
    graph_shape: "dict | None"
    views: dict
    offsets: list
    total: int


class KernelStatusError(RuntimeError):
    """A kernel found an index it could not use (a position without a page) and skipped work."""


MAX_GRAPHS = 128        # shapes of steps kept as CUDA graphs at a time
PORTION_REPEATS = 3     # a step with prompt portions is shaped for replay after this many like it


def _align(n: int) -> int:
    return (n + 3) & ~3


class StepRunner:
    def __init__(self, model, cache: CacheManager, use_graphs: bool = False,
                 status: "torch.Tensor | None" = None) -> None:
        """``status``: the int32 [1] device word in which kernels record skipped work; the
        runner makes its own unless the caller wants it somewhere (beside the sampled ids, so
        that it comes to the host with them)."""
        self.model, self.cache = model, cache
        self.device, self.dtype = model.device, model.dtype
        ops.require_device(self.device)
        self.vocabulary = model.config.vocabulary
        self.workspace = Workspace(self.device)
        self.status = (status if status is not None
                       else torch.zeros(1, dtype=torch.int32, device=self.device))
        self._host_meta: "torch.Tensor | None" = None        # pinned int32 staging
        self._dev_meta: "torch.Tensor | None" = None
        self._uploaded = torch.cuda.Event()
        self._upload_pending = False
        self.bindings = cache.bindings()
        self.use_graphs = use_graphs
        self.steps_run = 0
        self.last_arrays: dict[str, torch.Tensor] = {}
        # steps replayed as CUDA graphs: key -> (graph, logits, kernels in it, generation)
        self._graphs: dict[tuple, tuple] = {}
        # how often a shape of step with prompt portions has come (such a step is shaped for
        # replay once it has come PORTION_REPEATS times; steps of single tokens always are)
        self._portion_shapes: dict[tuple, int] = {}
        self._meta_generation = 0
        self._layouts: dict[tuple, tuple] = {}
        self.graph_replays = 0

    # ------------------------------------------------------------------ host side
    def _validate(self, entries: list[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if not isinstance(e.request_id, str) or not e.request_id:
                raise ValueError("request_id must be a nonempty string")
            if e.request_id in seen:
                raise ValueError(f"request '{e.request_id}' appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise ValueError(f"request '{e.request_id}': a step entry needs at least one token")
            if len(e.tokens) <= 8:
                for t in e.tokens:
                    if type(t) is not int:
                        raise ValueError("Token IDs must be integers")
                    if not 0 <= t < self.vocabulary:
                        raise ValueError(f"token id {t} is outside the model vocabulary "
                                         f"[0, {self.vocabulary})")
            else:
                # a prompt portion: the types in one pass of C code, the range as an array
                if set(map(type, e.tokens)) != {int}:
                    raise ValueError("Token IDs must be integers")
                ids = np.asarray(e.tokens)
                if ids.dtype != np.int64:                  # numbers beyond 64 bits
                    raise ValueError("Token IDs must be integers")
                if int(ids.min()) < 0 or int(ids.max()) >= self.vocabulary:
                    bad = int(ids[(ids < 0) | (ids >= self.vocabulary)][0])
                    raise ValueError(f"token id {bad} is outside the model vocabulary "
                                     f"[0, {self.vocabulary})")
            for w in e.want:
                if type(w) is not int or not 0 <= w < len(e.tokens):
                    raise ValueError(f"request '{e.request_id}': wanted place {w} is not among its "
                                     f"{len(e.tokens)} tokens")

    def _host_arrays(self, entries: list[StepEntry]) -> SimpleNamespace:
        lens = np.array([len(e.tokens) for e in entries], dtype=np.int32)
        n, s = int(lens.sum()), len(entries)
        pos0 = np.array([self.cache.length(e.request_id) for e in entries], dtype=np.int32)
        slots = np.array([self.cache.slot(e.request_id) for e in entries], dtype=np.int32)
        qstart = (np.cumsum(lens) - lens).astype(np.int32)
        token_seq = np.repeat(np.arange(s, dtype=np.int32), lens)
        offsets = np.arange(n, dtype=np.int32) - qstart[token_seq]
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        rows = np.array([qstart[i] + w for i, e in enumerate(entries) for w in e.want],
                        dtype=np.int32)
        return SimpleNamespace(
            n_tokens=n, n_seqs=s, token_ids=token_ids, positions=pos0[token_seq] + offsets,
            token_slot=slots[token_seq], token_seq=token_seq, seq_slot=slots, seq_qstart=qstart,
            seq_qlen=lens, seq_pos0=pos0, logit_rows=rows,
            request_ids=[e.request_id for e in entries])

    _BASE = ("token_ids", "positions", "token_slot", "token_seq", "seq_slot", "seq_qstart",
             "seq_qlen", "seq_pos0", "logit_rows")

    def _stage(self, host: SimpleNamespace, prep: StepPrep) -> "tuple[dict, list, int, list]":
        """Lay the step's arrays out in the pinned staging buffer.  Returns the device views, the
        offsets, the number of ints and the arrays."""
        arrays = [(name, getattr(host, name)) for name in self._BASE]
        arrays += list(prep.extra.items())
        total = sum(_align(a.size) for _, a in arrays)
        if self._host_meta is None or self._host_meta.numel() < total:
            cap = max(total * 2, 4096)
            self._host_meta = torch.empty(cap, dtype=torch.int32).pin_memory()
            self._dev_meta = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_generation += 1
            self._layouts = {}
        self.upload_bytes = total * 4
        if self._upload_pending:
            self._uploaded.synchronize()          # the staging buffer is free again
            self._upload_pending = False
        stage = self._host_meta.numpy()
        # where each array lies depends on the arrays' names and shapes only: keep the device
        # views of a layout (steady decoding repeats one layout step after step)
        layout_key = tuple((name, array.shape) for name, array in arrays)
        layout = self._layouts.get(layout_key)
        if layout is None:
            views, offsets, offset = {}, [], 0
            for name, array in arrays:
                views[name] = self._dev_meta[offset: offset + array.size].view(array.shape)
                offsets.append(offset)
                offset += _align(array.size)
            layout = self._layouts[layout_key] = (views, offsets)
        views, offsets = layout
        for (name, array), offset in zip(arrays, offsets):
            stage[offset: offset + array.size] = array.reshape(-1)
        return views, offsets, total, arrays

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: list[StepEntry],
                extra: "dict[str, np.ndarray] | None" = None) -> "PreparedStep":
        """The host half of a step: validate, admit, take pages, build the step's arrays and lay
        them out for upload.  Nothing is launched.  Only one prepared step may be outstanding: it
        owns the staging buffer until ``launch`` (or until another ``prepare`` replaces it).
        Raises ``OutOfPages`` (nothing changed) when the pool cannot hold the step's tokens."""
        self._validate(entries)
        admitted = []
        try:
            for e in entries:
                if not self.cache.has(e.request_id):
                    self.cache.admit(e.request_id)
                    admitted.append(e.request_id)
            self.cache.reserve([(e.request_id, self.cache.length(e.request_id) + len(e.tokens))
                                for e in entries])
        except Exception:
            for request_id in admitted:
                self.cache.release(request_id)
            raise
        host = self._host_arrays(entries)
        graph_shape = None
        if self.use_graphs and getattr(self.model, "graph_safe", True):
            # shape the step's arrays by the batch's shape only, so that it can be replayed; the
            # key range is capped at the next multiple of 512 positions.  Every step of single
            # tokens; a step with prompt portions once the same portions (their lengths, the cap,
            # the wanted rows) have come PORTION_REPEATS times - a long prompt's full portions, a
            # benchmark's prompts - since shaping costs padding and a capture costs more than a
            # step (measured: requests of random lengths through the scheduler, every shape
            # twice, lose 7 % when the second coming is already shaped and the third captured)
            longest = int((host.seq_pos0.astype(np.int64) + host.seq_qlen).max())
            cap = (longest + 511) // 512 * 512
            if int(host.seq_qlen.max()) == 1:
                graph_shape = {"context_cap": cap}
            else:
                shape = (host.seq_qlen.tobytes(), cap, len(host.logit_rows))
                if len(self._portion_shapes) > 512 and shape not in self._portion_shapes:
                    self._portion_shapes.clear()
                count = self._portion_shapes[shape] = self._portion_shapes.get(shape, 0) + 1
                if count > PORTION_REPEATS:
                    graph_shape = {"context_cap": cap}
        prep = StepPrep(host, graph_shape)
        self.model.prepare(prep)
        for name, array in (extra or {}).items():
            prep.add(name, array)
        views, offsets, total, arrays = self._stage(host, prep)
        return PreparedStep(entries, host, prep, graph_shape, views, offsets, total)

    def launch(self, prepared: "PreparedStep", token_source: "torch.Tensor | None" = None,
               tentative: bool = False) -> torch.Tensor:
        """The device half: upload the prepared arrays, run the model, advance the cache's
        lengths.  Returns logits float32 [wanted, vocabulary] on the device, in the order of the
        entries and of each entry's ``want``; the tensor is reused by the next step.
        ``token_source`` (int32 on the device, one id per token of the step): the token ids are
        taken from there instead of from the prepared arrays - ids that an earlier kernel in the
        stream produces and the host has not seen yet.
        ``tentative``: the caller may take the step back (``CacheManager.rewind``) or make it
        final (``CacheManager.confirm``): the cache keeps everything that a redo would need."""
        host, prep, views = prepared.host, prepared.prep, prepared.views
        if tentative:
            self.cache.save_states([e.request_id for e in prepared.entries])
        total = prepared.total
        self._dev_meta[:total].copy_(self._host_meta[:total], non_blocking=True)
        if token_source is not None:
            if token_source.dtype != torch.int32 or token_source.numel() != host.n_tokens:
                raise ValueError("token_source must hold one int32 id for each token of the step")
            views["token_ids"].copy_(token_source.view(-1), non_blocking=True)
        self.cache.flush_tables()
        self._uploaded.record()
        self._upload_pending = True
        ctx = StepContext(
            device=self.device, dtype=self.dtype, n_tokens=host.n_tokens, n_seqs=host.n_seqs,
            token_ids=views["token_ids"], positions=views["positions"],
            token_slot=views["token_slot"], token_seq=views["token_seq"],
            seq_slot=views["seq_slot"], seq_qstart=views["seq_qstart"],
            seq_qlen=views["seq_qlen"], seq_pos0=views["seq_pos0"],
            logit_rows=views["logit_rows"], host=host,
            arrays={k: v for k, v in views.items() if k not in self._BASE},
            notes=prep.notes, workspace=self.workspace, status=self.status)
        self.last_arrays = ctx.arrays
        if prepared.graph_shape is None:
            logits = self.model.forward(ctx, self.bindings)
        else:
            logits = self._forward_graphed(ctx, prep, prepared.graph_shape)
        for e in prepared.entries:
            self.cache.commit(e.request_id, self.cache.length(e.request_id) + len(e.tokens),
                              tentative=tentative)
        self.steps_run += 1
        return logits

    def step(self, entries: list[StepEntry],
             extra: "dict[str, np.ndarray] | None" = None) -> torch.Tensor:
        """Run the entries as one batch: ``prepare`` then ``launch``.  ``extra``: int32 arrays of
        the caller's that travel to the device with the step's own arrays
        (``self.last_arrays[name]`` afterwards)."""
        return self.launch(self.prepare(entries, extra))

    def set_tokens(self, prepared: "PreparedStep", tokens: list[int]) -> None:
        """Put the token ids into a step that was prepared before they were known (one token per
        entry): everything else of a decode step - positions, pages, work lists - does not depend
        on them, so it can be prepared while the previous step still runs."""
        if len(tokens) != prepared.host.n_tokens:
            raise ValueError("one token for each token of the prepared step")
        for t in tokens:
            if type(t) is not int or not 0 <= t < self.vocabulary:
                raise ValueError(f"token id {t} is outside the model vocabulary")
        ids = np.asarray(tokens, dtype=np.int32)
        prepared.host.token_ids = ids
        offset = prepared.offsets[0]                       # token_ids is the first array
        self._host_meta.numpy()[offset: offset + ids.size] = ids
        for e, t in zip(prepared.entries, tokens):
            e.tokens = [t]

    def _forward_graphed(self, ctx: StepContext, prep: StepPrep, graph_shape: dict) -> torch.Tensor:
        """Replay the step of this shape as a CUDA graph; the first step of a shape runs
        as it is (which also brings every scratch buffer to its size), the second is captured.
        The graph reads the step's arrays from the same device addresses every time; only their
        contents change."""
        key = (ctx.host.seq_qlen.tobytes(), graph_shape["context_cap"], ctx.logit_rows.shape[0],
               tuple((name, array.shape) for name, array in prep.extra.items()),
               tuple(sorted(prep.notes.items())))
        stamp = (self.workspace.generation, self._meta_generation)
        entry = self._graphs.get(key)
        if entry is not None and entry[3] != stamp:
            self._graphs.clear()                       # buffers moved: every graph is stale
            entry = None
        if entry is None:
            if len(self._graphs) >= MAX_GRAPHS:        # steps of ever new shapes: start over
                self._graphs.clear()
            logits = self.model.forward(ctx, self.bindings)
            self._graphs[key] = (None, logits, 0, (self.workspace.generation,
                                                    self._meta_generation))
            return logits
        graph, logits, kernels, _ = entry
        if graph is None:
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx, self.bindings)
            kernels = ops.launch_count - before
            ops.launch_count = before
            self._graphs[key] = (graph, logits, kernels, stamp)
        graph.replay()
        ops.launch_count += kernels
        self.graph_replays += 1
        return logits

    def release(self, request_id: str) -> None:
        self.cache.release(request_id)

    def check_status(self, code: "int | None" = None) -> None:
        """Raises if a kernel skipped work since the last check.  ``code``: the status word as
        the caller has already read it; without it the word is read here (a synchronisation)."""
        if code is None:
            code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            what = {1: "a token's position had no page in its request's block table",
                    2: "a key that a token reads had no page in its request's block table",
                    3: "a bounded wait inside a tcgen05 kernel ran out",
                    4: "a tcgen05 kernel found its shared memory misaligned"}.get(
                        code, "unknown code")
            raise KernelStatusError(f"a kernel reported status {code}: {what}")
