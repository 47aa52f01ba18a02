"""The Python entry point: ``Engine.submit`` / ``step`` / ``has_pending`` and ``generate``.

Names and meanings follow the reference where it has them: ``submit(request_id,
prompt_token_ids, max_new_tokens, eos_token_id)``, ``step()``, ``has_pending()`` and
``drain_completed()`` are the coordinator's interface (src/distengine/coordinator.py:141-152,
204, 460; protocol src/distengine/workload.py:217-230); a completion is the dict
``{request_id, prompt_token_ids, generated_token_ids, status, reason}``
(src/distengine/worker.py:66-73); ``generate_greedy(model, input_ids, max_new_tokens,
eos_token_id)`` mirrors src/utils/generation.py:49-54 and returns prompt plus generated ids.
"""

from __future__ import annotations

import time
from collections import deque

import torch

from ..cache.manager import CacheManager
from ..config.engine import EngineConfig
from ..models.loading import load_model
from ..sampling.sampler import Sampler, pack_sampling
from .request import Request
from .scheduler import Scheduler
from .step import StepEntry, StepRunner


class Engine:
    def __init__(self, model: "str | object", config: "EngineConfig | None" = None,
                 **overrides) -> None:
        """``model``: a model folder (config.json + model.safetensors) or a loaded model.
        ``overrides`` set fields of ``EngineConfig`` (dtype, block_size, num_blocks, ...)."""
        self.config = config or EngineConfig(**overrides)
        if config is not None and overrides:
            for key, value in overrides.items():
                setattr(self.config, key, value)
            self.config.__post_init__()
        cfg = self.config
        self.model = (load_model(model, cfg.dtype, cfg.device) if isinstance(model, str)
                      else model)
        device = self.model.device
        max_len = min(cfg.max_model_len or self.model.config.max_positions,
                      self.model.config.max_positions)
        specs = self.model.cache_specs()
        num_blocks = cfg.num_blocks
        if num_blocks is None:
            free, _ = torch.cuda.mem_get_info(device)
            per_page = CacheManager.bytes_per_page(specs, cfg.block_size, cfg.dtype)
            # no more than every slot at full length can ever use
            useful = cfg.decode_batch_size * ((max_len + cfg.block_size - 1) // cfg.block_size)
            num_blocks = max(1, min(int(free * cfg.memory_fraction) // max(per_page, 1), useful))
        self.cache = CacheManager(specs, [e.reads_cache_of for e in self.model.plan],
                                  cfg.block_size, num_blocks, cfg.decode_batch_size, max_len,
                                  cfg.dtype, device)
        self.sampler = Sampler(device, cfg.decode_batch_size)
        self.runner = StepRunner(self.model, self.cache, use_graphs=cfg.use_graphs,
                                 status=self.sampler.status)
        self.scheduler = Scheduler(self.cache, cfg.max_batch_tokens, cfg.decode_batch_size,
                                   max_len, self.model.config.vocabulary)
        self.completed: deque[dict] = deque()
        self._flying = None                     # (plan, sampler ticket) of the step that is running
        self.requests: dict[str, Request] = {}
        self.steps = 0
        self.tokens_fed = 0
        # for tests and debugging: called at every launch with [(request id, position)] and the
        # float32 logits [rows, vocabulary] at those places, which the next step overwrites (copy
        # them).  A step that is launched ahead and then taken back is reported too; the step
        # that redoes its positions reports them again.
        self.on_logits = None

    # ------------------------------------------------------------------ the reference's interface
    def submit(self, request_id: str, prompt_token_ids: list[int], max_new_tokens: int,
               eos_token_id: int, temperature: float = 0.0, seed: int = 0) -> None:
        """Validate and enqueue a request; nothing is allocated yet."""
        request = Request(request_id, prompt_token_ids, max_new_tokens, eos_token_id,
                          temperature, seed)
        self.scheduler.add(request)
        self.requests[request_id] = request

    def has_pending(self) -> bool:
        return self._flying is not None or self.scheduler.has_pending()

    def step(self) -> list[dict]:
        """Finish one batch: sample, account, finish and free.  Returns the completions of that
        step (they are also queued for ``drain_completed``).

        The GPU is kept one step ahead of the host.  While a step runs, the step after it is
        started if it can be foreseen (all running requests keep decoding one token): its
        positions, pages and work lists do not depend on the tokens being sampled, and the token
        ids themselves go from the sampler's output to the next step's input on the device.  Only
        then does the host wait for this step's tokens.  The plan always comes from the
        scheduler: a step that was started ahead counts only if it is exactly the plan the
        scheduler makes once the tokens are known; otherwise (an end-of-sequence token, a new
        request, a preemption) its cache lengths are taken back and the scheduler's plan runs.
        When this method returns, the next step, if there is one, is already running."""
        flying, self._flying = self._flying, None
        if flying is None:
            flying = self._start(self.scheduler.schedule())
            if flying is None:
                return []
        plan, ticket = flying
        ahead = self._start_ahead(plan)                       # before this step's tokens are known
        tokens = self.sampler.wait(ticket)
        self.runner.check_status(self.sampler.last_status)     # came to the host with the ids
        self.steps += 1
        self.tokens_fed += plan.num_tokens
        finished = self.scheduler.update(plan, tokens)
        if self.scheduler.has_pending():
            following = self.scheduler.schedule()
            if ahead is not None and self._same_step(ahead[0], following):
                for entry in ahead[0].entries:
                    self.cache.confirm(entry.request_id)
                self._flying = (following, ahead[1])
            else:
                if ahead is not None:
                    self._take_back(ahead[0])
                self._flying = self._start(following)
        elif ahead is not None:
            self._take_back(ahead[0])
        done = []
        for request in finished:
            record = request.snapshot()
            self.completed.append(record)
            self.requests.pop(request.request_id, None)
            done.append(record)
        return done

    def _start(self, plan):
        """Prepare and launch the scheduler's plan and its sampling; (plan, ticket) or None."""
        if not plan.entries:
            return None
        entries = [StepEntry(e.request.request_id, e.tokens,
                             [len(e.tokens) - 1] if e.sample else []) for e in plan.entries]
        sampling = [e.request for e in plan.entries if e.sample]
        # the sampled token will sit at position num_computed + len(portion) = len(known tokens)
        extra = pack_sampling([r.temperature for r in sampling], [r.seed for r in sampling],
                              [r.num_tokens for r in sampling])
        logits = self.runner.launch(self.runner.prepare(entries, extra))
        if self.on_logits is not None:
            self.on_logits([(e.request.request_id, e.request.num_computed + len(e.tokens) - 1)
                            for e in plan.entries if e.sample], logits)
        return plan, self.sampler.launch(logits, self.runner.last_arrays)

    @staticmethod
    def _same_step(prepared, plan) -> bool:
        mine = prepared.entries
        return (len(mine) == len(plan.entries)
                and all(a.request_id == b.request.request_id and len(b.tokens) == 1 and b.sample
                        for a, b in zip(mine, plan.entries)))

    def _start_ahead(self, plan):
        """Launch the step after ``plan`` (which is running) if it is sure to be one decoded
        token for every running request: every running request samples in ``plan``, none reaches
        its length limit, nothing waits, and the pages are there.  Returns (prepared step,
        sampler ticket) or None."""
        sched = self.scheduler
        running = sched.running
        if (sched.waiting or not running or len(plan.entries) != len(running)
                or len(running) > sched.max_seqs or len(running) > sched.max_batch_tokens):
            return None
        for entry, request in zip(plan.entries, running):
            if (entry.request is not request or not entry.sample
                    or request.num_generated_tokens + 1 >= request.max_new_tokens):
                return None
        need = sum(self.cache.pages_needed(r.request_id, self.cache.length(r.request_id) + 1)
                   for r in running)
        if need > self.cache.num_free_pages():
            return None
        entries = [StepEntry(r.request_id, [0], [0]) for r in running]
        extra = pack_sampling([r.temperature for r in running], [r.seed for r in running],
                              [r.num_tokens + 1 for r in running])
        prepared = self.runner.prepare(entries, extra)
        # the ids this step feeds are the ones the running step is about to sample
        logits = self.runner.launch(prepared, token_source=self.sampler.ids[: len(running)],
                                    tentative=True)
        if self.on_logits is not None:
            self.on_logits([(r.request_id, r.num_tokens) for r in running], logits)
        return prepared, self.sampler.launch(logits, self.runner.last_arrays)

    def _take_back(self, prepared) -> None:
        """A step that was started ahead and is not the scheduler's plan: its requests that still
        run go back to where they were: their lengths, and whatever fixed-size state the step
        advanced (keys and values that it wrote lie beyond the length and are written again; no
        page that a window had passed was given back meanwhile).  The GPU work itself is lost."""
        for entry in prepared.entries:
            if self.cache.has(entry.request_id):
                self.cache.rewind(entry.request_id)

    def drain_completed(self) -> list[dict]:
        results = list(self.completed)
        self.completed.clear()
        return results

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: list[list[int]], max_new_tokens: int, eos_token_id: int = -1,
                 temperature: float = 0.0, seed: int = 0) -> list[list[int]]:
        """Generate for every prompt (token ids in, generated token ids out, in order).  Request
        i samples with seed ``seed + i``."""
        base = f"gen-{time.monotonic_ns()}"
        ids = [f"{base}-{i}" for i in range(len(prompts))]
        for i, (rid, prompt) in enumerate(zip(ids, prompts)):
            self.submit(rid, list(prompt), max_new_tokens, eos_token_id, temperature, seed + i)
        results: dict[str, list[int]] = {}
        while self.has_pending():
            for record in self.step():
                results[record["request_id"]] = record["generated_token_ids"]
        self.drain_completed()
        return [results[rid] for rid in ids]


def generate_greedy(model, input_ids, max_new_tokens: int, eos_token_id: int,
                    **engine_options) -> torch.Tensor:
    """``input_ids`` [1, T] -> [1, T + generated], greedily, like the reference's
    ``generate_greedy`` (src/utils/generation.py:49-91); ``model`` is a model folder, a loaded
    model or an ``Engine``."""
    ids = torch.as_tensor(input_ids)
    if ids.ndim != 2 or ids.shape[0] != 1:
        raise ValueError("Expected input_ids with shape [1, T]")
    if ids.shape[1] == 0:
        raise ValueError("The prompt must contain at least one token")
    if max_new_tokens <= 0:
        raise ValueError("max_new_tokens must be positive")
    engine = model if isinstance(model, Engine) else Engine(model, **engine_options)
    prompt = [int(t) for t in ids[0].tolist()]
    generated = engine.generate([prompt], max_new_tokens, eos_token_id)[0]
    return torch.tensor([prompt + generated], dtype=ids.dtype, device=ids.device)
