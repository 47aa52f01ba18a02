"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees; and decides what happens when pages run out.

Every step it plans one batch for the step function:

1. Running requests that have one token left to feed (decoding) come first, one token each.
2. Running requests whose prompt is not yet in the cache get the next portion of it, as large as
   the remaining token budget and the free pages allow.
3. Waiting requests are admitted first-in first-out while a slot is free, budget is left and the
   pages for their first portion are free.

A request's *known tokens* are its prompt plus what it generated.  It always feeds
``tokens[num_computed:]`` (a portion of it); when a step feeds its last known token, the logits
at that token are wanted and a new token is sampled.  Decoding is the case of one known token left.

When pages run out: pages are taken on demand, page by page (the reference reserves a request's
whole ``P + max_new - 1`` before decoding, src/distengine/coordinator.py:403-406, so its decode
never runs out; its prefill simply waits, PROGRESS.md:162-170).  Here a decoding request that
finds no free page preempts the most recently admitted running request: that request gives back
all its pages and its slot, keeps its tokens, and goes to the front of the waiting queue; when it
is admitted again its prompt and generated tokens are recomputed in portions.  A prompt portion
that finds too few pages is shortened or waits.  If no running request can feed anything, the most
recently admitted one is preempted too, so the oldest always makes progress.  A request that could
never fit is refused at ``add`` (src/distengine/coordinator.py:183-186).

Kept from the reference: first-in first-out admission (:192-194), finish rules and immediate
release on finish (src/distengine/request.py:53-63, src/distengine/worker.py:332-334), at most
``decode_batch_size`` requests in a decode batch (:417-421).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from .request import Request, RequestStatus


@dataclass
class PlannedEntry:
    request: Request
    tokens: list[int]
    sample: bool                  # the portion ends at the last known token: logits are wanted


@dataclass
class Plan:
    entries: list[PlannedEntry] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache, max_batch_tokens: int, max_seqs: int, max_model_len: int,
                 vocabulary: int) -> None:
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_seqs = min(max_seqs, cache.max_seqs)
        self.max_model_len = max_model_len
        self.vocabulary = vocabulary
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []               # in order of admission
        self.seen_ids: set[str] = set()
        self.num_preemptions = 0

    # ------------------------------------------------------------------ admission
    def add(self, request: Request) -> None:
        """Validate and enqueue; nothing is allocated (src/distengine/coordinator.py:146-194)."""
        if request.request_id in self.seen_ids:
            raise ValueError("Request ID has already been submitted")
        for token_id in request.prompt_token_ids:
            if type(token_id) is not int:
                raise ValueError("Token IDs must be integers")
            if not 0 <= token_id < self.vocabulary:
                raise ValueError("Token ID is outside the model vocabulary")
        most = request.num_prompt_tokens + request.max_new_tokens - 1     # the last token is never cached
        if most > self.cache.capacity_tokens:
            raise ValueError(f"Request exceeds KV capacity: it may hold {most} tokens, the pool "
                             f"has room for {self.cache.capacity_tokens}")
        if request.num_prompt_tokens + request.max_new_tokens > self.max_model_len:
            raise ValueError(f"Request exceeds the model's length: prompt "
                             f"{request.num_prompt_tokens} + max_new_tokens "
                             f"{request.max_new_tokens} > {self.max_model_len}")
        self.seen_ids.add(request.request_id)
        self.waiting.append(request)

    def has_pending(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _preempt(self, victim: Request, plan: Plan) -> None:
        self.running.remove(victim)
        if self.cache.has(victim.request_id):
            self.cache.release(victim.request_id)
        victim.num_computed = 0
        victim.num_preemptions += 1
        victim.status = RequestStatus.WAITING
        self.waiting.appendleft(victim)
        self.num_preemptions += 1
        plan.preempted.append(victim)
        plan.entries = [e for e in plan.entries if e.request is not victim]

    def _pages_for(self, request: Request, count: int) -> int:
        if not self.cache.has(request.request_id):
            page = self.cache.page_size
            return (count + page - 1) // page
        return self.cache.pages_needed(request.request_id, request.num_computed + count)

    def schedule(self) -> Plan:
        plan = Plan()
        while True:
            plan.entries = []
            budget = self.max_batch_tokens
            free = self.cache.num_free_pages()
            victim = None
            # 1. decoding requests, oldest first
            decoding = [r for r in self.running if r.num_tokens - r.num_computed == 1]
            for request in decoding[: self.max_seqs]:
                if budget < 1:
                    break
                need = self._pages_for(request, 1)
                if need > free:
                    victim = self.running[-1]
                    break
                free -= need
                budget -= 1
                plan.entries.append(PlannedEntry(request, request.tokens_from(request.num_tokens - 1, 1),
                                                 True))
            if victim is not None:
                self._preempt(victim, plan)
                continue
            # 2. prompts in progress
            for request in self.running:
                left = request.num_tokens - request.num_computed
                if left <= 1 or budget <= 0:
                    continue
                count = self._fit(request, min(left, budget), free)
                if count == 0:
                    continue
                free -= self._pages_for(request, count)
                budget -= count
                tokens = request.tokens_from(request.num_computed, count)
                plan.entries.append(PlannedEntry(request, tokens, count == left))
            # 3. admissions
            while (self.waiting and budget > 0 and len(self.running) < self.max_seqs
                   and self.cache.slots.num_free > len(self._new_in(plan))):
                request = self.waiting[0]
                left = request.num_tokens - request.num_computed
                count = self._fit(request, min(left, budget), free)
                if count == 0:
                    break
                self.waiting.popleft()
                request.status = RequestStatus.RUNNING
                self.running.append(request)
                free -= self._pages_for(request, count)
                budget -= count
                tokens = request.tokens_from(0, count)
                plan.entries.append(PlannedEntry(request, tokens, count == left))
            if plan.entries or not self.running:
                if not plan.entries and self.waiting:
                    raise RuntimeError("Pending requests cannot make progress")
                return plan
            # nothing could be fed although requests are running: free the newest one's pages
            self._preempt(self.running[-1], plan)

    def _new_in(self, plan: Plan) -> list[Request]:
        return [e.request for e in plan.entries if not self.cache.has(e.request.request_id)]

    def _fit(self, request: Request, count: int, free_pages: int) -> int:
        """The largest portion of at most ``count`` tokens whose pages are free."""
        while count > 0 and self._pages_for(request, count) > free_pages:
            page = self.cache.page_size
            # drop the tokens of the last page touched
            end = request.num_computed + count
            count = max(0, ((end - 1) // page) * page - request.num_computed)
        return count

    # ------------------------------------------------------------------ after a step
    def update(self, plan: Plan, sampled: list[int]) -> list[Request]:
        """Account a finished step: ``sampled`` holds one token for every entry with ``sample``,
        in order.  Returns the requests that finished; their pages and slots are given back."""
        finished = []
        it = iter(sampled)
        for entry in plan.entries:
            request = entry.request
            request.num_computed += len(entry.tokens)
            if not entry.sample:
                continue
            request.append_token(int(next(it)))
            if request.is_finished:
                self.running.remove(request)
                self.cache.release(request.request_id)
                finished.append(request)
        return finished
