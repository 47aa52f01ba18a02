"""The scheduler's decisions on the CPU, with the real cache manager and a stand-in for the step
function that fakes logits: budgets, portions, decode-first order, admission, finishing, and what
happens when pages run out."""

import pytest
import torch

from distengine_b200.cache import CacheManager
from distengine_b200.engine.request import Request, RequestStatus
from distengine_b200.engine.scheduler import Scheduler
from distengine_b200.parts.base import PagedKVSpec

VOCAB = 1000


def next_token(tokens):
    """A stand-in model: the next token is a function of the whole history."""
    h = 7
    for t in tokens:
        h = (h * 31 + t + 1) % 100003
    return h % VOCAB


class Harness:
    def __init__(self, pages=16, page=8, seqs=4, budget=32, max_len=512):
        self.cache = CacheManager([PagedKVSpec(1, 8, None)], [None], page, pages, seqs, max_len,
                                  torch.float32, "cpu")
        self.sched = Scheduler(self.cache, budget, seqs, max_len, VOCAB)
        self.history = []

    def step(self):
        plan = self.sched.schedule()
        # what StepRunner.step does with the cache
        for e in plan.entries:
            rid = e.request.request_id
            if not self.cache.has(rid):
                self.cache.admit(rid)
            assert self.cache.length(rid) == e.request.num_computed
        self.cache.reserve([(e.request.request_id, e.request.num_computed + len(e.tokens))
                            for e in plan.entries])
        sampled = []
        for e in plan.entries:
            rid = e.request.request_id
            self.cache.commit(rid, e.request.num_computed + len(e.tokens))
            assert e.tokens == e.request.token_ids[e.request.num_computed:
                                                   e.request.num_computed + len(e.tokens)]
            if e.sample:
                assert e.request.num_computed + len(e.tokens) == e.request.num_tokens
                sampled.append(next_token(e.request.token_ids))
        self.history.append(plan)
        finished = self.sched.update(plan, sampled)
        self.cache.check_invariants()
        return plan, finished

    def run(self, limit=10000):
        done = {}
        for _ in range(limit):
            if not self.sched.has_pending():
                return done
            _, finished = self.step()
            for r in finished:
                done[r.request_id] = r
        raise AssertionError("the scheduler did not finish")


def expected_generation(prompt, n, eos=-1):
    tokens, out = list(prompt), []
    for _ in range(n):
        t = next_token(tokens)
        out.append(t)
        tokens.append(t)
        if t == eos:
            break
    return out


def test_portions_under_the_token_budget_and_decode_first():
    h = Harness(budget=10, pages=32)
    h.sched.add(Request("a", list(range(23)), 3, -1))
    h.sched.add(Request("b", list(range(100, 104)), 2, -1))
    plan, _ = h.step()
    assert [(e.request.request_id, len(e.tokens), e.sample) for e in plan.entries] == [("a", 10, False)]
    plan, _ = h.step()
    assert [(e.request.request_id, len(e.tokens), e.sample) for e in plan.entries] == [("a", 10, False)]
    plan, _ = h.step()          # the prompt's rest, and the budget that is left admits b
    assert [(e.request.request_id, len(e.tokens), e.sample) for e in plan.entries] == [
        ("a", 3, True), ("b", 4, True)]
    plan, _ = h.step()          # both decode, one token each
    assert [(e.request.request_id, len(e.tokens), e.sample) for e in plan.entries] == [
        ("a", 1, True), ("b", 1, True)]
    assert all(p.num_tokens <= 10 for p in h.history)


def test_decoding_requests_come_before_prompt_portions():
    h = Harness(budget=8, pages=32)
    h.sched.add(Request("a", [1, 2, 3], 5, -1))
    h.step()
    h.sched.add(Request("b", list(range(30)), 2, -1))
    plan, _ = h.step()
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 7)]


def test_results_equal_uninterrupted_generation_and_everything_is_freed():
    h = Harness(budget=16, pages=64, seqs=3)
    prompts = {f"r{i}": list(range(i, i + n)) for i, n in enumerate([1, 9, 40, 70, 5])}
    for rid, p in prompts.items():
        h.sched.add(Request(rid, p, 12, -1))
    done = h.run()
    for rid, p in prompts.items():
        assert done[rid].generated_token_ids == expected_generation(p, 12)
        assert done[rid].reason == "length" and done[rid].status == RequestStatus.FINISHED
    assert h.cache.num_free_pages() == 64 and not h.cache.live and h.cache.slots.num_free == 3
    assert max(len({e.request.request_id for e in p.entries}) for p in h.history) <= 3


def test_eos_finishes_early_also_at_the_prompts_end():
    prompt = [5, 6, 7]
    first = next_token(prompt)
    h = Harness()
    h.sched.add(Request("a", prompt, 10, first))
    done = h.run()
    assert done["a"].generated_token_ids == [first] and done["a"].reason == "eos"
    assert h.cache.num_free_pages() == 16


def test_out_of_pages_preempts_the_newest_and_recomputes():
    # 6 pages of 8 tokens; two requests that together outgrow them
    h = Harness(pages=6, page=8, seqs=4, budget=64)
    h.sched.add(Request("old", list(range(20)), 20, -1))      # grows to 39 tokens: 5 pages
    h.sched.add(Request("new", list(range(50, 70)), 20, -1))  # the same
    done = h.run()
    assert h.sched.num_preemptions >= 1
    assert done["old"].generated_token_ids == expected_generation(list(range(20)), 20)
    assert done["new"].generated_token_ids == expected_generation(list(range(50, 70)), 20)
    assert done["old"].num_preemptions == 0 and done["new"].num_preemptions >= 1
    # after the preemption the victim fed its prompt and its generated tokens again
    fed = sum(len(e.tokens) for p in h.history for e in p.entries
              if e.request.request_id == "new")
    assert fed > 39
    assert sum(len(e.tokens) for p in h.history for e in p.entries
               if e.request.request_id == "old") == 39
    assert h.cache.num_free_pages() == 6 and not h.cache.live


def test_preempted_request_goes_to_the_front_of_the_queue():
    h = Harness(pages=6, page=8, seqs=4, budget=64)
    h.sched.add(Request("old", list(range(20)), 20, -1))
    h.sched.add(Request("new", list(range(50, 70)), 20, -1))
    h.sched.add(Request("later", [1, 2, 3], 2, -1))
    order = []
    while h.sched.has_pending():
        plan, finished = h.step()
        for p in plan.preempted:
            assert h.sched.waiting[0] is p or p in h.sched.running
        order += [r.request_id for r in finished]
    assert set(order) == {"old", "new", "later"}


def test_a_prompt_portion_is_shortened_to_the_free_pages():
    h = Harness(pages=4, page=8, budget=64)
    h.sched.add(Request("a", list(range(10)), 4, -1))
    h.step()                                              # a holds 2 pages
    h.sched.add(Request("b", list(range(30)), 1, -1))     # wants 4 pages, 2 are free
    plan, _ = h.step()
    got = {e.request.request_id: len(e.tokens) for e in plan.entries}
    assert got == {"a": 1, "b": 16}                        # two pages' worth


def test_requests_that_can_never_fit_are_refused_at_submission():
    h = Harness(pages=4, page=8, max_len=64)
    with pytest.raises(ValueError, match="KV capacity"):
        h.sched.add(Request("big", list(range(30)), 4, -1))       # 33 > 32
    h.sched.add(Request("fits", list(range(30)), 3, -1))           # the last token is never cached
    with pytest.raises(ValueError, match="length"):
        Harness(pages=64, max_len=40).sched.add(Request("long", list(range(30)), 11, -1))
    with pytest.raises(ValueError, match="already"):
        h.sched.add(Request("fits", [1], 1, -1))
    with pytest.raises(ValueError, match="vocabulary"):
        h.sched.add(Request("bad", [VOCAB], 1, -1))
    with pytest.raises(ValueError):
        Request("r", [], 1, -1)
    with pytest.raises(ValueError):
        Request("r", [1], 0, -1)


def test_slots_bound_the_live_requests():
    h = Harness(pages=64, seqs=2, budget=64)
    for i in range(5):
        h.sched.add(Request(f"r{i}", [i + 1, i + 2], 3, -1))
    plan, _ = h.step()
    assert len(plan.entries) == 2 and len(h.sched.waiting) == 3
    done = h.run()
    assert len(done) == 5
