"""The request-level benchmark's bookkeeping, driven with a fake engine and a fake clock: when
requests are submitted, which step's time a token gets, the measures of a request
(src/distengine/metric.py:33-49), the quantiles (:52-62) and the figures over repeats
(src/utils/benchmark.py:52-81)."""

import math

import pytest

from distengine_b200.engine import benchmark as bm


class FakeClock:
    def __init__(self):
        self.now = 0.0

    def __call__(self):
        return self.now

    def sleep(self, seconds):
        self.now += max(seconds, 1e-3)


class FakeRequest:
    def __init__(self, budget):
        self.budget, self.num_generated_tokens = budget, 0


class FakeEngine:
    """Every step takes ``step_s`` on the fake clock and gives each live request one token; a
    request's first step (its prompt) takes ``prefill_s`` more."""

    def __init__(self, clock, step_s=0.010, prefill_s=0.005):
        self.clock, self.step_s, self.prefill_s = clock, step_s, prefill_s
        self.requests = {}
        self.submitted = []

    def submit(self, request_id, prompt, max_new_tokens, eos, temperature, seed):
        self.requests[request_id] = FakeRequest(max_new_tokens)
        self.submitted.append((request_id, self.clock.now, len(prompt), seed))

    def has_pending(self):
        return bool(self.requests)

    def step(self):
        fresh = any(r.num_generated_tokens == 0 for r in self.requests.values())
        self.clock.now += self.step_s + (self.prefill_s if fresh else 0.0)
        done = []
        for rid, request in list(self.requests.items()):
            request.num_generated_tokens += 1
            if request.num_generated_tokens == request.budget:
                done.append({"request_id": rid,
                             "generated_token_ids": [7] * request.budget})
                del self.requests[rid]
        return done


def test_percentile_interpolates_between_sorted_observations():
    assert bm.percentile([], 0.5) is None
    assert bm.percentile([3.0], 0.99) == 3.0
    assert bm.percentile([4.0, 1.0, 3.0, 2.0], 0.5) == pytest.approx(2.5)
    assert bm.percentile([1.0, 2.0, 3.0, 4.0, 5.0], 0.95) == pytest.approx(4.8)
    assert bm.percentile([1.0, 2.0], 0.0) == 1.0 and bm.percentile([1.0, 2.0], 1.0) == 2.0


def test_workload_is_seeded_and_poisson_or_burst():
    a = bm.make_workload(6, [1, 8, 16], 4, vocabulary=50, seed=42, rate_rps=100.0)
    b = bm.make_workload(6, [1, 8, 16], 4, vocabulary=50, seed=42, rate_rps=100.0)
    assert a == b
    assert [len(r.prompt_token_ids) for r in a] == [1, 8, 16, 1, 8, 16]
    assert a[0].arrival_s == 0.0
    assert all(x.arrival_s < y.arrival_s for x, y in zip(a, a[1:]))
    assert all(0 <= t < 50 for r in a for t in r.prompt_token_ids)
    burst = bm.make_workload(3, [5], 2, vocabulary=9, seed=1)
    assert [r.arrival_s for r in burst] == [0.0, 0.0, 0.0]
    assert bm.make_workload(6, [1, 8, 16], 4, 50, seed=43, rate_rps=100.0) != a
    with pytest.raises(ValueError):
        bm.make_workload(0, [1], 1, 10)
    with pytest.raises(ValueError):
        bm.make_workload(1, [0], 1, 10)
    with pytest.raises(ValueError):
        bm.make_workload(1, [1], 1, 10, rate_rps=-1.0)


def test_requests_are_submitted_when_due_and_tokens_timed_by_the_step_that_gave_them():
    clock = FakeClock()
    engine = FakeEngine(clock)
    workload = [bm.BenchRequest("a", 0.0, (1, 2, 3), 3),
                bm.BenchRequest("b", 0.012, (4,), 2),
                bm.BenchRequest("c", 0.500, (5, 6), 1)]          # arrives when the engine is idle
    report = bm.run_workload(engine, workload, seed=10, clock=clock, sleep=clock.sleep)
    # a at once; b after the first step (0.015 >= 0.012); c once its time has come
    assert [(rid, n, seed) for rid, _, n, seed in engine.submitted] == \
        [("a", 3, 10), ("b", 1, 11), ("c", 2, 12)]
    when = {rid: t for rid, t, _, _ in engine.submitted}
    assert when["a"] == 0.0 and when["b"] == pytest.approx(0.015) and when["c"] >= 0.5
    rows = report["per_request"]
    # a: tokens at 0.015, 0.030 (b's first step is a prompt step too), 0.040
    assert rows["a"]["output_tokens"] == 3
    assert rows["a"]["ttft_s"] == pytest.approx(0.015)
    assert rows["a"]["e2e_s"] == pytest.approx(0.040)
    assert rows["a"]["tpot_s"] == pytest.approx((0.040 - 0.015) / 2)
    # b: submitted at 0.015, tokens at 0.030 and 0.040
    assert rows["b"]["ttft_s"] == pytest.approx(0.015)
    assert rows["b"]["tpot_s"] == pytest.approx(0.010)
    assert rows["b"]["submission_delay_s"] == pytest.approx(0.003)
    # c: one token: no time per output token
    assert rows["c"]["tpot_s"] is None and rows["c"]["output_tokens"] == 1
    assert report["completed"] == 3 and report["output_tokens"] == 6
    assert report["request_throughput_rps"] == pytest.approx(3 / report["elapsed_s"])
    assert report["completed_output_tokens_per_s"] == pytest.approx(6 / report["elapsed_s"])
    assert report["goodput_rps"] == report["request_throughput_rps"]
    assert report["latencies"]["ttft_s"]["p50"] == pytest.approx(0.015)


def test_goodput_counts_requests_within_all_three_limits():
    fast = bm._Timing(0.0, 0.0, [0.01, 0.02, 0.03], 0.03)
    slow_first = bm._Timing(0.0, 0.0, [3.0, 3.01], 3.01)
    slow_tokens = bm._Timing(0.0, 0.0, [0.01, 0.5], 0.5)
    unfinished = bm._Timing(0.0, 0.0, [0.01], None)
    report = bm.summarize({"a": fast, "b": slow_first, "c": slow_tokens, "d": unfinished}, 2.0)
    assert report["completed"] == 3 and report["requests"] == 4
    assert report["request_throughput_rps"] == pytest.approx(1.5)
    assert report["goodput_rps"] == pytest.approx(0.5)
    with pytest.raises(ValueError):
        bm.LatencyLimits(ttft_s=0.0)
    with pytest.raises(ValueError):
        bm.LatencyLimits(e2e_s=math.inf)


def test_aggregate_gives_mean_and_spread_over_repeats():
    runs = []
    for step_s in (0.010, 0.020):
        clock = FakeClock()
        engine = FakeEngine(clock, step_s=step_s, prefill_s=0.0)
        runs.append(bm.run_workload(engine, bm.make_workload(4, [2], 3, 11), clock=clock,
                                    sleep=clock.sleep))
    out = bm.aggregate(runs)
    assert out["executed_repeats"] == 2
    rate = out["aggregate"]["completed_output_tokens_per_s"]
    assert rate["values"] == pytest.approx([12 / 0.030, 12 / 0.060])
    assert rate["mean"] == pytest.approx(300.0) and rate["stdev"] > 0
    assert out["latency_across_runs"]["ttft_s"]["p99"]["values"] == pytest.approx([0.010, 0.020])
    assert out["latency_across_runs"]["tpot_s"]["p50"]["mean"] == pytest.approx(0.015)
    assert bm.aggregate(runs[:1])["aggregate"]["goodput_rps"]["stdev"] is None
