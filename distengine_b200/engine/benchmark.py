"""A request set run through ``Engine`` and what the requests saw of it.

The reference's benchmark (src/utils/benchmark.py:84-170) replays a set of requests with arrival
times through its serving stack and reports, from the driver's clock, request throughput, output
tokens a second and the quantiles of three latencies a request; the measures are defined in
src/distengine/metric.py:33-49 (a request's time to its first token, its time per output token
after the first, its time from submission to its end) and :52-62 (quantiles by linear
interpolation between the sorted observations).  This module keeps those names and meanings for
the one-GPU engine: no server, no workers, the loop that steps the engine is the driver.

Host-side only; the engine is anything with ``submit``, ``step``, ``has_pending`` and
``requests`` (tests drive it with a fake).
"""

from __future__ import annotations

import math
import statistics
import time
from dataclasses import dataclass, field

import numpy as np

QUANTILES = (("p50", 0.50), ("p95", 0.95), ("p99", 0.99))
LATENCIES = ("ttft_s", "tpot_s", "e2e_s")
RATES = ("request_throughput_rps", "completed_output_tokens_per_s", "goodput_rps")


@dataclass(frozen=True)
class LatencyLimits:
    """A request counts towards goodput when it stays within all three
    (the reference's defaults: src/utils/benchmark.py:141)."""
    ttft_s: float = 2.0
    tpot_s: float = 0.1
    e2e_s: float = 10.0

    def __post_init__(self) -> None:
        for value in (self.ttft_s, self.tpot_s, self.e2e_s):
            if not math.isfinite(value) or value <= 0:
                raise ValueError("latency limits must be finite and positive")


@dataclass(frozen=True)
class BenchRequest:
    request_id: str
    arrival_s: float                     # when the request is due, from the start of the run
    prompt_token_ids: tuple[int, ...]
    max_new_tokens: int


@dataclass
class _Timing:
    arrival_s: float
    submitted_s: float
    token_s: list[float] = field(default_factory=list)     # when each output token was seen
    finished_s: "float | None" = None


def make_workload(num_requests: int, prompt_lengths: list[int], max_new_tokens: int,
                  vocabulary: int, seed: int = 0, rate_rps: float = 0.0) -> list[BenchRequest]:
    """``num_requests`` requests with uniform random token ids; request i's prompt has
    ``prompt_lengths[i % len(prompt_lengths)]`` tokens.  ``rate_rps`` 0: all due at the start;
    otherwise arrivals of a Poisson process of that rate (exponential gaps), from ``seed``."""
    if num_requests <= 0 or max_new_tokens <= 0 or vocabulary <= 0:
        raise ValueError("num_requests, max_new_tokens and vocabulary must be positive")
    if not prompt_lengths or min(prompt_lengths) <= 0:
        raise ValueError("prompt lengths must be positive")
    if not math.isfinite(rate_rps) or rate_rps < 0:
        raise ValueError("rate_rps must be finite and not negative")
    rng = np.random.default_rng(seed)
    arrival = 0.0
    requests = []
    for i in range(num_requests):
        if rate_rps > 0 and i > 0:
            arrival += float(rng.exponential(1.0 / rate_rps))
        length = prompt_lengths[i % len(prompt_lengths)]
        tokens = tuple(int(t) for t in rng.integers(0, vocabulary, size=length))
        requests.append(BenchRequest(f"bench-{i}", arrival, tokens, max_new_tokens))
    return requests


def percentile(values: list[float], fraction: float) -> "float | None":
    """Linear interpolation between the sorted observations (src/distengine/metric.py:52-62)."""
    if not values:
        return None
    ordered = sorted(values)
    position = (len(ordered) - 1) * fraction
    lower, upper = math.floor(position), math.ceil(position)
    return ordered[lower] + (ordered[upper] - ordered[lower]) * (position - lower)


def request_measures(timing: _Timing) -> dict:
    """src/distengine/metric.py:33-49: first token and end count from the submission, the time
    per output token is the span from the first to the last token over the tokens after the
    first."""
    tokens = timing.token_s
    first = tokens[0] if tokens else None
    return {
        "output_tokens": len(tokens),
        "submission_delay_s": timing.submitted_s - timing.arrival_s,
        "ttft_s": first - timing.submitted_s if first is not None else None,
        "tpot_s": (tokens[-1] - first) / (len(tokens) - 1) if len(tokens) > 1 else None,
        "e2e_s": (timing.finished_s - timing.submitted_s
                  if timing.finished_s is not None else None),
    }


def summarize(timings: dict[str, _Timing], elapsed_s: float,
              limits: "LatencyLimits | None" = None) -> dict:
    """The run's figures from the requests' timings."""
    limits = limits or LatencyLimits()
    rows = {rid: request_measures(t) for rid, t in timings.items()}
    done = [m for m in rows.values() if m["e2e_s"] is not None]
    good = [m for m in done
            if m["ttft_s"] is not None and m["ttft_s"] <= limits.ttft_s
            and m["e2e_s"] <= limits.e2e_s
            and (m["tpot_s"] is None or m["tpot_s"] <= limits.tpot_s)]
    span = elapsed_s if elapsed_s > 0 else float("nan")
    latencies = {}
    for name in LATENCIES + ("submission_delay_s",):
        values = [m[name] for m in rows.values() if m[name] is not None]
        latencies[name] = {label: percentile(values, fraction) for label, fraction in QUANTILES}
        latencies[name]["mean"] = statistics.mean(values) if values else None
    return {
        "elapsed_s": elapsed_s,
        "requests": len(rows),
        "completed": len(done),
        "output_tokens": sum(m["output_tokens"] for m in done),
        "request_throughput_rps": len(done) / span,
        "completed_output_tokens_per_s": sum(m["output_tokens"] for m in done) / span,
        "goodput_rps": len(good) / span,
        "latencies": latencies,
        "per_request": rows,
    }


def run_workload(engine, workload: list[BenchRequest], eos_token_id: int = -1,
                 temperature: float = 0.0, seed: int = 0,
                 limits: "LatencyLimits | None" = None, clock=time.perf_counter,
                 sleep=time.sleep) -> dict:
    """Submit every request when it is due, step the engine until all are finished, and note when
    the host saw each output token.  Returns ``summarize``'s figures."""
    due = sorted(workload, key=lambda r: r.arrival_s)
    if len({r.request_id for r in due}) != len(due):
        raise ValueError("request ids must be distinct")
    timings: dict[str, _Timing] = {}
    seen: dict[str, int] = {}
    start = clock()
    at = 0
    while at < len(due) or engine.has_pending():
        now = clock() - start
        while at < len(due) and due[at].arrival_s <= now:
            request = due[at]
            engine.submit(request.request_id, list(request.prompt_token_ids),
                          request.max_new_tokens, eos_token_id, temperature, seed + at)
            timings[request.request_id] = _Timing(request.arrival_s, clock() - start)
            seen[request.request_id] = 0
            at += 1
        if not engine.has_pending():
            sleep(max(0.0, min(due[at].arrival_s - (clock() - start), 0.01)))
            continue
        finished = engine.step()
        now = clock() - start
        counts = {rid: request.num_generated_tokens for rid, request in engine.requests.items()}
        for record in finished:
            counts[record["request_id"]] = len(record["generated_token_ids"])
        for rid, count in counts.items():
            timing = timings.get(rid)
            if timing is None:
                continue                          # a request of someone else's on this engine
            timing.token_s.extend([now] * (count - seen[rid]))
            seen[rid] = count
        for record in finished:
            if record["request_id"] in timings:
                timings[record["request_id"]].finished_s = now
    return summarize(timings, clock() - start, limits)


def aggregate(reports: list[dict]) -> dict:
    """Mean and standard deviation over repeated runs, of the rates and of every latency
    quantile (as the reference's ``aggregate_runs``, src/utils/benchmark.py:52-81)."""
    def spread(values):
        values = [v for v in values if v is not None]
        return {"values": values,
                "mean": statistics.mean(values) if values else None,
                "stdev": statistics.stdev(values) if len(values) > 1 else None}

    return {
        "aggregate": {name: spread([r[name] for r in reports]) for name in RATES},
        "latency_across_runs": {
            name: {label: spread([r["latencies"][name][label] for r in reports])
                   for label, _ in QUANTILES}
            for name in LATENCIES},
        "executed_repeats": len(reports),
    }
