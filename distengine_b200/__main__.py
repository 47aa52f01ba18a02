"""Command line: ``python -m distengine_b200 <command>``.

``generate`` follows the reference's ``utils.manual_generate`` (src/utils/manual_generate.py:10-58):
``--prompt`` and ``--max-new-tokens`` (default 32, must be positive) keep their names and
meanings, and it prints the generated token ids and, with a tokenizer, the decoded text.  The
reference downloads its model and tokenizer; here ``--model`` names a folder (or ``--random``
names a config.json, for which a random-weights model folder is written into a temporary folder
from ``--weights-seed``), ``--prompt-ids`` gives token ids directly, and ``--prompt`` needs a
``tokenizer.json`` in the model folder.
``--decode-batch-size`` is the reference's benchmark flag (src/utils/benchmark.py:593).
``random-model`` writes a model folder from a configuration and a seed.
``bench`` runs a set of requests with arrival times through the engine and reports what the
reference's benchmark reports of its requests (src/utils/benchmark.py:585-609: ``--repeats``,
``--output``, a folder that must not exist yet and receives ``baseline.json``, and
``--decode-batch-size``); its default request set is the reference's smoke workload
(src/utils/benchmark.py:26-40: six requests with prompts of 1, 8 and 16 tokens, four new tokens
each, Poisson arrivals at 100 requests a second from seed 42).
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def _tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def _with_model_folder(args: argparse.Namespace, run) -> int:
    """``run(args)`` with ``args.model`` naming a model folder: the given one, or a temporary one
    with random weights for ``--random CONFIG``."""
    if args.max_new_tokens <= 0:
        raise SystemExit("--max-new-tokens must be positive")
    if (args.model is None) == (args.random is None):
        raise SystemExit("give either --model DIR or --random CONFIG.json")
    scratch = None
    if args.random is not None:
        import tempfile
        from .weights.random_init import write_random_model
        with open(args.random) as handle:
            config_json = json.load(handle)
        scratch = tempfile.TemporaryDirectory(prefix="distengine_b200-random-")
        args.model = write_random_model(config_json, os.path.join(scratch.name, "model"),
                                        args.weights_seed, dtype=args.dtype)
    try:
        return run(args)
    finally:
        if scratch is not None:
            scratch.cleanup()


def _generate(args: argparse.Namespace) -> int:
    return _with_model_folder(args, _generate_from_folder)


def _bench(args: argparse.Namespace) -> int:
    if args.repeats <= 0 or args.warmup_requests <= 0:
        raise SystemExit("--repeats and --warmup-requests must be positive")
    if os.path.exists(args.output):
        raise SystemExit("Choose a new output directory")
    return _with_model_folder(args, _bench_from_folder)


def _bench_from_folder(args: argparse.Namespace) -> int:
    from .config.engine import EngineConfig
    from .engine import benchmark
    from .engine.engine import Engine

    lengths = [int(t) for t in args.prompt_lengths.replace(",", " ").split()]
    config = EngineConfig(dtype=args.dtype, block_size=args.block_size,
                          num_blocks=args.num_blocks, decode_batch_size=args.decode_batch_size,
                          max_batch_tokens=args.max_batch_tokens, device=args.device)
    engine = Engine(args.model, config)
    workload = benchmark.make_workload(args.num_requests, lengths, args.max_new_tokens,
                                       engine.model.config.vocabulary, args.seed, args.rate_rps)
    # before every measured run, unmeasured: copies of the longest request, as the reference does
    # (src/utils/benchmark.py:311-323); the first of them also compiles and loads the kernels
    longest = max(workload, key=lambda r: len(r.prompt_token_ids))
    runs = []
    for repeat in range(args.repeats):
        benchmark.run_workload(engine, [
            benchmark.BenchRequest(f"warmup-{repeat}-{i}", 0.0, longest.prompt_token_ids,
                                   longest.max_new_tokens) for i in range(args.warmup_requests)])
        named = [benchmark.BenchRequest(f"run{repeat}-{r.request_id}", r.arrival_s,
                                        r.prompt_token_ids, r.max_new_tokens) for r in workload]
        runs.append(benchmark.run_workload(engine, named))
    report = {
        "workload": {"num_requests": args.num_requests, "prompt_lengths": lengths,
                     "warmup_requests": args.warmup_requests,
                     "max_new_tokens": args.max_new_tokens, "rate_rps": args.rate_rps,
                     "seed": args.seed, "arrival_mode": "poisson" if args.rate_rps > 0 else "burst"},
        "engine": {"model": os.path.abspath(args.model), "dtype": args.dtype,
                   "decode_batch_size": args.decode_batch_size,
                   "max_batch_tokens": args.max_batch_tokens, "block_size": args.block_size},
        "runs": runs,
    }
    report.update(benchmark.aggregate(runs))
    os.makedirs(args.output)
    path = os.path.join(args.output, "baseline.json")
    with open(path, "w") as handle:
        json.dump(report, handle, indent=2)
    rates = report["aggregate"]
    print(f"requests/s {rates['request_throughput_rps']['mean']:.2f}  output tokens/s "
          f"{rates['completed_output_tokens_per_s']['mean']:.1f}  "
          f"ttft p50 {report['latency_across_runs']['ttft_s']['p50']['mean'] * 1e3:.2f} ms")
    print(f"Saved {path}")
    return 0


def _generate_from_folder(args: argparse.Namespace) -> int:
    from .config.engine import EngineConfig
    from .engine.engine import Engine

    tokenizer = _tokenizer(args.model)
    prompts: list[list[int]] = []
    for text in args.prompt_ids or []:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    for text in args.prompt or []:
        if tokenizer is None:
            raise SystemExit(f"--prompt needs {os.path.join(args.model, 'tokenizer.json')} and "
                             f"the 'tokenizers' package; give token ids with --prompt-ids instead")
        prompts.append(tokenizer.encode(text).ids)
    if not prompts:
        raise SystemExit("give at least one --prompt-ids or --prompt")

    config = EngineConfig(dtype=args.dtype, block_size=args.block_size,
                          num_blocks=args.num_blocks, decode_batch_size=args.decode_batch_size,
                          max_batch_tokens=args.max_batch_tokens, device=args.device)
    engine = Engine(args.model, config)
    eos = args.eos_token_id
    if eos is None:
        eos = engine.model.config.eos_token_id if getattr(engine.model.config, "eos_token_id",
                                                          None) is not None else -1
    outputs = engine.generate(prompts, args.max_new_tokens, eos, args.temperature, args.seed)
    for generated in outputs:
        print("Generated token IDs:", generated)
        if tokenizer is not None:
            print(tokenizer.decode(generated, skip_special_tokens=True))
    return 0


def _random_model(args: argparse.Namespace) -> int:
    from .weights.random_init import write_random_model
    with open(args.config) as handle:
        config = json.load(handle)
    write_random_model(config, args.out, args.seed, dtype=args.dtype, norm_init=args.norm_init)
    print(f"wrote {args.out}/config.json and {args.out}/model.safetensors")
    return 0


def _replay(args: argparse.Namespace) -> int:
    from .engine.replay import build_runner, replay
    runner = build_runner(args.model, args.dtype, args.max_tokens, args.block_size, args.device)
    replay(runner, sys.stdin, args.out)
    return 0


def main(argv: "list[str] | None" = None) -> int:
    parser = argparse.ArgumentParser(prog="distengine_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    gen = sub.add_parser("generate", help="generate tokens for one or more prompts")
    gen.add_argument("--model", help="folder with config.json, model.safetensors")
    gen.add_argument("--random", metavar="CONFIG", help="a config.json: generate with random "
                     "weights of that shape instead of a model folder")
    gen.add_argument("--weights-seed", type=int, default=0, help="seed of --random's weights")
    gen.add_argument("--prompt", action="append", help="prompt text (needs tokenizer.json)")
    gen.add_argument("--prompt-ids", action="append",
                     help="prompt as token ids, separated by spaces or commas; may repeat")
    gen.add_argument("--max-new-tokens", type=int, default=32)
    gen.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    gen.add_argument("--seed", type=int, default=0, help="sampling seed of the first prompt")
    gen.add_argument("--eos-token-id", type=int, default=None,
                     help="default: the configuration's, else none (-1)")
    gen.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    gen.add_argument("--block-size", type=int, default=16, help="tokens in a page of the cache")
    gen.add_argument("--num-blocks", type=int, default=None, help="pages in the pool")
    gen.add_argument("--decode-batch-size", type=int, default=64,
                     help="most requests live at a time")
    gen.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of a step")
    gen.add_argument("--device", default="cuda:0")
    gen.set_defaults(run=_generate)

    rnd = sub.add_parser("random-model", help="write a model folder with random weights")
    rnd.add_argument("--config", required=True, help="a config.json to take the sizes from")
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    rnd.add_argument("--norm-init", default="ones", choices=["ones", "uniform"])
    rnd.set_defaults(run=_random_model)

    ben = sub.add_parser("bench", help="run a request set through the engine; request "
                                       "throughput, output tokens a second, latencies")
    ben.add_argument("--model", help="folder with config.json, model.safetensors")
    ben.add_argument("--random", metavar="CONFIG", help="a config.json: random weights in a "
                     "temporary model folder")
    ben.add_argument("--weights-seed", type=int, default=0, help="seed of --random's weights")
    ben.add_argument("--repeats", type=int, default=3)
    ben.add_argument("--output", required=True, help="a new folder; receives baseline.json")
    ben.add_argument("--decode-batch-size", type=int, default=64,
                     help="most requests decoded together in one step")
    ben.add_argument("--warmup-requests", type=int, default=4,
                     help="copies of the longest request run before every measured run")
    ben.add_argument("--num-requests", type=int, default=6)
    ben.add_argument("--prompt-lengths", default="1,8,16",
                     help="prompt lengths, taken in turn by the requests")
    ben.add_argument("--max-new-tokens", type=int, default=4)
    ben.add_argument("--rate-rps", type=float, default=100.0,
                     help="Poisson arrivals at this rate; 0: all requests at once")
    ben.add_argument("--seed", type=int, default=42, help="seed of prompts and arrivals")
    ben.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ben.add_argument("--block-size", type=int, default=16, help="tokens in a page of the cache")
    ben.add_argument("--num-blocks", type=int, default=None, help="pages in the pool")
    ben.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of a step")
    ben.add_argument("--device", default="cuda:0")
    ben.set_defaults(run=_bench)

    rep = sub.add_parser("replay", help="trace replay (same as bin/trace_run)")
    rep.add_argument("--model", required=True)
    rep.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    rep.add_argument("--out", required=True)
    rep.add_argument("--max-tokens", type=int, required=True)
    rep.add_argument("--block-size", type=int, default=16)
    rep.add_argument("--device", default="cuda:0")
    rep.set_defaults(run=_replay)

    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
