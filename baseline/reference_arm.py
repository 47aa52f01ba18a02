"""The reference arm of ``bench.py``: the unmodified reference (``baseline/_ref``, see
``install_reference.py``) on the same shape, batch, prompt length, steps and warm-up as the
engine's own arm.  Nothing of ``distengine_b200`` is imported or called here.

What runs is the reference's own serving path for one GPU: its ``LlamaForCausalLM`` built from a
``transformers.LlamaConfig`` (src/models/llama.py:194-217), its ``BlockManager`` and ``KVStorage``
(src/distengine/block_manager.py, src/distengine/paged_kv_cache.py:4-23), ``ModelRunner.prefill``
for each prompt and ``ModelRunner.decode_batch`` for the timed steps
(src/distengine/model_runner.py:113-173,226-269), in float32 with TF32 off, which is how its
workers run on CUDA (src/distengine/worker.py:427-430).  ``decode_batch`` takes host token ids
and returns host token ids (its ``.tolist()`` at model_runner.py:261), so every timed step
includes the copy in and the read back: the device-timed figure and the end-to-end one are taken
around the same calls, once with CUDA events and once with the host clock.
"""

from __future__ import annotations

import os
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available() -> "str | None":
    """None if the reference can run here, else the reason in one line."""
    if not os.path.isfile(os.path.join(REF, "distengine", "model_runner.py")):
        return ("baseline/_ref does not hold the reference (run baseline/install_reference.py "
                "where the reference's tree is mounted)")
    try:
        import transformers  # noqa: F401
    except ImportError as error:
        return f"the reference needs the 'transformers' package for its LlamaConfig: {error}"
    return None


def run(model: dict, batch: int, prompt_len: int, steps: int, warmup: int, prefill_len: int,
        points: "tuple[int, ...]" = (1, 16, 64), page: int = 16, seed: int = 0) -> dict:
    sys.path.insert(0, REF)
    import torch
    from transformers import LlamaConfig

    from distengine.block_manager import BlockManager
    from distengine.model_runner import ModelRunner
    from distengine.paged_kv_cache import KVStorage
    from distengine.request import Request, RequestStatus
    from models.llama import LlamaForCausalLM

    # the reference's policy on CUDA (src/distengine/worker.py:427-428)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    device = torch.device("cuda:0")
    config = LlamaConfig(
        vocab_size=model["vocab_size"], hidden_size=model["hidden_size"],
        intermediate_size=model["intermediate_size"],
        num_hidden_layers=model["num_hidden_layers"],
        num_attention_heads=model["num_attention_heads"],
        num_key_value_heads=model["num_key_value_heads"], rms_norm_eps=model["rms_norm_eps"],
        max_position_embeddings=model["max_position_embeddings"],
        rope_parameters={"rope_type": "default", "rope_theta": model["rope_theta"]},
        tie_word_embeddings=False)
    torch.manual_seed(seed)
    net = LlamaForCausalLM(config).float()
    with torch.no_grad():
        for name, parameter in net.named_parameters():
            if parameter.dim() == 2:
                parameter.normal_(0.0, 0.02)            # random weights N(0, 0.02), as the other arm
    net = net.to(device).eval()

    head_dim = config.hidden_size // config.num_attention_heads
    most = max(max(points + (batch,)) * (prompt_len + warmup + steps + 2), prefill_len)
    num_blocks = (most + page - 1) // page + 2 * max(points + (batch,))
    manager = BlockManager(num_blocks, page)
    storage = KVStorage(config.num_hidden_layers, config.num_key_value_heads, head_dim,
                        num_blocks, page, device, torch.float32)
    runner = ModelRunner(net, manager, storage)
    generator = torch.Generator().manual_seed(seed)

    def tokens(n: int) -> list[int]:
        return [int(t) for t in torch.randint(0, config.vocab_size, (n,), generator=generator)]

    def request(name: str, n: int, new: int):
        r = Request(name, tokens(n), new, -1)
        r.status = RequestStatus.RUNNING
        return r

    def prefill_once() -> float:
        r = request("prefill", prefill_len, 2)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.prefill(r)
        stop.record()
        torch.cuda.synchronize()
        runner.release(r)
        return start.elapsed_time(stop)

    def decode(b: int, k_steps: int, w_steps: int) -> tuple[float, float]:
        """(ms a step by CUDA events, ms a step by the host clock) over k_steps."""
        live = [request(f"d{b}-{i}", prompt_len, w_steps + k_steps + 2) for i in range(b)]
        for r in live:
            runner.prefill(r)
        for _ in range(w_steps):
            runner.decode_batch(live)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        start.record()
        for _ in range(k_steps):
            runner.decode_batch(live)
        stop.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3 / k_steps
        for r in live:
            runner.release(r)
        return start.elapsed_time(stop) / k_steps, wall

    for _ in range(2):
        prefill_once()
    prefill_ms = statistics.median(prefill_once() for _ in range(3))
    ms, wall_ms = decode(batch, steps, warmup)
    extra = {}
    for b in points:
        b_ms, _ = decode(b, min(steps, 32), warmup)
        extra[f"decode_b{b}"] = round(b / b_ms * 1e3, 1)
    return {"ms_per_step": ms, "wall_ms_per_step": wall_ms, "prefill_ms": prefill_ms,
            "points": extra, "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 8 * batch}
