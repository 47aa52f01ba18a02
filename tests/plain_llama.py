"""Plain, slow implementation of the Llama decoder, written from the reference's formulas.

Whole sequences, no cache, one function for each part, float32 math on the CPU.  It shares no
code with the product path (``distengine_b200``): it reads ``config.json`` and the safetensors
file itself (through the ``safetensors`` package; the product has its own reader).

Every function cites the file and line of the reference (paths within the reference project)
whose formula it restates.  ``tests/golden/make_golden.py`` compared this file once with the
reference's own model code on tiny random models; the committed ``tests/golden/*.npz`` hold those
outputs and ``tests/test_plain.py`` re-checks this file against them.

``act_dtype`` selects the rounding model.  ``torch.float32``: no rounding anywhere (the
reference's own mode).  ``torch.bfloat16``: matrices and activations are rounded to bfloat16 at the
places where the engine's bfloat16 path rounds them (every matrix product's output, the norm's
output, the rotated q/k, the cached k/v, silu(gate)*up), while the norm statistics, rotation angles,
softmax and the residual sum stay in 32-bit.
"""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch


# ----------------------------------------------------------------------------- helpers


def _rnd(x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
    """Round to the activation dtype and come back to float32."""
    if act_dtype == torch.float32:
        return x
    return x.to(act_dtype).to(torch.float32)


def load_model_folder(folder: str) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor of model.safetensors as float32."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    return config, {name: t.to(torch.float32) for name, t in tensors.items()}


def rope_theta_of(config: dict) -> float:
    """theta from ``rope_parameters`` (src/models/llama.py:105-110) or the top-level key."""
    params = config.get("rope_parameters")
    if params is not None and "rope_theta" in params:
        return float(params["rope_theta"])
    return float(config["rope_theta"])


def head_dim_of(config: dict) -> int:
    """head_dim = hidden_size // num_attention_heads (src/layers/attention.py:90)."""
    return int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])


# ----------------------------------------------------------------------------- parts


def plain_embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather, no scaling (src/layers/embed_head.py:12-13)."""
    return table[ids.long()]


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float,
                  act_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """mean of squares, rsqrt, cast, then times weight (src/layers/layernorm.py:12-23)."""
    xf = x.to(torch.float32)
    variance = (xf * xf).mean(dim=-1, keepdim=True)
    normalized = xf * torch.rsqrt(variance + eps)
    return _rnd(_rnd(normalized, act_dtype) * weight.to(torch.float32), act_dtype)


def plain_linear(x: torch.Tensor, weight: torch.Tensor,
                 act_dtype: torch.dtype = torch.float32, keep_f32: bool = False) -> torch.Tensor:
    """x @ W^T without bias, W stored [out, in] (src/layers/linear.py:19-20)."""
    w = _rnd(weight.to(torch.float32), act_dtype)
    out = x.to(torch.float64) @ w.to(torch.float64).t()
    out = out.to(torch.float32)
    return out if keep_f32 else _rnd(out, act_dtype)


def plain_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """1 / theta^(2i/d) for i in 0..d/2-1, in float32 (src/layers/rotary_embedding.py:14-15)."""
    indices = torch.arange(0, head_dim, 2, dtype=torch.float32)
    return 1.0 / (theta ** (indices / head_dim))


def plain_rope(x: torch.Tensor, positions: torch.Tensor, theta: float,
               act_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Half-split rotation of x [T, heads, d] (src/layers/rotary_embedding.py:29-54).

    Feature j pairs with feature j + d/2; angles, cos and sin in float32.
    """
    d = x.shape[-1]
    angles = positions.to(torch.float32)[:, None] * plain_inv_freq(d, theta)[None, :]
    cos = angles.cos()[:, None, :]
    sin = angles.sin()[:, None, :]
    first, second = x.to(torch.float32)[..., : d // 2], x.to(torch.float32)[..., d // 2:]
    rotated = torch.cat((first * cos - second * sin, second * cos + first * sin), dim=-1)
    return _rnd(rotated, act_dtype)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    q_positions: torch.Tensor, window: int | None = None,
                    act_dtype: torch.dtype = torch.float32,
                    scale: float | None = None) -> torch.Tensor:
    """Dense grouped-query causal attention (src/layers/attention.py:35-71).

    q [T, nh, d] are the queries of the keys' last T positions or of any positions given in
    ``q_positions``; k, v [S, nkv, d] hold the keys of positions 0..S-1.  Query head h reads KV head
    h // g (repeat_interleave, :35-36); scores are (q k^T) * d^-0.5 (:22,38); a key is masked when
    its position is greater than the query's (:41-58); softmax in float32 (:66-69).  ``window``
    (not in the reference: it has causal masking only) also masks keys at positions
    <= query - window.
    """
    T, nh, d = q.shape
    S, nkv, _ = k.shape
    g = nh // nkv
    scale = d ** -0.5 if scale is None else scale
    kk = k.to(torch.float32).repeat_interleave(g, dim=1)   # [S, nh, d]
    vv = v.to(torch.float32).repeat_interleave(g, dim=1)
    scores = torch.einsum("thd,shd->hts", q.to(torch.float32), kk) * scale
    key_pos = torch.arange(S)
    masked = key_pos[None, :] > q_positions[:, None]
    if window is not None:
        masked = masked | (key_pos[None, :] <= q_positions[:, None] - window)
    scores = scores.masked_fill(masked[None, :, :], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    ctx = torch.einsum("hts,shd->thd", probs, vv)
    return _rnd(ctx, act_dtype)


def plain_swiglu(gate: torch.Tensor, up: torch.Tensor,
                 act_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """silu(gate) * up with silu(z) = z * sigmoid(z) (src/layers/activation.py:6-9)."""
    g = gate.to(torch.float32)
    return _rnd(g * torch.sigmoid(g) * up.to(torch.float32), act_dtype)


def plain_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
              act_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """gate and up products, silu(gate)*up, down product (src/models/llama.py:22-29)."""
    gate = plain_linear(x, w_gate, act_dtype)
    up = plain_linear(x, w_up, act_dtype)
    return plain_linear(plain_swiglu(gate, up, act_dtype), w_down, act_dtype)


def plain_attention_block(x: torch.Tensor, positions: torch.Tensor, w: dict[str, torch.Tensor],
                          prefix: str, nh: int, nkv: int, d: int, theta: float,
                          act_dtype: torch.dtype = torch.float32,
                          window: int | None = None) -> torch.Tensor:
    """q/k/v products, rotation of q and k, attention, output product
    (src/layers/attention.py:111-155)."""
    T = x.shape[0]
    q = plain_linear(x, w[prefix + "q_proj.weight"], act_dtype).view(T, nh, d)
    k = plain_linear(x, w[prefix + "k_proj.weight"], act_dtype).view(T, nkv, d)
    v = plain_linear(x, w[prefix + "v_proj.weight"], act_dtype).view(T, nkv, d)
    q = plain_rope(q, positions, theta, act_dtype)
    k = plain_rope(k, positions, theta, act_dtype)
    ctx = plain_attention(q, k, v, positions, window, act_dtype)
    return plain_linear(ctx.reshape(T, nh * d), w[prefix + "o_proj.weight"], act_dtype)


def plain_decoder_layer(x: torch.Tensor, positions: torch.Tensor, w: dict[str, torch.Tensor],
                        layer: int, config: dict,
                        act_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Pre-norm block with two residual sums (src/models/llama.py:74-89).

    The residual stream ``x`` stays in float32 in both rounding models.
    """
    p = f"model.layers.{layer}."
    eps = float(config["rms_norm_eps"])
    nh = int(config["num_attention_heads"])
    nkv = int(config.get("num_key_value_heads") or nh)
    h = plain_rmsnorm(x, w[p + "input_layernorm.weight"], eps, act_dtype)
    x = x + plain_attention_block(h, positions, w, p + "self_attn.", nh, nkv, head_dim_of(config),
                                  rope_theta_of(config), act_dtype)
    h = plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps, act_dtype)
    x = x + plain_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                      w[p + "mlp.down_proj.weight"], act_dtype)
    return x


def plain_forward(config: dict, w: dict[str, torch.Tensor], token_ids,
                  act_dtype: torch.dtype = torch.float32, rows=None) -> torch.Tensor:
    """Logits [T, V] in float32 of one whole sequence from position 0
    (src/models/llama.py:131-191, 206-217).  ``rows``: only these positions go through the final
    norm and the output matrix (the result is [len(rows), V]); the reference computes all.

    ``tie_word_embeddings`` true and no ``lm_head.weight`` in the file: the embedding table is the
    output matrix (the reference always has a separate ``lm_head.weight``, src/models/llama.py:201).
    """
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    table = _rnd(w["model.embed_tokens.weight"], act_dtype)
    x = plain_embedding(ids, table)
    for layer in range(int(config["num_hidden_layers"])):
        x = plain_decoder_layer(x, positions, w, layer, config, act_dtype)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    x = plain_rmsnorm(x, w["model.norm.weight"], float(config["rms_norm_eps"]), act_dtype)
    head = w.get("lm_head.weight")
    if head is None:
        if not config.get("tie_word_embeddings", False):
            raise KeyError("lm_head.weight")
        head = w["model.embed_tokens.weight"]
    return plain_linear(x, head, act_dtype, keep_f32=True)


# ----------------------------------------------------------------------------- generation


def plain_greedy(logits_row: torch.Tensor) -> int:
    """argmax; the lowest id wins a tie (src/layers/sampler.py:5-8)."""
    return int(torch.argmax(logits_row.to(torch.float32)).item())


def plain_uniform(seed: int, position: int, vocab: int) -> np.ndarray:
    """Counter-based uniforms in (0,1), one for each token id: a 64-bit mix (splitmix64's
    finaliser) of (seed, position, id).  No reference counterpart (the reference samples greedily
    only); the engine's kernel restates the same integer arithmetic."""
    mask = (1 << 64) - 1
    base = (seed * 0x9E3779B97F4A7C15 + position * 0xD1B54A32D192ED03) & mask
    with np.errstate(over="ignore"):
        ids = np.arange(1, vocab + 1, dtype=np.uint64)
        z = np.uint64(base) + ids * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    top = (z >> np.uint64(41)).astype(np.float32)          # 23 bits, + 0.5: exact in float32
    return (top + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def plain_temperature_sample(logits_row: torch.Tensor, temperature: float, seed: int,
                             position: int) -> int:
    """A draw from softmax(logits / temperature) by the Gumbel-max rule:
    argmax_i(logits_i / T - log(-log(u_i))), u_i from ``plain_uniform``.  Temperature 0 is greedy."""
    if temperature == 0.0:
        return plain_greedy(logits_row)
    u = plain_uniform(seed, position, logits_row.shape[0])
    gumbel = -np.log(-np.log(u.astype(np.float32))).astype(np.float32)
    scores = logits_row.to(torch.float32).numpy() / np.float32(temperature) + gumbel
    return int(np.argmax(scores))


def plain_generate(config: dict, w: dict[str, torch.Tensor], prompt: list[int],
                   max_new_tokens: int, eos_token_id: int = -1, temperature: float = 0.0,
                   seed: int = 0, act_dtype: torch.dtype = torch.float32) -> list[int]:
    """Whole-sequence recompute for every new token (src/utils/generation.py:49-91); a request
    ends on eos or at max_new_tokens (src/distengine/request.py:53-63)."""
    tokens = list(prompt)
    generated: list[int] = []
    while len(generated) < max_new_tokens:
        logits = plain_forward(config, w, tokens, act_dtype)
        token = plain_temperature_sample(logits[-1], temperature, seed, len(tokens))
        generated.append(token)
        tokens.append(token)
        if token == eos_token_id:
            break
    return generated


def softmax_probabilities(logits_row: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / T) in float32, what temperature sampling draws from."""
    return torch.softmax(logits_row.to(torch.float32) / temperature, dim=-1)


__all__ = [name for name in dir() if name.startswith("plain_")] + [
    "load_model_folder", "rope_theta_of", "head_dim_of", "softmax_probabilities", "math"]
