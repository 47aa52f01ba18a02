"""The kernels as functions of torch tensors.  Every function launches on the current CUDA stream
and checks shapes, dtypes and strides before it passes pointers on; a size that a kernel does not
take is refused with an error that names it.  Nothing here falls back to the CPU or to library
model code.
"""

from __future__ import annotations

import os

import torch

from . import library
from .library import KernelsUnavailable

F32, BF16 = 0, 1

# how many kernels of this package were launched (bench.py reports it)
launch_count = 0


def _tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Every launch asks for it, so it takes the short way
    (a step of a few hundred launches spent more time in ``torch.cuda.current_stream()`` than in
    anything else on the host); it follows stream switches such as a graph capture."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: "torch.Tensor | None") -> int | None:
    return None if t is None else t.data_ptr()


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code == 0:
        return
    if code < 0:
        raise ValueError(f"{what}: the kernel refuses these sizes (code {code})")
    raise RuntimeError(f"{what}: CUDA error {code} at launch")


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise ValueError(message)


def require_device(device: "torch.device | str") -> torch.device:
    """The CUDA device to run on; raises if there is none."""
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelsUnavailable(f"distengine_b200 runs on a CUDA device only, got '{device}'")
    if not torch.cuda.is_available():
        raise KernelsUnavailable("distengine_b200 needs a CUDA device (sm_100a) and none is "
                                 "visible; there is no CPU path")
    return device


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous() and t.is_cuda,
          f"{name} must be a contiguous int32 CUDA tensor")


# ------------------------------------------------------------------------------- embedding
def embed_rows(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[n] = float32(table[ids[n]]); ids int32 [N], table [V, H], out float32 [N, H]."""
    _i32(ids, "ids")
    n, (vocab, width) = ids.shape[0], table.shape
    _need(table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32
          and tuple(out.shape) == (n, width), "embed_rows: out must be float32 [N, H]")
    lib = library.load("core")
    _check(lib.de_embed_rows(_tag(table.dtype), ids.data_ptr(), table.data_ptr(), out.data_ptr(),
                             n, width, vocab, _stream()), "embed_rows")


# ------------------------------------------------------------------------------- norm
def add_rmsnorm(resid: torch.Tensor, delta: "torch.Tensor | None", weight: torch.Tensor,
                eps: float, out: torch.Tensor, rows: "torch.Tensor | None" = None) -> None:
    """out = rmsnorm(resid + delta) * weight; resid (float32) takes the sum unless ``rows`` picks
    the rows to normalise (then out[i] comes from row rows[i] and resid is not written)."""
    width = resid.shape[1]
    n_out = resid.shape[0] if rows is None else rows.shape[0]
    _need(resid.dtype == torch.float32 and resid.is_contiguous(), "resid must be float32")
    _need(out.is_contiguous() and tuple(out.shape) == (n_out, width), "add_rmsnorm: out shape")
    _need(weight.is_contiguous() and weight.shape == (width,), "add_rmsnorm: weight shape")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous()
              and delta.shape == resid.shape, "add_rmsnorm: delta must match resid's shape and "
              "the output's dtype")
    if rows is not None:
        _i32(rows, "rows")
    lib = library.load("core")
    _check(lib.de_add_rmsnorm(_tag(out.dtype), _tag(weight.dtype), resid.data_ptr(), _ptr(delta),
                              weight.data_ptr(), out.data_ptr(), _ptr(rows), n_out, width,
                              float(eps), _stream()), "add_rmsnorm")


# ------------------------------------------------------------------------------- rotation + cache write
def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_slot: torch.Tensor,
                  inv_freq: "torch.Tensor | None", rotary_dim: int, heads: int, kv_heads: int,
                  head_dim: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                  block_table: torch.Tensor, write_kv: bool, status: torch.Tensor) -> None:
    """Rotate q and k of qkv [N, (heads + 2 kv_heads) * d] in place by position and store k, v in
    the pages [pages, kv_heads, page, d] through block_table [slots, max_pages]."""
    n = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (heads + 2 * kv_heads) * head_dim,
          "rope_kv_write: qkv must be [N, (heads + 2 kv_heads) * head_dim]")
    _i32(positions, "positions"), _i32(token_slot, "token_slot"), _i32(block_table, "block_table")
    _i32(status, "status")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape == v_pages.shape
          and k_pages.dtype == qkv.dtype == v_pages.dtype and k_pages.dim() == 4
          and k_pages.shape[1] == kv_heads and k_pages.shape[3] == head_dim,
          "rope_kv_write: pages must be [pages, kv_heads, page, head_dim] of qkv's dtype")
    _need(rotary_dim % 2 == 0 and 0 <= rotary_dim <= head_dim,
          f"rope_kv_write: rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
              and inv_freq.shape == (rotary_dim // 2,), "rope_kv_write: inv_freq shape")
    lib = library.load("core")
    _check(lib.de_rope_kv_write(_tag(qkv.dtype), qkv.data_ptr(), qkv.stride(0),
                                positions.data_ptr(), token_slot.data_ptr(), _ptr(inv_freq),
                                rotary_dim, heads, kv_heads, head_dim, k_pages.data_ptr(),
                                v_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0),
                                k_pages.shape[2], int(write_kv), k_pages.shape[0], n,
                                status.data_ptr(), _stream()), "rope_kv_write")


# ------------------------------------------------------------------------------- feed-forward
def silu_mul(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, i] = silu(x[n, i]) * x[n, inner + i]; x [N, 2 inner], out [N, inner]."""
    n, inner = out.shape
    _need(x.is_contiguous() and out.is_contiguous() and x.shape == (n, 2 * inner)
          and x.dtype == out.dtype, "silu_mul: x must be [N, 2 inner] and out [N, inner]")
    lib = library.load("core")
    _check(lib.de_silu_mul(_tag(x.dtype), x.data_ptr(), out.data_ptr(), n, inner, _stream()),
           "silu_mul")


# ------------------------------------------------------------------------------- matrix products
def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, m] = sum_k x[n, k] w[m, k] in IEEE float32 on the CUDA cores."""
    _need(x.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32 takes float32 tensors")
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1]
          and tuple(out.shape) == (x.shape[0], w.shape[0]), "gemm_f32: shapes do not agree")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1,
          "gemm_f32: rows must be contiguous")
    lib = library.load("gemm_f32")
    _check(lib.de_gemm_f32(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.shape[0], w.shape[0],
                           x.shape[1], x.stride(0), w.stride(0), out.stride(0), _stream()),
           "gemm_f32")


# Up to this many tokens a product streams the weights through linear_small (the kernel takes up
# to 32; measured on B200 in decode steps, the library product is faster from 17 rows on: batch
# 24: 1.17 against 1.42 ms a step, batch 32: 1.21 against 1.56; at 12 rows linear_small wins).
SMALL_ROWS = int(os.environ.get("DISTENGINE_B200_SMALL_ROWS", "16"))


def _small_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (0 < x.shape[0] <= SMALL_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and w.is_contiguous() and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


# The RMS norm between two weight-streaming products can ride on them (``csrc/linear_small.cu``):
# the product before it adds to the residual and leaves residual * norm weight plus shares of the
# rows' sums of squares, the product after it applies the rows' factors to its sums.
# DISTENGINE_B200_NORM_RIDE=0 keeps the norm a kernel of its own (for measurements).
NORM_RIDE = os.environ.get("DISTENGINE_B200_NORM_RIDE", "1") != "0"
NORM_RIDE_ROWS = 16


# From SMALL_ROWS + 1 to this many tokens a product goes to the swapped-operand tcgen05 kernel
# (``csrc/linear_mid.cu``, which takes up to 128); DISTENGINE_B200_MID_ROWS=0 gives those to the
# library product.  Measured on B200 in decode steps (TinyLlama shape, a step in ms, this kernel
# against the library product with separate norm and activation kernels): batch 20 1.12 / 1.16,
# batch 32 1.18 / 1.20, batch 48 1.36 / 1.28, batch 64 1.42 / 1.33.
MID_ROWS = int(os.environ.get("DISTENGINE_B200_MID_ROWS", "32"))


def _mid_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (SMALL_ROWS < x.shape[0] <= MID_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and w.is_contiguous() and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def _linear_mid(x, w, out, gated, before, after, status) -> None:
    global _tcgen05_status
    n_out = w.shape[0] // 2 if gated else w.shape[0]
    _need(out.dtype in (torch.bfloat16, torch.float32) and out.stride(1) == 1
          and tuple(out.shape) == (x.shape[0], n_out), "linear_mid: out [tokens, n]")
    if status is None:
        if _tcgen05_status is None or _tcgen05_status.device != x.device:
            _tcgen05_status = torch.zeros(1, dtype=torch.int32, device=x.device)
        status = _tcgen05_status
    in_parts = in_count = width = 0
    eps = 0.0
    if before is not None:
        parts = before.parts
        _need(parts.dtype == torch.float32 and parts.is_contiguous()
              and parts.shape[0] == x.shape[0], "linear: before.parts must be float32 [rows, count]")
        in_parts, in_count, width, eps = parts.data_ptr(), parts.shape[1], before.width, before.eps
    resid = ld_resid = weight = out_parts = 0
    lib = library.load("linear_mid")
    if after is not None:
        _need(after.resid.dtype == torch.float32 and after.resid.stride(1) == 1
              and tuple(after.resid.shape) == tuple(out.shape) and out.dtype == torch.bfloat16
              and after.weight.dtype == torch.bfloat16 and after.weight.is_contiguous()
              and after.weight.shape == (n_out,) and after.parts.dtype == torch.float32
              and after.parts.is_contiguous()
              and tuple(after.parts.shape) == (x.shape[0], lib.de_linear_mid_parts(n_out)),
              "linear: after needs resid float32 [rows, n], weight bfloat16 [n] and parts "
              "float32 [rows, norm_ride_parts(...)]")
        resid, ld_resid = after.resid.data_ptr(), after.resid.stride(0)
        weight, out_parts = after.weight.data_ptr(), after.parts.data_ptr()
    _check(lib.de_linear_mid(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                             out.stride(0), x.shape[0], n_out, x.shape[1],
                             int(out.dtype == torch.float32), int(gated), in_parts, in_count,
                             int(width), float(eps), resid, ld_resid, weight, out_parts, 0,
                             status.data_ptr(), _stream()), "linear_mid")


def norm_ride_parts(rows: int, w: torch.Tensor, dtype: torch.dtype) -> int:
    """How many shares of every row's sum of squares a product of ``rows`` rows against ``w``
    leaves when it does the following norm's work (``linear(..., after=)``), or 0 if such a
    product does not go to the weight-streaming kernel.  The same condition says whether a product
    against ``w`` can apply a preceding norm's row factors (``linear(..., before=)``)."""
    if not (NORM_RIDE and dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and w.is_contiguous() and w.data_ptr() % 16 == 0):
        return 0
    if 0 < rows <= min(SMALL_ROWS, NORM_RIDE_ROWS):
        return int(library.load("linear_small").de_linear_small_parts(w.shape[0]))
    if SMALL_ROWS < rows <= MID_ROWS:
        return int(library.load("linear_mid").de_linear_mid_parts(w.shape[0]))
    return 0


def _linear_small_norm(x, w, out, gated, before, after, status=None) -> None:
    if _mid_ok(x, w):
        _linear_mid(x, w, out, gated, before, after, status)
        return
    n_out = w.shape[0] // 2 if gated else w.shape[0]
    _need(_small_ok(x, w) and x.shape[0] <= NORM_RIDE_ROWS and out.dtype == torch.bfloat16
          and out.stride(1) == 1, "linear: a product that carries a norm must be one the "
          "weight-streaming kernel takes (see norm_ride_parts)")
    in_parts = in_count = width = 0
    eps = 0.0
    if before is not None:
        parts = before.parts
        _need(parts.dtype == torch.float32 and parts.is_contiguous()
              and parts.shape[0] == x.shape[0], "linear: before.parts must be float32 [rows, count]")
        in_parts, in_count, width, eps = parts.data_ptr(), parts.shape[1], before.width, before.eps
    resid = ld_resid = weight = out_parts = 0
    if after is not None:
        lib_parts = norm_ride_parts(x.shape[0], w, x.dtype)
        _need(after.resid.dtype == torch.float32 and after.resid.stride(1) == 1
              and tuple(after.resid.shape) == tuple(out.shape)
              and after.weight.dtype == torch.bfloat16 and after.weight.is_contiguous()
              and after.weight.shape == (n_out,) and after.parts.dtype == torch.float32
              and after.parts.is_contiguous()
              and tuple(after.parts.shape) == (x.shape[0], lib_parts),
              "linear: after needs resid float32 [rows, n], weight bfloat16 [n] and parts "
              "float32 [rows, norm_ride_parts(...)]")
        resid, ld_resid = after.resid.data_ptr(), after.resid.stride(0)
        weight, out_parts = after.weight.data_ptr(), after.parts.data_ptr()
    lib = library.load("linear_small")
    _check(lib.de_linear_small_norm(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                                    out.data_ptr(), out.stride(0), x.shape[0], n_out, x.shape[1],
                                    int(gated), in_parts, in_count, int(width), float(eps), resid,
                                    ld_resid, weight, out_parts, _stream()),
           "linear_small (with norm)")


TCGEN05_ROWS = 1024     # from this many rows on, products go to this package's tcgen05 kernel
_tile_fits: dict[tuple[int, int], bool] = {}


def _tcgen05_fits(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether a plain product of this shape goes to this package's tcgen05 kernel: many rows, and
    a shape whose tiles fill the SMs in whole rounds with wide tiles.  (Measured on B200 against
    cuBLAS at 2,048 rows: equal or within 4% where this holds, up to a third slower where the
    tiles have to be narrow or the last round is nearly empty; with few rows cuBLAS splits k,
    which this kernel does not.)"""
    m, n = x.shape[0], w.shape[0]
    if (m < TCGEN05_ROWS or x.shape[1] % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.stride(1) != 1
            or w.stride(1) != 1 or x.data_ptr() % 16 or w.data_ptr() % 16):
        return False
    key = (m, n)
    fits = _tile_fits.get(key)
    if fits is None:
        lib = library.load("gemm_tcgen05")
        bn, sms = lib.de_gemm_tcgen05_tile(m, n, 0), lib.de_gemm_tcgen05_sms()
        tiles = -(-m // 128) * -(-n // bn)
        rounds = -(-tiles // sms)
        fits = _tile_fits[key] = bn >= 192 and m * n >= 0.75 * rounds * sms * 128 * bn
    return fits


def linear(x: torch.Tensor, w: torch.Tensor, out: "torch.Tensor | None" = None,
           out_dtype: "torch.dtype | None" = None,
           status: "torch.Tensor | None" = None, before=None, after=None) -> torch.Tensor:
    """x @ w^T, float32 accumulation.

    ``before`` (``.parts`` float32 [rows, count], ``.width``, ``.eps``): x is the output of an RMS
    norm but for the rows' factors rsqrt(sum of the row's parts / width + eps), which the product
    applies to its sums.  ``after`` (``.resid`` float32 [rows, n], ``.weight`` bfloat16 [n],
    ``.parts`` float32 [rows, norm_ride_parts(...)]): the result is added to ``resid`` and ``out``
    becomes resid * weight, ``parts`` the shares of the rows' sums of squares - what ``before``
    of the next product needs.  Both only where ``norm_ride_parts`` is not 0.

    float32: this package's own CUDA-core kernel (true 32-bit).  bfloat16 with up to 16 rows
    (decode steps): this package's weight-streaming kernel (``csrc/linear_small.cu``).  bfloat16
    with a thousand rows or more in a shape that suits it: this package's tcgen05 kernel
    (``csrc/gemm_tcgen05.cu``).  Otherwise the library matrix product (cuBLAS through torch),
    where the reference calls a library too (src/layers/linear.py:19-20).  The output is bfloat16
    or float32.  ``status`` (int32 [1]): where the tcgen05 kernel records a wait that ran out."""
    out_dtype = out_dtype or (out.dtype if out is not None else x.dtype)
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    if x.shape[0] == 0:
        return out
    if x.dtype == torch.float32:
        _need(out.dtype == torch.float32, "linear: a float32 product has a float32 output")
        _need(before is None and after is None, "linear: float32 products carry no norm")
        gemm_f32(x, w, out)
        return out
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16,
          "linear: operands must both be bfloat16 or both float32")
    _need(x.shape[1] == w.shape[1] and tuple(out.shape) == (x.shape[0], w.shape[0])
          and out.stride(1) == 1, "linear: shapes do not agree")
    if before is not None or after is not None:
        _linear_small_norm(x, w, out, False, before, after, status)
    elif _mid_ok(x, w):
        _linear_mid(x, w, out, False, None, None, status)
    elif _small_ok(x, w):
        lib = library.load("linear_small")
        _check(lib.de_linear_small(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                                   out.data_ptr(), out.stride(0), x.shape[0], w.shape[0],
                                   x.shape[1], int(out.dtype == torch.float32), 0, _stream()),
               "linear_small")
    elif _tcgen05_fits(x, w, out):
        gemm_tcgen05(x, w, out, status=status)
    elif out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    return out


def gated_needs_scratch(x: torch.Tensor, w_gate_up: torch.Tensor) -> bool:
    """Whether ``linear_gated`` forms the [gate | up] product in memory for these operands: not
    for bfloat16 with up to 16 rows (weight-streaming kernel) or with a thousand rows or more
    (tcgen05 kernel; with fewer rows its tiles leave most SMs idle and the library product plus
    the activation kernel is faster)."""
    if x.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16:
        return True
    if _small_ok(x, w_gate_up) or _mid_ok(x, w_gate_up):
        return False
    return not (x.shape[0] >= TCGEN05_ROWS and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
                and w_gate_up.stride(0) % 8 == 0 and x.stride(1) == 1
                and w_gate_up.stride(1) == 1 and x.data_ptr() % 16 == 0
                and w_gate_up.data_ptr() % 16 == 0)


def linear_gated(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor,
                 scratch: "torch.Tensor | None" = None,
                 status: "torch.Tensor | None" = None, before=None) -> torch.Tensor:
    """out[n, i] = silu(x . gate_i) * (x . up_i) for w_gate_up = [gate rows; up rows] of shape
    [2 inner, k].  bfloat16: one kernel whose epilogue applies the activation, the
    weight-streaming one up to 16 rows, the tcgen05 one from 1,024 rows.  float32 (or operands that are not
    16-byte aligned): the product into ``scratch`` [N, 2 inner], then ``silu_mul``."""
    inner = w_gate_up.shape[0] // 2
    _need(tuple(out.shape) == (x.shape[0], inner), "linear_gated: out must be [N, inner]")
    if x.shape[0] == 0:
        return out
    if before is not None:          # x lacks its norm's row factors (see ``linear``)
        _linear_small_norm(x, w_gate_up, out, True, before, None, status)
        return out
    if (x.dtype == torch.bfloat16 and _mid_ok(x, w_gate_up) and out.stride(1) == 1
            and out.dtype == torch.bfloat16):
        _linear_mid(x, w_gate_up, out, True, None, None, status)
        return out
    if x.dtype == torch.bfloat16 and _small_ok(x, w_gate_up) and out.stride(1) == 1:
        lib = library.load("linear_small")
        _check(lib.de_linear_small(x.data_ptr(), x.stride(0), w_gate_up.data_ptr(),
                                   w_gate_up.stride(0), out.data_ptr(), out.stride(0), x.shape[0],
                                   inner, x.shape[1], 0, 1, _stream()), "linear_small (gated)")
        return out
    if not gated_needs_scratch(x, w_gate_up) and out.stride(1) == 1 and out.dtype == x.dtype:
        return gemm_tcgen05(x, w_gate_up, out, gated=True, status=status)
    if scratch is None:
        scratch = torch.empty((x.shape[0], 2 * inner), dtype=x.dtype, device=x.device)
    linear(x, w_gate_up, out=scratch)
    silu_mul(scratch, out)
    return out


_tcgen05_status: "torch.Tensor | None" = None


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False,
                 status: "torch.Tensor | None" = None) -> torch.Tensor:
    """out = x @ w^T on the 5th-generation tensor cores (``csrc/gemm_tcgen05.cu``: TMA loads,
    tcgen05.mma with the accumulator in tensor memory), bfloat16 operands, bfloat16 or float32
    output.  ``gated``: w = [gate rows; up rows] ([2 n, k]) and out [m, n] = silu(gate) * up.
    ``status`` (int32 [1]) receives 3 if a wait inside the kernel ran out."""
    global _tcgen05_status
    n = w.shape[0] // 2 if gated else w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2
          and w.dim() == 2 and x.shape[1] == w.shape[1] and tuple(out.shape) == (x.shape[0], n)
          and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1,
          "gemm_tcgen05: x [m, k] and w [n, k] bfloat16 with contiguous rows, out [m, n]")
    _need(out.dtype in (torch.bfloat16, torch.float32), "gemm_tcgen05: out bfloat16 or float32")
    if status is None:
        if _tcgen05_status is None or _tcgen05_status.device != x.device:
            _tcgen05_status = torch.zeros(1, dtype=torch.int32, device=x.device)
        status = _tcgen05_status
    lib = library.load("gemm_tcgen05")
    _check(lib.de_gemm_tcgen05(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                               out.data_ptr(), out.stride(0), x.shape[0], n, x.shape[1],
                               int(out.dtype == torch.float32), int(gated), status.data_ptr(),
                               _stream()), "gemm_tcgen05")
    return out


# ------------------------------------------------------------------------------- sampling
def sample_rows(logits: torch.Tensor, out: torch.Tensor,
                temperature: "torch.Tensor | None" = None, seed: "torch.Tensor | None" = None,
                position: "torch.Tensor | None" = None) -> None:
    """out[r] = arg-max of row r (temperature null or 0) or a seeded draw from
    softmax(logits / temperature)."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be float32")
    _i32(out, "out")
    if temperature is not None:
        _need(temperature.dtype == torch.float32 and seed is not None and position is not None
              and seed.dtype == torch.int64 and position.dtype == torch.int32
              and temperature.shape[0] == seed.shape[0] == position.shape[0] == rows,
              "sample_rows: temperature float32, seed int64, position int32, one per row")
    lib = library.load("core")
    _check(lib.de_sample_rows(logits.data_ptr(), rows, vocab, _ptr(temperature), _ptr(seed),
                              _ptr(position), out.data_ptr(), _stream()), "sample_rows")
