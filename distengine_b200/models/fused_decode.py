"""The whole decode step as one persistent kernel (``csrc/decode_fused.cu``), for models whose
layers all have the shape that kernel implements: pre-norm block, RMS norm, paged grouped-query
attention with full rotary position encoding and no window, gated feed-forward, bfloat16, identity
run plan, one cache group.  ``FusedDecoder.try_build`` checks the built model part by part and
returns None when anything differs; the step function then runs the parts one by one as always.
It is an optimisation of the step function, not a second model: weights, cache pages, block
tables and the step's arrays are the same objects.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from ..kernels import library, ops
from ..parts.attention import PagedAttention
from ..parts.block import PreNormBlock
from ..parts.mlp import GatedMLP
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryPositionEncoding


class _LayerPtrs(ctypes.Structure):
    _fields_ = [(name, c_void_p) for name in ("w_qkv", "w_o", "w_gate_up", "w_down", "norm1",
                                               "norm2", "k_pages", "v_pages")]


class _Args(ctypes.Structure):
    _fields_ = [
        ("layers", c_void_p), ("num_layers", c_int), ("embedding", c_void_p),
        ("final_norm", c_void_p), ("lm_head", c_void_p), ("norm_f32", c_int), ("width", c_int),
        ("heads", c_int), ("kv_heads", c_int), ("inner", c_int), ("vocab", c_int),
        ("eps", c_float), ("scale", c_float), ("inv_freq", c_void_p), ("block_table", c_void_p),
        ("table_stride", c_int), ("page", c_int), ("num_pages", c_int), ("m", c_int),
        ("token_ids", c_void_p), ("positions", c_void_p), ("slots", c_void_p),
        ("logit_rows", c_void_p), ("num_logit_rows", c_int), ("resid_a", c_void_p),
        ("resid_b", c_void_p), ("ssq_part", c_void_p), ("qkv", c_void_p), ("ctx", c_void_p),
        ("act", c_void_p), ("part_acc", c_void_p), ("part_ml", c_void_p), ("chunks", c_int),
        ("chunk_keys", c_int), ("logits", c_void_p), ("barrier", c_void_p), ("status", c_void_p),
        ("timing", c_void_p), ("timing_slots", c_int),
    ]


class FusedDecoder:
    MAX_TOKENS = 16

    @staticmethod
    def try_build(model, cache) -> "FusedDecoder | None":
        try:
            return FusedDecoder(model, cache)
        except _NotThisShape:
            return None

    def __init__(self, model, cache) -> None:
        need = _need
        need(model.dtype == torch.bfloat16)
        need(len(model.plan) == len(model.blocks))
        need(all(e.layer == i and e.reads_cache_of is None for i, e in enumerate(model.plan)))
        need(len(cache.paged) == 1 and not cache.states)
        first = model.blocks[0]
        need(isinstance(first.mixer, PagedAttention) and isinstance(first.feed_forward, GatedMLP))
        mixer, ffn = first.mixer, first.feed_forward
        need(isinstance(model.final_norm, RMSNorm))
        eps, weight_dtype = model.final_norm.eps, model.final_norm.weight.dtype
        for block in model.blocks:
            need(type(block) is PreNormBlock)
            m, f = block.mixer, block.feed_forward
            need(type(m) is PagedAttention and type(f) is GatedMLP)
            need((m.width, m.heads, m.kv_heads, m.head_dim, m.scale, m.window)
                 == (mixer.width, mixer.heads, mixer.kv_heads, mixer.head_dim, mixer.scale, None))
            need(type(m.position) is RotaryPositionEncoding
                 and m.position.rotary_dim == m.head_dim)
            need(torch.equal(m.position.inv_freq, mixer.position.inv_freq))
            need((f.width, f.inner) == (ffn.width, ffn.inner))
            for norm in (block.mixer_norm, block.feed_forward_norm):
                need(type(norm) is RMSNorm and norm.eps == eps and norm.weight.dtype == weight_dtype)
        width, d = mixer.width, mixer.head_dim
        need(d % 32 == 0 and d <= 256 and width % 8 == 0 and ffn.inner % 8 == 0)
        need(weight_dtype in (torch.bfloat16, torch.float32))
        self.module = ("decode_fused", (f"HEAD_DIM={d}",))
        lib = library.load(*self.module)
        need(lib.de_decode_fused_args_bytes() == ctypes.sizeof(_Args)
             and lib.de_decode_fused_layer_bytes() == ctypes.sizeof(_LayerPtrs))
        self.MAX_TOKENS = lib.de_decode_fused_max_tokens()
        self.grid = lib.de_decode_fused_grid(width)
        need(self.grid >= 1)
        self.lib, self.model, self.cache = lib, model, cache
        self.mixer, self.ffn = mixer, ffn
        dev, mt = model.device, self.MAX_TOKENS
        group = cache.paged[0]
        layers = (_LayerPtrs * len(model.blocks))()
        for i, block in enumerate(model.blocks):
            binding_k, binding_v = group.k[i], group.v[i]
            layers[i] = _LayerPtrs(block.mixer.w_qkv.data_ptr(), block.mixer.w_o.data_ptr(),
                                   block.feed_forward.w_gate_up.data_ptr(),
                                   block.feed_forward.w_down.data_ptr(),
                                   block.mixer_norm.weight.data_ptr(),
                                   block.feed_forward_norm.weight.data_ptr(),
                                   binding_k.data_ptr(), binding_v.data_ptr())
        raw = bytes(layers)
        self.layers_dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        f32, bf16 = torch.float32, torch.bfloat16
        self.resid_a = torch.zeros(mt, width, dtype=f32, device=dev)
        self.resid_b = torch.zeros(mt, width, dtype=f32, device=dev)
        self.ssq = torch.zeros((2 * len(model.blocks) + 1) * self.grid * mt, dtype=f32, device=dev)
        self.qkv = torch.zeros(mt, (mixer.heads + 2 * mixer.kv_heads) * d, dtype=bf16, device=dev)
        self.ctx = torch.zeros(mt, mixer.heads * d, dtype=bf16, device=dev)
        self.act = torch.zeros(mt, ffn.inner, dtype=bf16, device=dev)
        group_heads = mixer.heads // mixer.kv_heads
        self.tiles_rows = (group_heads + 15) // 16
        self.max_units = 4 * self.grid
        slots = self.max_units * self.tiles_rows * 16
        self.part_acc = torch.zeros(slots * d, dtype=f32, device=dev)
        self.part_ml = torch.zeros(slots * 2, dtype=f32, device=dev)
        self.barrier = torch.zeros(1, dtype=torch.int32, device=dev)
        self.args = _Args(
            layers=self.layers_dev.data_ptr(), num_layers=len(model.blocks),
            embedding=model.embedding.data_ptr(), final_norm=model.final_norm.weight.data_ptr(),
            lm_head=model.output.data_ptr(), norm_f32=int(weight_dtype == f32), width=width,
            heads=mixer.heads, kv_heads=mixer.kv_heads, inner=ffn.inner,
            vocab=model.config.vocabulary, eps=eps, scale=mixer.scale,
            inv_freq=mixer.position.inv_freq.data_ptr(),
            block_table=group.device_table.data_ptr(), table_stride=group.device_table.stride(0),
            page=cache.page_size, num_pages=group.pool.num_pages,
            resid_a=self.resid_a.data_ptr(), resid_b=self.resid_b.data_ptr(),
            ssq_part=self.ssq.data_ptr(), qkv=self.qkv.data_ptr(), ctx=self.ctx.data_ptr(),
            act=self.act.data_ptr(), part_acc=self.part_acc.data_ptr(),
            part_ml=self.part_ml.data_ptr(), barrier=self.barrier.data_ptr())

    def takes(self, host) -> bool:
        """A step of single tokens, few enough for the kernel."""
        return host.n_tokens <= self.MAX_TOKENS and int(host.seq_qlen.max()) == 1

    def _chunks(self, host) -> tuple[int, int]:
        """(chunks, keys a chunk): one block reads all keys of a (token, kv head) unit, its 16 warps
        sharing them; the ranges are cut over several blocks only when they are long and the units
        too few to occupy the SMs."""
        units = host.n_tokens * self.mixer.kv_heads
        longest = int(host.seq_pos0.max()) + 1
        if units * 2 >= self.grid or longest <= 2048:
            return 1, max(longest, 64)
        wanted = min(self.grid // units, self.max_units // units, (longest + 63) // 64)
        keys = ((longest + wanted - 1) // wanted + 63) // 64 * 64
        return (longest + keys - 1) // keys, keys

    def run(self, ctx) -> torch.Tensor:
        host = ctx.host
        rows = ctx.logit_rows.shape[0]
        logits = ctx.buffer("model.logits", (rows, self.model.config.vocabulary), torch.float32)
        a = self.args
        a.m, a.num_logit_rows = host.n_tokens, rows
        a.token_ids, a.positions = ctx.token_ids.data_ptr(), ctx.seq_pos0.data_ptr()
        a.slots, a.logit_rows = ctx.seq_slot.data_ptr(), ctx.logit_rows.data_ptr()
        a.chunks, a.chunk_keys = self._chunks(host)
        a.logits, a.status = logits.data_ptr(), ctx.status.data_ptr()
        self.barrier.zero_()
        code = self.lib.de_decode_fused(ctypes.byref(a), self.grid,
                                        torch.cuda.current_stream().cuda_stream)
        ops._check(code, "decode_fused")
        return logits


class _NotThisShape(Exception):
    pass


def _need(condition: bool) -> None:
    if not condition:
        raise _NotThisShape()
