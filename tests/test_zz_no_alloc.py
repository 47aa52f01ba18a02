"""The attention entry point that allocates nothing (csrc/attention_static_scratch.h), called
through its exported C symbol, against the ordinary entry points.

Some callers of this library cannot allocate device memory: the GPU's memory was handed to pools
of their own at start-up, or they run inside another runtime that forbids cudaMalloc, or an
allocation's possible device synchronisation does not fit their loop.  For them the split-key
attention keeps its scratch for partial results in an array inside the library.  This test runs
the same work through both ways, twice in a row with different queries (the second call finds the
first call's partial results in the array and must not be affected by them), and checks the
refusal of a request that does not fit the array.

This file sorts last on purpose: a run that stops at the first failure has then run every other
test before it.
"""

import ctypes

import numpy as np
import pytest
import torch

import plain_llama as plain
from gpu_helpers import PagedFixture, assert_close, run_paged_attention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20


def _symbol():
    from distengine_b200.kernels import library
    lib = library.load("attention_simt")
    fn = lib.de_attn_simt_static_scratch
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [I, P, I, P, I, P, P, P, I, I, P, P, P, P, P, I, P, I, I, I, I, I, I, F, I, P]
    fn.restype = I
    lib.de_attn_static_scratch_error.argtypes = []
    lib.de_attn_static_scratch_error.restype = ctypes.c_char_p
    return fn, lib.de_attn_static_scratch_error


def _call(fn, fx, q_list, heads, kv_heads, d, scale, window, chunk, num_partials_override=None,
          check_free_memory=False):
    from distengine_b200.kernels.attention_plan import build_plan
    dtype = fx.dtype
    qlen = np.array([q.shape[0] for q in q_list], dtype=np.int32)
    pos0 = np.array([n - ql for n, ql in zip(fx.kv_lens, qlen)], dtype=np.int32)
    qstart = (np.cumsum(qlen) - qlen).astype(np.int32)
    plan = build_plan(qlen, pos0, heads // kv_heads, kv_heads, 8, window or 0, chunk,
                      sm_count=torch.cuda.get_device_properties(0).multi_processor_count)
    assert plan.num_partials > 0
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    q = torch.cat([x.reshape(x.shape[0], heads * d) for x in q_list]).to(DEV, dtype).contiguous()
    out = torch.full((q.shape[0], heads * d), float("nan"), dtype=dtype, device=DEV)
    k_pages, v_pages, table = fx.to_device()
    arrays = [t(np.array(fx.slots)), t(qstart), t(qlen), t(pos0), t(plan.items), t(plan.combine)]
    torch.cuda.synchronize()
    # what the driver reports as free on the device: a cudaMalloc inside the library would show
    # here (torch's own counters would not see it).  The first call on a device may make the
    # context load the kernels' code, so the comparison is made on later calls.
    before = torch.cuda.mem_get_info()[0]
    code = fn(0 if dtype == torch.float32 else 1, q.data_ptr(), q.stride(0), out.data_ptr(),
              out.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), table.data_ptr(),
              table.stride(0), k_pages.shape[0], arrays[0].data_ptr(), arrays[1].data_ptr(),
              arrays[2].data_ptr(), arrays[3].data_ptr(), arrays[4].data_ptr(),
              plan.items.shape[0], arrays[5].data_ptr(), plan.combine.shape[0],
              plan.num_partials if num_partials_override is None else num_partials_override,
              heads, kv_heads, d, fx.page, float(scale), int(window or 0),
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    if check_free_memory:
        assert torch.cuda.mem_get_info()[0] == before     # no device memory was taken
    return code, out.float().cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_the_ordinary_entry_points_twice(dtype):
    fn, _ = _symbol()
    heads, kv_heads, d, page = 6, 2, 48, 16
    fx = PagedFixture([300, 77, 130], kv_heads, d, page, dtype, DEV, seed=3)
    g = torch.Generator().manual_seed(9)
    for call in range(2):
        # the second call: other queries, another window, other chunks, over the first call's leftovers
        window = None if call == 0 else 90
        chunk = 64 if call == 0 else 128
        q_list = [torch.randn(ql, heads, d, generator=g).to(dtype).float() for ql in (1, 1, 5)]
        code, got = _call(fn, fx, q_list, heads, kv_heads, d, d ** -0.5, window, chunk,
                          check_free_memory=call == 1)
        assert code == 0
        # the existing entry points, with scratch from the allocator (the float32 kernel for both
        # dtypes: a head size of 48 is forced onto it by asking for its tile shape)
        from distengine_b200.kernels.attention import AttentionLauncher
        launcher_is_simt = not AttentionLauncher(dtype, heads, kv_heads, d, 1.0, window).tensor_cores
        if launcher_is_simt:
            want, partials = run_paged_attention(fx, q_list, heads, kv_heads, d, d ** -0.5, window,
                                                 chunk=chunk)
            assert sum(partials.values()) > 0
            assert torch.equal(got, want)                    # the same kernels: bit for bit
        outs = []
        for i, q in enumerate(q_list):
            n, ql = fx.kv_lens[i], q.shape[0]
            outs.append(plain.plain_attention(q, fx.k[i], fx.v[i], torch.arange(n - ql, n), window,
                                              dtype, d ** -0.5).reshape(ql, heads * d))
        assert_close(got, torch.cat(outs), dtype, f"static scratch, call {call}")


def test_static_scratch_refuses_what_does_not_fit():
    fn, error = _symbol()
    heads, kv_heads, d = 4, 2, 64
    fx = PagedFixture([200], kv_heads, d, 16, torch.float32, DEV, seed=1)
    q = [torch.randn(1, heads, d)]
    too_many = SCRATCH_FLOATS // (kv_heads * 8 * (d + 2)) + 1
    code, out = _call(fn, fx, q, heads, kv_heads, d, d ** -0.5, None, 64,
                      num_partials_override=too_many)
    assert code == -10
    assert torch.isnan(out).all()                            # nothing was launched
    text = error().decode()
    assert "floats" in text and str(SCRATCH_FLOATS) in text
    # a request that fits clears the message
    code, _ = _call(fn, fx, q, heads, kv_heads, d, d ** -0.5, None, 64)
    assert code == 0 and error().decode() == ""


def test_static_scratch_skips_items_beyond_the_slots_it_was_told():
    """The size check is made with ``num_partials``; a work item that names a slot at or beyond it
    must not write there (that could lie past the end of the array).  Told one slot fewer than the
    plan uses, the call leaves the rows of the tile that owns the last slot as they were and
    computes every other row as before."""
    fn, _ = _symbol()
    heads, kv_heads, d = 4, 2, 32
    dtype = torch.float32
    fx = PagedFixture([200, 150], kv_heads, d, 16, dtype, DEV, seed=5)
    g = torch.Generator().manual_seed(2)
    q_list = [torch.randn(1, heads, d, generator=g) for _ in range(2)]
    code, whole = _call(fn, fx, q_list, heads, kv_heads, d, d ** -0.5, None, 64)
    assert code == 0 and torch.isfinite(whole).all()
    from distengine_b200.kernels.attention_plan import build_plan
    plan = build_plan(np.array([1, 1], dtype=np.int32), np.array([199, 149], dtype=np.int32),
                      heads // kv_heads, kv_heads, 8, 0, 64)
    code, short = _call(fn, fx, q_list, heads, kv_heads, d, d ** -0.5, None, 64,
                        num_partials_override=plan.num_partials - 1)
    assert code == 0
    assert torch.equal(short[0], whole[0])                   # the first sequence's slots all fit
    assert torch.isnan(short[1]).all()                       # the tile of the last slot: untouched
