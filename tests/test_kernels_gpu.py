"""Each kernel alone against its plain reference, at sizes other than the engine's."""

import numpy as np
import pytest
import torch

import plain_llama as plain
from gpu_helpers import PagedFixture, assert_close, run_paged_attention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _ops():
    from distengine_b200.kernels import ops
    return ops


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_rows(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    table = torch.randn(331, 120, generator=g).to(dtype)
    ids = torch.randint(0, 331, (37,), generator=g, dtype=torch.int32)
    out = torch.empty(37, 120, dtype=torch.float32, device=DEV)
    ops.embed_rows(ids.to(DEV), table.to(DEV), out)
    assert torch.equal(out.cpu(), plain.plain_embedding(ids, table.float()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 120, 2048, 4100])
@pytest.mark.parametrize("weight_dtype", DTYPES)
def test_add_rmsnorm(dtype, width, weight_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(width)
    n, eps = 19, 3e-6
    resid = torch.randn(n, width, generator=g) * 3
    delta = torch.randn(n, width, generator=g).to(dtype)
    weight = (torch.rand(width, generator=g) + 0.5).to(weight_dtype)
    want_sum = resid + delta.float()
    want = plain.plain_rmsnorm(want_sum, weight.float(), eps, dtype)

    r = resid.clone().to(DEV)
    out = torch.empty(n, width, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r, delta.to(DEV), weight.to(DEV), eps, out)
    assert torch.equal(r.cpu(), want_sum)                     # the residual took the sum
    assert_close(out, want, dtype, "add_rmsnorm")

    # without a branch output
    out2 = torch.empty(n, width, dtype=dtype, device=DEV)
    r2 = resid.clone().to(DEV)
    ops.add_rmsnorm(r2, None, weight.to(DEV), eps, out2)
    assert torch.equal(r2.cpu(), resid)
    assert_close(out2, plain.plain_rmsnorm(resid, weight.float(), eps, dtype), dtype, "rmsnorm")

    # picked rows: the residual stays as it was
    rows = torch.tensor([5, 0, 18, 5], dtype=torch.int32)
    r3 = resid.clone().to(DEV)
    out3 = torch.empty(4, width, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r3, delta.to(DEV), weight.to(DEV), eps, out3, rows.to(DEV))
    assert torch.equal(r3.cpu(), resid)
    assert_close(out3, want[rows.long()], dtype, "add_rmsnorm rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,rot,page", [(4, 2, 16, 16, 16), (3, 3, 32, 32, 8),
                                                       (6, 1, 48, 48, 32), (5, 5, 80, 32, 4),
                                                       (8, 2, 128, 128, 64), (2, 1, 256, 256, 16)])
def test_rope_kv_write(dtype, heads, kv_heads, d, rot, page):
    ops = _ops()
    g = torch.Generator().manual_seed(d + page)
    theta = 25000.0
    # three sequences; their new tokens start at different positions, one crosses a page's edge
    starts, lens = [0, page - 1, 3 * page + 2], [5, 4, 1]
    slots = [2, 0, 3]
    n = sum(lens)
    positions = torch.tensor([s + i for s, l in zip(starts, lens) for i in range(l)],
                             dtype=torch.int32)
    token_slot = torch.tensor([sl for sl, l in zip(slots, lens) for _ in range(l)],
                              dtype=torch.int32)
    num_pages, max_pages = 24, 6
    table = torch.full((4, max_pages), -1, dtype=torch.int32)
    perm = torch.randperm(num_pages, generator=g).tolist()
    for sl in slots:
        for p in range(max_pages):
            table[sl, p] = perm.pop()
    qkv = torch.randn(n, (heads + 2 * kv_heads) * d, generator=g).to(dtype)
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))

    x = qkv.float().view(n, heads + 2 * kv_heads, d)
    want_q = x[:, :heads].clone()
    want_k = x[:, heads: heads + kv_heads].clone()
    want_q[..., :rot] = plain.plain_rope(want_q[..., :rot], positions, theta, dtype)
    want_k[..., :rot] = plain.plain_rope(want_k[..., :rot], positions, theta, dtype)
    want_v = x[:, heads + kv_heads:]

    k_pages = torch.full((num_pages, kv_heads, page, d), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full_like(k_pages, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    dev_qkv = qkv.to(DEV)
    ops.rope_kv_write(dev_qkv, positions.to(DEV), token_slot.to(DEV), inv_freq.to(DEV), rot, heads,
                      kv_heads, d, k_pages, v_pages, table.to(DEV), True, status)
    assert status.item() == 0
    got = dev_qkv.float().cpu().view(n, heads + 2 * kv_heads, d)
    assert_close(got[:, :heads], want_q, dtype, "rotated q")
    assert torch.equal(got[:, heads:], x[:, heads:]), "k and v in the qkv buffer stay as they were"
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for i in range(n):
        pos, sl = int(positions[i]), int(token_slot[i])
        pid = int(table[sl, pos // page])
        written[pid, pos % page] = True
        assert_close(k_pages[pid, :, pos % page], want_k[i], dtype, "stored k")
        assert torch.equal(v_pages[pid, :, pos % page].float().cpu(), want_v[i]), "stored v"
    # nothing else was touched
    untouched = ~written[:, None, :, None].expand(-1, kv_heads, -1, d)
    assert torch.isnan(k_pages.float().cpu()[untouched]).all()
    assert torch.isnan(v_pages.float().cpu()[untouched]).all()

    # a position without a page is reported, not written
    bad_table = table.clone()
    bad_table[slots[0], 0] = -1
    ops.rope_kv_write(qkv.to(DEV), positions.to(DEV), token_slot.to(DEV), inv_freq.to(DEV), rot,
                      heads, kv_heads, d, k_pages, v_pages, bad_table.to(DEV), True, status)
    assert status.item() == 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(23, 2 * 200, generator=g) * 4).to(dtype)
    out = torch.empty(23, 200, dtype=dtype, device=DEV)
    ops.silu_mul(x.to(DEV), out)
    assert_close(out, plain.plain_swiglu(x[:, :200].float(), x[:, 200:].float(), dtype), dtype,
                 "silu_mul")


@pytest.mark.parametrize("n,k,m", [(1, 64, 50), (7, 100, 256), (65, 2051, 331), (130, 176, 64),
                                   (64, 2048, 2560), (3, 5632, 2048), (20, 2048, 300),
                                   (33, 72, 40), (32, 200, 17)])
def test_gemm_f32(n, k, m):
    """(up to 32 rows take the kernel of narrow tiles, more the wide one; a row alone and the same
    row in a batch of more than 32 go through both and must agree bit for bit)"""
    ops = _ops()
    g = torch.Generator().manual_seed(n + k + m)
    x = torch.randn(n, k, generator=g)
    w = torch.randn(m, k, generator=g)
    out = torch.empty(n, m, dtype=torch.float32, device=DEV)
    ops.gemm_f32(x.to(DEV), w.to(DEV), out)
    assert_close(out, plain.plain_linear(x, w), torch.float32, "gemm_f32")
    # a row's result does not depend on the rows beside it
    one = torch.empty(1, m, dtype=torch.float32, device=DEV)
    ops.gemm_f32(x[n - 1:].to(DEV), w.to(DEV), one)
    assert torch.equal(one.cpu()[0], out.cpu()[n - 1])


def test_gemm_f32_is_true_32_bit():
    """Operands with 12 mantissa bits: a 10-bit (TF32) or 8-bit (bfloat16) mantissa would round
    them to 1 and give exactly k.  Every partial sum n * (1 + 2^-12), n <= 64, fits float32, so
    the true 32-bit result is exact."""
    ops = _ops()
    k = 64
    x = torch.full((4, k), 1.0 + 2.0 ** -12)
    w = torch.ones(8, k)
    out = torch.empty(4, 8, dtype=torch.float32, device=DEV)
    ops.gemm_f32(x.to(DEV), w.to(DEV), out)
    assert torch.all(out.cpu() == k * (1.0 + 2.0 ** -12))


@pytest.mark.parametrize("n,k,m", [(1, 64, 50), (8, 2048, 2560), (100, 120, 331)])
def test_linear_bf16(n, k, m):
    ops = _ops()
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16)
    w = torch.randn(m, k, generator=g).to(torch.bfloat16)
    got = ops.linear(x.to(DEV), w.to(DEV))
    assert got.dtype == torch.bfloat16
    assert_close(got, plain.plain_linear(x.float(), w.float(), torch.bfloat16), torch.bfloat16,
                 "linear bf16")
    wide = ops.linear(x.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert wide.dtype == torch.float32
    assert_close(wide, plain.plain_linear(x.float(), w.float(), torch.bfloat16, keep_f32=True),
                 torch.float32, "linear bf16 -> f32")


@pytest.mark.parametrize("vocab", [32003, 32000, 40004, 64])
def test_sample_rows_greedy_and_ties(vocab):
    """(vocabularies that are and are not multiples of four: 16-byte and single loads)"""
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(9, vocab, generator=g)
    far = vocab - vocab // 30
    logits[3, vocab // 300] = logits[3, far] = 50.0      # a tie: the lowest id wins
    logits[4, vocab - 1] = 60.0                          # the last id
    logits[5, 0] = 60.0
    logits[6, far] = logits[6, far + 1] = 55.0           # a tie inside one 16-byte piece
    out = torch.empty(9, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits.to(DEV), out)
    want = [plain.plain_greedy(row) for row in logits]
    assert out.cpu().tolist() == want
    assert want[3] == vocab // 300 and want[4] == vocab - 1 and want[5] == 0 and want[6] == far


@pytest.mark.parametrize("vocab", [331, 332])
def test_sample_rows_temperature_matches_plain_and_softmax(vocab):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(6, vocab, generator=g) * 2
    temperature = torch.tensor([0.8, 0.0, 1.5, 0.8, 0.3, 1.0])
    seed = torch.tensor([7, 7, 123456789012, 8, 7, -3], dtype=torch.int64)
    position = torch.tensor([5, 5, 70, 5, 6, 0], dtype=torch.int32)
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits.to(DEV), out, temperature.to(DEV), seed.to(DEV), position.to(DEV))
    want = [plain.plain_temperature_sample(logits[r], float(temperature[r]), int(seed[r]),
                                           int(position[r])) for r in range(6)]
    assert out.cpu().tolist() == want
    # the draws follow softmax(logits / T): 4000 positions of one row
    rows = 4000
    many = logits[0:1].expand(rows, vocab).contiguous()
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample_rows(many.to(DEV), out, torch.full((rows,), 0.8, device=DEV),
                    torch.full((rows,), 11, dtype=torch.int64, device=DEV),
                    torch.arange(rows, dtype=torch.int32, device=DEV))
    counts = torch.bincount(out.cpu().long(), minlength=vocab).float()
    probs = plain.softmax_probabilities(logits[0], 0.8)
    top = torch.topk(probs, 5).indices
    for i in top.tolist():
        expect = probs[i].item() * rows
        assert abs(counts[i].item() - expect) <= 5 * np.sqrt(expect) + 3, (i, counts[i], expect)


# ----------------------------------------------------------------------------- attention
def _plain_attention_case(fx, q_list, heads, kv_heads, d, scale, window, dtype):
    outs = []
    for i, q in enumerate(q_list):
        n, ql = fx.kv_lens[i], q.shape[0]
        qpos = torch.arange(n - ql, n)
        outs.append(plain.plain_attention(q, fx.k[i], fx.v[i], qpos, window, dtype, scale)
                    .reshape(ql, heads * d))
    return torch.cat(outs)


def _shapes(dtype, d):
    """The tile shapes to force: the launcher's own choice, and each shape of its kernel alone."""
    from distengine_b200.kernels.attention import uses_tensor_cores
    return [None, "wide", "narrow"] if uses_tensor_cores(dtype, d) else [None]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,page", [(4, 2, 16, 16), (3, 3, 32, 8), (6, 1, 48, 32),
                                                   (8, 1, 64, 16), (5, 5, 80, 4), (16, 2, 128, 64),
                                                   (2, 1, 256, 16), (32, 4, 64, 16), (3, 1, 18, 16),
                                                   (32, 1, 64, 16), (8, 8, 128, 16)])
def test_paged_attention_mixed_batch(dtype, heads, kv_heads, d, page):
    """Prompt portions beside decoded tokens, scrambled block tables, NaN in every free page."""
    g = torch.Generator().manual_seed(heads * d + page)
    kv_lens = [130, 1, 77, 300, 33]
    q_lens = [130, 1, 1, 21, 2]             # whole prompt, first token, decode, portion, two tokens
    fx = PagedFixture(kv_lens, kv_heads, d, page, dtype, DEV, seed=d)
    q_list = [torch.randn(ql, heads, d, generator=g).to(dtype).float() for ql in q_lens]
    scale = d ** -0.5
    want = _plain_attention_case(fx, q_list, heads, kv_heads, d, scale, None, dtype)
    for shape in _shapes(dtype, d):
        got, partials = run_paged_attention(fx, q_list, heads, kv_heads, d, scale, None, chunk=0,
                                            shape=shape)
        assert sum(partials.values()) == 0
        assert_close(got, want, dtype, f"paged attention {shape}")
        got, _ = run_paged_attention(fx, q_list, heads, kv_heads, d, scale, None, shape=shape)
        assert_close(got, want, dtype, f"paged attention, chunk chosen by the plan {shape}")
        # the same with every key range cut into chunks of 64 and merged
        got, partials = run_paged_attention(fx, q_list, heads, kv_heads, d, scale, None, chunk=64,
                                            shape=shape)
        assert sum(partials.values()) > 0
        assert_close(got, want, dtype, f"paged attention, split keys {shape}")
        # and with the fixed-shape plan that a replayed graph uses
        got, _ = run_paged_attention(fx, q_list, heads, kv_heads, d, scale, None, chunk=128,
                                     chunks_cap=4, shape=shape)
        assert_close(got, want, dtype, f"paged attention, capped chunks {shape}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,page,window", [(32, 8, 24), (64, 16, 100), (48, 16, 16), (128, 32, 100)])
def test_paged_attention_window(dtype, d, page, window):
    heads, kv_heads = 4, 2
    g = torch.Generator().manual_seed(window)
    kv_lens, q_lens = [200, 90, 17], [1, 40, 17]
    fx = PagedFixture(kv_lens, kv_heads, d, page, dtype, DEV, seed=window)
    q_list = [torch.randn(ql, heads, d, generator=g).to(dtype).float() for ql in q_lens]
    # the key just outside the first sequence's window would dominate if it were read, and the
    # first key inside must be read
    edge = kv_lens[0] - window
    fx.k[0][edge - 1] = q_list[0][0, :kv_heads] * 4
    fx.k[0][edge] = q_list[0][0, :kv_heads] * 2
    fx.rewrite()
    want = _plain_attention_case(fx, q_list, heads, kv_heads, d, d ** -0.5, window, dtype)
    for shape in _shapes(dtype, d):
        for chunk in (0, None, 64):
            got, _ = run_paged_attention(fx, q_list, heads, kv_heads, d, d ** -0.5, window,
                                         chunk=chunk, shape=shape)
            assert_close(got, want, dtype, f"windowed attention chunk={chunk} {shape}")
    # pages wholly behind the window may be gone from the table: same result
    first_kept = (kv_lens[0] - window + 1) // page
    for p in range(first_kept):
        fx.block_table[fx.slots[0], p] = -1
    for shape in _shapes(dtype, d):
        got, _ = run_paged_attention(fx, q_list, heads, kv_heads, d, d ** -0.5, window, chunk=0,
                                     shape=shape)
        assert_close(got, want, dtype, f"windowed attention, released pages {shape}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 15, 16, 511, 512, 1023, 1100])
@pytest.mark.parametrize("d", [64, 128])
def test_paged_attention_one_far_key_stands_out(dtype, far, d):
    """One key among 1101 is made to dominate one head's softmax: the output must be that key's
    value.  A wrong page, offset or tile edge would show as a different value."""
    heads, kv_heads, page = 8, 2, 16
    g = torch.Generator().manual_seed(far)
    fx = PagedFixture([1101], kv_heads, d, page, dtype, DEV, seed=far)
    q = torch.randn(1, heads, d, generator=g).to(dtype).float()
    q[0, 5] = (q[0, 5] / q[0, 5].norm() * 8).to(dtype).float()
    fx.k[0][far, 1] = (q[0, 5] * 4).to(dtype).float()         # head 5 reads kv head 1
    fx.rewrite()
    want = _plain_attention_case(fx, [q], heads, kv_heads, d, d ** -0.5, None, dtype)
    assert torch.allclose(want[0, 5 * d: 6 * d], fx.v[0][far, 1], atol=2e-2)
    for shape in _shapes(dtype, d):
        for chunk in (0, 256):
            got, _ = run_paged_attention(fx, [q], heads, kv_heads, d, d ** -0.5, None, chunk=chunk,
                                         shape=shape)
            assert_close(got, want, dtype, f"far key {far} chunk={chunk} {shape}")


@pytest.mark.parametrize("writes", [True, False])
@pytest.mark.parametrize("heads,kv_heads,d,page,rot,window",
                         [(8, 2, 64, 16, 64, None), (6, 1, 48, 32, 24, None),
                          (32, 4, 64, 16, 64, None), (16, 2, 128, 64, 128, 100),
                          (40, 2, 32, 8, 32, None), (4, 4, 16, 16, 0, None),
                          (3, 1, 80, 4, 80, 7)])
def test_decode_attention_in_one_launch(heads, kv_heads, d, page, rot, window, writes):
    """Decoded tokens: rotation of q and k, the cache write, attention and the merge of split key
    ranges in one kernel.  The token's own key is not in the cache beforehand (NaN stands there),
    so it must come from the launch itself; with ``writes`` off it is there and must be left."""
    from gpu_helpers import run_decode_attention
    dtype, theta = torch.bfloat16, 10000.0
    g = torch.Generator().manual_seed(heads * d + page)
    kv_lens = [130, 1, 77, 300, 1101, 64, 65]
    n = len(kv_lens)
    fx = PagedFixture(kv_lens, kv_heads, d, page, dtype, DEV, seed=d + page)
    qkv = torch.randn(n, (heads + 2 * kv_heads) * d, generator=g).to(dtype)
    x = qkv.float().view(n, heads + 2 * kv_heads, d)
    positions = torch.tensor([length - 1 for length in kv_lens], dtype=torch.int32)
    q, k_new = x[:, :heads].clone(), x[:, heads: heads + kv_heads].clone()
    inv_freq = None
    if rot:
        inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
        q[..., :rot] = plain.plain_rope(q[..., :rot], positions, theta, dtype)
        k_new[..., :rot] = plain.plain_rope(k_new[..., :rot], positions, theta, dtype)
    v_new = x[:, heads + kv_heads:]
    for i in range(n):
        fx.k[i][-1], fx.v[i][-1] = k_new[i], v_new[i]
    want = _plain_attention_case(fx, [q[i: i + 1] for i in range(n)], heads, kv_heads, d,
                                 d ** -0.5, window, dtype)
    fx.rewrite()
    pages_full = fx.k_pages.clone(), fx.v_pages.clone()
    if writes:                                # the cache does not hold the tokens' own keys yet
        for i, length in enumerate(kv_lens):
            pid = int(fx.block_table[fx.slots[i], (length - 1) // page])
            fx.k_pages[pid, :, (length - 1) % page] = float("nan")
            fx.v_pages[pid, :, (length - 1) % page] = float("nan")
    # the launcher's choice; one block; a cluster of 4 and of 8; several clusters a tile, which
    # merge through global memory (twice on the same buffers: the counters must be zero again);
    # clusters of one block
    for split, repeats in ((None, 1), ((1, 1, 2048), 1), ((4, 1, 320), 1), ((8, 1, 192), 2),
                           ((2, 3, 192), 3), ((1, 5, 256), 2), ((4, 2, 192), 1),
                           ((6, 1, 256), 1), ((3, 2, 192), 2), ((7, 1, 192), 1), ((5, 1, 256), 1)):
        got, k_after, v_after = run_decode_attention(
            fx, qkv, heads, kv_heads, d, d ** -0.5, window, inv_freq, rot, writes, split=split,
            repeats=repeats)
        chunk = split
        assert_close(got, want, dtype, f"decode attention split={split}")
        # the pages afterwards: the tokens' keys and values where they belong, the rest untouched
        # (NaN in free pages and beyond the sequences' ends included)
        fresh = torch.zeros(fx.k_pages.shape[0], page, dtype=torch.bool)
        for i, length in enumerate(kv_lens):
            fresh[int(fx.block_table[fx.slots[i], (length - 1) // page]), (length - 1) % page] = True
        for after, full in ((k_after, pages_full[0]), (v_after, pages_full[1])):
            after, full = after.transpose(1, 2), full.transpose(1, 2)      # [pages, page, kv, d]
            same = (after == full) | (torch.isnan(after) & torch.isnan(full))
            assert same[~fresh].all(), f"pages after the decode kernel, chunk={chunk}"
            assert_close(after[fresh], full[fresh], dtype, "the tokens' own keys and values")


def test_attention_refuses_sizes_it_does_not_take():
    from distengine_b200.kernels.attention import AttentionLauncher
    with pytest.raises(ValueError, match="head sizes"):
        AttentionLauncher(torch.bfloat16, 4, 2, 257, 1.0, None)
    with pytest.raises(ValueError, match="head sizes"):
        AttentionLauncher(torch.float32, 4, 2, 33, 1.0, None)
    with pytest.raises(ValueError, match="multiple"):
        AttentionLauncher(torch.float32, 5, 2, 32, 1.0, None)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 31, 32])
@pytest.mark.parametrize("k,n", [(64, 50), (2048, 2560), (120, 331), (5632, 2048), (200, 8)])
def test_linear_small(m, k, n, monkeypatch):
    """The weight-streaming product for a handful of tokens, plain and with float32 output: all
    row counts the kernel takes, also those that the engine gives to the library product."""
    ops = _ops()
    g = torch.Generator().manual_seed(m * k + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16)
    from distengine_b200.kernels import ops as raw
    monkeypatch.setattr(raw, "SMALL_ROWS", 32)
    assert raw._small_ok(x.to(DEV), w.to(DEV))
    got = ops.linear(x.to(DEV), w.to(DEV))
    assert_close(got, plain.plain_linear(x.float(), w.float(), torch.bfloat16), torch.bfloat16,
                 "linear_small")
    wide = ops.linear(x.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert_close(wide, plain.plain_linear(x.float(), w.float(), torch.bfloat16, keep_f32=True),
                 torch.float32, "linear_small -> f32")
    # rows of a wider buffer as input (a row stride that is not the width)
    buf = torch.zeros(m, k + 64, dtype=torch.bfloat16, device=DEV)
    buf[:, :k] = x.to(DEV)
    again = ops.linear(buf[:, :k], w.to(DEV))
    assert torch.equal(again, got)


@pytest.mark.parametrize("m", [1, 8, 13, 32, 40])
@pytest.mark.parametrize("k,inner", [(64, 176), (2048, 5632), (120, 200)])
@pytest.mark.parametrize("small_rows", [16, 32])
def test_linear_gated(m, k, inner, small_rows, monkeypatch):
    """silu(gate) * up in the product's epilogue (up to 32 rows) and as product + kernel."""
    from distengine_b200.kernels import ops as raw
    monkeypatch.setattr(raw, "SMALL_ROWS", small_rows)
    ops = _ops()
    g = torch.Generator().manual_seed(m + k + inner)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inner, k, generator=g) * 0.1).to(torch.bfloat16)
    out = torch.empty(m, inner, dtype=torch.bfloat16, device=DEV)
    ops.linear_gated(x.to(DEV), w.to(DEV), out)
    gate = plain.plain_linear(x.float(), w[:inner].float(), torch.bfloat16)
    up = plain.plain_linear(x.float(), w[inner:].float(), torch.bfloat16)
    assert_close(out, plain.plain_swiglu(gate, up, torch.bfloat16), torch.bfloat16, "linear_gated")


@pytest.mark.parametrize("m", [17, 32, 50, 64, 100, 128])
@pytest.mark.parametrize("k,n", [(64, 50), (2048, 2560), (120, 331), (5632, 2048), (200, 8),
                                 (2048, 4100)])
def test_linear_mid(m, k, n, monkeypatch):
    """The swapped-operand tcgen05 product for 17 to 128 tokens (all token counts the kernel takes,
    also those that the engine gives to the library product): bfloat16 and float32 output, the
    split of k chosen by the kernel and every split forced, the gated epilogue."""
    from distengine_b200.kernels import library
    from distengine_b200.kernels import ops as raw
    monkeypatch.setattr(raw, "MID_ROWS", 128)
    g = torch.Generator().manual_seed(m * k + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16)
    dx, dw = x.to(DEV), w.to(DEV)
    assert raw._mid_ok(dx, dw)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = plain.plain_linear(x.float(), w.float(), torch.bfloat16)
    got = raw.linear(dx, dw, status=status)
    assert status.item() == 0
    assert_close(got, want, torch.bfloat16, "linear_mid")
    wide = raw.linear(dx, dw, out_dtype=torch.float32, status=status)
    assert_close(wide, plain.plain_linear(x.float(), w.float(), torch.bfloat16, keep_f32=True),
                 torch.float32, "linear_mid -> f32")
    lib = library.load("linear_mid")
    for split in (1, 2, 4, 8):
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        code = lib.de_linear_mid(dx.data_ptr(), dx.stride(0), dw.data_ptr(), dw.stride(0),
                                 out.data_ptr(), out.stride(0), m, n, k, 0, 0, 0, 0, 0, 0.0, 0, 0,
                                 0, 0, split, status.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
        assert code == 0 and status.item() == 0
        assert_close(out, want, torch.bfloat16, f"linear_mid split {split}")
    if n % 2 == 0:
        inner = n // 2
        out = torch.empty(m, inner, dtype=torch.bfloat16, device=DEV)
        raw.linear_gated(dx, dw, out, status=status)
        assert status.item() == 0
        gate = plain.plain_linear(x.float(), w[:inner].float(), torch.bfloat16)
        up = plain.plain_linear(x.float(), w[inner:].float(), torch.bfloat16)
        assert_close(out, plain.plain_swiglu(gate, up, torch.bfloat16), torch.bfloat16,
                     "linear_mid gated")


@pytest.mark.parametrize("m", [1, 5, 8, 11, 16, 17, 40, 64, 128])
@pytest.mark.parametrize("width,inner,eps", [(2048, 5632, 1e-5), (120, 200, 3e-6), (4096, 1024, 1e-6),
                                             (72, 4800, 1e-5)])
def test_norm_carried_by_the_products_around_it(m, width, inner, eps, monkeypatch):
    """down -> (residual sum, RMS norm) -> gate/up and -> plain product, with the norm's work done
    by the epilogues of the products: the residual, and the outputs of the products after the
    norm, against the plain product, sum, norm, product.  Up to 16 tokens in the weight-streaming
    kernel, more in the swapped-operand tcgen05 kernel."""
    from types import SimpleNamespace
    from distengine_b200.kernels import ops as raw
    monkeypatch.setattr(raw, "MID_ROWS", 128)
    g = torch.Generator().manual_seed(m * width + inner)
    act = torch.randn(m, inner, generator=g).to(torch.bfloat16)
    w_down = (torch.randn(width, inner, generator=g) * 0.05).to(torch.bfloat16)
    resid = torch.randn(m, width, generator=g) * 3.0
    resid[m // 2] *= 40.0                                  # rows of very different norms
    norm_w = (1.0 + 0.5 * torch.randn(width, generator=g)).to(torch.bfloat16)
    w_next = (torch.randn(2 * inner, width, generator=g) * 0.1).to(torch.bfloat16)
    dev = lambda t: t.to(DEV)
    count = raw.norm_ride_parts(m, dev(w_down), torch.bfloat16)
    assert count > 0
    ahead = SimpleNamespace(resid=dev(resid).clone(), weight=dev(norm_w),
                            parts=torch.full((m, count), float("nan"), device=DEV),
                            width=width, eps=eps)
    rows = torch.full((m, width), float("nan"), dtype=torch.bfloat16, device=DEV)
    raw.linear(dev(act), dev(w_down), out=rows, after=ahead)
    # plain: product (rounded), sum in float32, norm
    branch = plain.plain_linear(act.float(), w_down.float(), torch.bfloat16)
    total = resid + branch
    # (the branch is a bfloat16 value: where the kernel's float32 sum and the plain float64 sum
    # fall on different sides of a rounding boundary the residual differs by a bfloat16 step)
    assert_close(ahead.resid, total, torch.bfloat16, "residual sum in the epilogue")
    squares = ahead.parts.sum(dim=1).cpu()
    mine = ahead.resid.cpu()
    assert torch.allclose(squares, (mine * mine).sum(dim=1), rtol=1e-5)
    assert torch.equal(rows.cpu(), (mine * norm_w.float()).to(torch.bfloat16))
    normed = plain.plain_rmsnorm(total, norm_w.float(), eps, torch.bfloat16)
    out = torch.empty(m, inner, dtype=torch.bfloat16, device=DEV)
    raw.linear_gated(rows, dev(w_next), out, before=ahead)
    gate = plain.plain_linear(normed, w_next[:inner].float(), torch.bfloat16)
    up = plain.plain_linear(normed, w_next[inner:].float(), torch.bfloat16)
    assert_close(out, plain.plain_swiglu(gate, up, torch.bfloat16), torch.bfloat16,
                 "gated product after the carried norm")
    out = torch.empty(m, 2 * inner, dtype=torch.bfloat16, device=DEV)
    raw.linear(rows, dev(w_next), out=out, before=ahead)
    assert_close(out, plain.plain_linear(normed, w_next.float(), torch.bfloat16), torch.bfloat16,
                 "product after the carried norm")


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (77, 200, 120), (300, 384, 2048), (129, 331 + 5, 72),
                                   (2048, 256, 5632), (33, 50, 8), (2048, 2560, 136),
                                   (1500, 4100, 72), (20000, 264, 64)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(m, n, k, out_dtype):
    """The tensor-memory matrix product (TMA + tcgen05.mma) at sizes that are no multiples of its
    tiles; a poisoned output shows rows or columns it would skip."""
    ops = _ops()
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.gemm_tcgen05(x.to(DEV), w.to(DEV), out, status=status)
    assert status.item() == 0
    want = plain.plain_linear(x.float(), w.float(), torch.bfloat16, keep_f32=out_dtype == torch.float32)
    assert_close(out, want, out_dtype, "gemm_tcgen05")


@pytest.mark.parametrize("m,inner,k", [(128, 64, 64), (200, 192, 120), (2048, 5632, 2048), (40, 320, 264),
                                       (1100, 176, 72), (3000, 1000, 40)])
def test_gemm_tcgen05_gated(m, inner, k):
    """silu(gate) * up as the epilogue of the tensor-memory product."""
    ops = _ops()
    g = torch.Generator().manual_seed(m + inner + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inner, k, generator=g) * 0.1).to(torch.bfloat16)
    out = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.gemm_tcgen05(x.to(DEV), w.to(DEV), out, gated=True, status=status)
    assert status.item() == 0
    gate = plain.plain_linear(x.float(), w[:inner].float(), torch.bfloat16)
    up = plain.plain_linear(x.float(), w[inner:].float(), torch.bfloat16)
    assert_close(out, plain.plain_swiglu(gate, up, torch.bfloat16), torch.bfloat16, "gated tcgen05")


def test_products_of_many_rows_take_the_tcgen05_kernel():
    """From a thousand rows on, ``linear`` (in a shape that suits it) and ``linear_gated`` run this
    package's tcgen05 kernel: the results agree with the plain product, and the kernel library is
    the one that was called (its launch leaves the status word alone, the output is written)."""
    from distengine_b200.kernels import ops as raw
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    m, k, n, inner = 2048, 64, 2048, 200
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16)
    dev_x, dev_w = x.to(DEV), w.to(DEV)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert raw._tcgen05_fits(dev_x, dev_w, out)
    assert not raw._tcgen05_fits(dev_x[:1000], dev_w, out[:1000])
    assert not raw._tcgen05_fits(dev_x, dev_w[:2560 - 2048 + 100], out[:, :612])
    ops.linear(dev_x, dev_w, out=out)
    assert_close(out, plain.plain_linear(x.float(), w.float(), torch.bfloat16), torch.bfloat16,
                 "linear, many rows")
    wg = (torch.randn(2 * inner, k, generator=g) * 0.1).to(torch.bfloat16)
    dev_wg = wg.to(DEV)
    assert not raw.gated_needs_scratch(dev_x, dev_wg)
    assert raw.gated_needs_scratch(dev_x[:500], dev_wg)
    act = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.linear_gated(dev_x, dev_wg, act)
    gate = plain.plain_linear(x.float(), wg[:inner].float(), torch.bfloat16)
    up = plain.plain_linear(x.float(), wg[inner:].float(), torch.bfloat16)
    assert_close(act, plain.plain_swiglu(gate, up, torch.bfloat16), torch.bfloat16,
                 "linear_gated, many rows")
