"""Helpers of the GPU tests: tolerances, a paged cache built from dense keys and values."""

from __future__ import annotations

import numpy as np
import torch

# Tolerances, set once.  float32: the engine and the plain implementation differ by the order of
# float32 additions only.  bfloat16: both round activations to bfloat16 (eps 2^-8) at the same
# places, but sums are formed in different orders, so roundings flip by one unit here and there and
# the flips spread through the layers.
F32_REL = 2e-5          # max |a - b| <= F32_REL * max(1, max |b|)
BF16_MAX_REL = 4e-2     # max |a - b| <= BF16_MAX_REL * max |b|
BF16_RMS_REL = 1e-2     # rms(a - b)  <= BF16_RMS_REL * max |b|


def assert_close(got, want, dtype: torch.dtype, what: str = "") -> None:
    got = torch.as_tensor(got, dtype=torch.float32).cpu()
    want = torch.as_tensor(want, dtype=torch.float32).cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: result is not finite"
    err = (got - want).abs()
    scale = want.abs().max().item()
    if dtype == torch.float32:
        bound = F32_REL * max(1.0, scale)
        assert err.max().item() <= bound, (
            f"{what}: max error {err.max().item():.3e} > {bound:.3e} (scale {scale:.3e}) at "
            f"{np.unravel_index(int(err.argmax()), tuple(err.shape))}")
    else:
        assert err.max().item() <= BF16_MAX_REL * scale, (
            f"{what}: max error {err.max().item():.3e} > {BF16_MAX_REL * scale:.3e} at "
            f"{np.unravel_index(int(err.argmax()), tuple(err.shape))}")
        rms = err.pow(2).mean().sqrt().item()
        assert rms <= BF16_RMS_REL * scale, f"{what}: rms error {rms:.3e} > {BF16_RMS_REL * scale:.3e}"


class PagedFixture:
    """Dense keys/values of several sequences laid into pages through a scrambled block table.
    Free pages hold NaN so that a read outside a sequence's own keys shows."""

    def __init__(self, kv_lens, kv_heads, head_dim, page, dtype, device, seed=0, spare_pages=5):
        g = torch.Generator().manual_seed(seed)
        self.page, self.kv_lens = page, list(kv_lens)
        need = [(n + page - 1) // page for n in kv_lens]
        total = sum(need) + spare_pages
        order = torch.randperm(total, generator=g).tolist()
        max_pages = max(need) + 2
        self.block_table = torch.full((len(kv_lens) + 3, max_pages), -1, dtype=torch.int32)
        # slots are scrambled too: sequence i lives in slot slots[i]
        self.slots = torch.randperm(len(kv_lens) + 3, generator=g)[: len(kv_lens)].tolist()
        self.k = [torch.randn(n, kv_heads, head_dim, generator=g) for n in kv_lens]
        self.v = [torch.randn(n, kv_heads, head_dim, generator=g) for n in kv_lens]
        self.k = [t.to(dtype).float() for t in self.k]
        self.v = [t.to(dtype).float() for t in self.v]
        self.k_pages = torch.full((total, kv_heads, page, head_dim), float("nan"))
        self.v_pages = torch.full((total, kv_heads, page, head_dim), float("nan"))
        at = 0
        for i, n in enumerate(kv_lens):
            for p in range(need[i]):
                pid = order[at]
                at += 1
                self.block_table[self.slots[i], p] = pid
                lo, hi = p * page, min((p + 1) * page, n)
                self.k_pages[pid, :, : hi - lo] = self.k[i][lo:hi].transpose(0, 1)
                self.v_pages[pid, :, : hi - lo] = self.v[i][lo:hi].transpose(0, 1)
        self.dtype, self.device = dtype, device

    def rewrite(self):
        """Lay self.k / self.v into the pages again (after a test changed them)."""
        for i, n in enumerate(self.kv_lens):
            for p in range((n + self.page - 1) // self.page):
                pid = int(self.block_table[self.slots[i], p])
                lo, hi = p * self.page, min((p + 1) * self.page, n)
                self.k_pages[pid, :, : hi - lo] = self.k[i][lo:hi].transpose(0, 1)
                self.v_pages[pid, :, : hi - lo] = self.v[i][lo:hi].transpose(0, 1)

    def to_device(self):
        return (self.k_pages.to(self.device, self.dtype).contiguous(),
                self.v_pages.to(self.device, self.dtype).contiguous(),
                self.block_table.to(self.device))


def run_paged_attention(fx: PagedFixture, q_list, heads, kv_heads, head_dim, scale, window,
                        chunk=None, chunks_cap=None, shape=None):
    """q_list[i]: [q_len_i, heads, d] float32 queries of the LAST q_len_i positions of sequence i.
    Runs the engine's own launcher (``kernels.attention.AttentionLauncher``): ``chunk`` /
    ``chunks_cap`` pin how key ranges are split (0: not at all, None: the launcher's choice),
    ``shape`` pins the tile shape.  Returns the output [N, heads*d] float32 on the CPU and the
    number of partial results per tile shape."""
    from types import SimpleNamespace
    from distengine_b200.kernels.attention import AttentionLauncher
    from distengine_b200.parts.context import StepPrep, Workspace
    dev, dtype = fx.device, fx.dtype
    qlen = np.array([q.shape[0] for q in q_list], dtype=np.int32)
    pos0 = np.array([n - ql for n, ql in zip(fx.kv_lens, qlen)], dtype=np.int32)
    qstart = (np.cumsum(qlen) - qlen).astype(np.int32)
    launcher = AttentionLauncher(dtype, heads, kv_heads, head_dim, scale, window)
    prep = StepPrep(SimpleNamespace(seq_qlen=qlen, seq_pos0=pos0))
    launcher.prepare(prep, force_chunk=chunk, force_cap=chunks_cap, force_shape=shape,
                     allow_decode=False)
    q = torch.cat([t.reshape(t.shape[0], heads * head_dim) for t in q_list]).to(dev, dtype)
    # q lives inside a wider row, as in the engine's fused qkv buffer
    wide = torch.zeros(q.shape[0], heads * head_dim + 2 * kv_heads * head_dim, dtype=dtype,
                       device=dev)
    wide[:, : heads * head_dim] = q
    out = torch.full((q.shape[0], heads * head_dim), float("nan"), dtype=dtype, device=dev)
    k_pages, v_pages, table = fx.to_device()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    workspace = Workspace(torch.device(dev))
    ctx = SimpleNamespace(seq_slot=t(np.array(fx.slots)), seq_qstart=t(qstart), seq_qlen=t(qlen),
                          seq_pos0=t(pos0), notes=prep.notes,
                          arrays={k: t(v) for k, v in prep.extra.items()},
                          buffer=lambda name, shape, dt=None: workspace.get(name, shape, dt or dtype))
    launcher.run(wide, out, k_pages, v_pages, table, ctx)
    torch.cuda.synchronize()
    return out.float().cpu(), dict(prep.notes[launcher.key])


def run_decode_attention(fx: PagedFixture, qkv, heads, kv_heads, head_dim, scale, window, inv_freq,
                         rotary_dim, writes, split=None, repeats=1):
    """One decoded token per sequence of ``fx`` (at its last position) through the launcher's
    one-kernel decode path.  ``qkv`` [sequences, (heads + 2 kv_heads) * d]: unrotated q, k, v of
    the tokens.  ``split``: (blocks a cluster, clusters a tile, chunk length) or None for the
    launcher's choice.  Returns the output (float32, CPU) and the pages afterwards (float32, CPU)."""
    from types import SimpleNamespace
    from distengine_b200.kernels.attention import AttentionLauncher
    from distengine_b200.parts.context import StepPrep, Workspace
    dev, dtype = fx.device, fx.dtype
    n = len(fx.kv_lens)
    qlen = np.ones(n, dtype=np.int32)
    pos0 = np.array([length - 1 for length in fx.kv_lens], dtype=np.int32)
    qstart = np.arange(n, dtype=np.int32)
    launcher = AttentionLauncher(dtype, heads, kv_heads, head_dim, scale, window)
    prep = StepPrep(SimpleNamespace(seq_qlen=qlen, seq_pos0=pos0,
                                    seq_slot=np.array(fx.slots, dtype=np.int32)))
    launcher.prepare(prep, force_split=split)
    k_pages, v_pages, table = fx.to_device()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)
    workspace = Workspace(torch.device(dev))
    ctx = SimpleNamespace(seq_slot=t(np.array(fx.slots)), seq_qstart=t(qstart), seq_qlen=t(qlen),
                          seq_pos0=t(pos0), notes=prep.notes,
                          arrays={k: t(v) for k, v in prep.extra.items()},
                          status=torch.zeros(1, dtype=torch.int32, device=dev),
                          buffer=lambda name, shape, dt=None, zero=False: workspace.get(
                              name, shape, dt or dtype, zero))
    assert launcher.decode_step(ctx), "a step of single tokens must take the decode kernel"
    dev_qkv = qkv.to(dev, dtype)
    before = dev_qkv.clone()
    for _ in range(repeats):        # again on the same buffers: counters must be left at zero
        out = torch.full((n, heads * head_dim), float("nan"), dtype=dtype, device=dev)
        launcher.run_decode(dev_qkv, out, k_pages, v_pages, table,
                            None if inv_freq is None else inv_freq.to(dev), rotary_dim, writes, ctx)
    torch.cuda.synchronize()
    assert ctx.status.item() == 0
    assert torch.equal(dev_qkv, before), "the decode kernel must leave qkv as it was"
    return out.float().cpu(), k_pages.float().cpu(), v_pages.float().cpu()


class PartHarness:
    """Runs single parts through the engine's own step machinery (``StepRunner`` and
    ``CacheManager``): ``run(entries, fn)`` calls ``fn(ctx, bindings)`` with the step's context."""

    class _Config:
        def __init__(self, vocabulary, width):
            self.vocabulary, self.width = vocabulary, width

    class _Model:
        def __init__(self, parts, dtype, device, vocabulary, width):
            self.parts, self.dtype, self.device = parts, dtype, torch.device(device)
            self.config = PartHarness._Config(vocabulary, width)
            self.fn = None

        def prepare(self, prep):
            for part in self.parts:
                part.prepare(prep)

        def forward(self, ctx, bindings):
            return self.fn(ctx, bindings)

    def __init__(self, parts, cache_specs, dtype, page_size=16, num_pages=64, max_seqs=8,
                 max_len=1024, device="cuda:0", reads=None, vocabulary=1000, width=1):
        from distengine_b200.cache import CacheManager
        from distengine_b200.engine.step import StepRunner
        self.model = self._Model(parts, dtype, device, vocabulary, width)
        self.cache = CacheManager(cache_specs, reads or [None] * len(cache_specs), page_size,
                                  num_pages, max_seqs, max_len, dtype, device,
                                  poison_freed_pages=True)
        self.runner = StepRunner(self.model, self.cache)

    def run(self, entries, fn):
        """entries: list of (request id, number of new tokens)."""
        from distengine_b200.engine.step import StepEntry
        self.model.fn = fn
        out = self.runner.step([StepEntry(rid, [0] * n, []) for rid, n in entries])
        self.runner.check_status()
        return out
