"""Each part of a layer alone, built from a PartSpec through the registries and run through the
engine's step machinery, against the plain function of the same part; sizes differ from the
models' (a width and head counts that are no power of two, partial rotation, a window)."""

import pytest
import torch

import plain_llama as plain
from gpu_helpers import PartHarness, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _specs():
    from distengine_b200.config.model import PartSpec
    return PartSpec


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from distengine_b200.parts import ResidualStream, build_norm
    PartSpec = _specs()
    width, eps = 200, 2e-6
    norm = build_norm(PartSpec.of("rmsnorm", width=width, eps=eps), dtype, torch.device(DEV))
    assert norm.tensors() == {"weight": ((width,), "vector")}
    g = torch.Generator().manual_seed(0)
    weight = torch.rand(width, generator=g) + 0.5
    norm.load({"weight": weight})
    resid, branch = torch.randn(11, width, generator=g), torch.randn(11, width, generator=g).to(dtype)
    h = PartHarness([norm], [], dtype)

    def fn(ctx, bindings):
        stream = ResidualStream(resid.to(DEV))
        stream.pending = branch.to(DEV)
        out = norm.forward(stream, ctx).clone()
        assert stream.pending is None
        return out, stream.resid.clone()

    out, new_resid = h.run([("a", 11)], fn)
    assert torch.equal(new_resid.cpu(), resid + branch.float())
    assert_close(out, plain.plain_rmsnorm(resid + branch.float(), weight, eps, dtype), dtype)


def test_rotary_table_and_no_position_encoding():
    from distengine_b200.parts import build_position_encoding
    PartSpec = _specs()
    rope = build_position_encoding(PartSpec.of("rope", rotary_dim=48, theta=25000.0),
                                   torch.float32, torch.device(DEV))
    table, dim = rope.rotation_table()
    assert dim == 48 and torch.equal(table.cpu(), plain.plain_inv_freq(48, 25000.0))
    none = build_position_encoding(PartSpec.of("none"), torch.float32, torch.device(DEV))
    assert none.rotation_table() == (None, 0)
    with pytest.raises(ValueError, match="unknown position encoding"):
        build_position_encoding(PartSpec.of("alibi"), torch.float32, torch.device(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from distengine_b200.parts import build_feed_forward
    PartSpec = _specs()
    width, inner = 120, 200
    mlp = build_feed_forward(PartSpec.of("gated_mlp", width=width, inner=inner,
                                         activation="silu"), dtype, torch.device(DEV))
    g = torch.Generator().manual_seed(1)
    w = {"gate_proj.weight": torch.randn(inner, width, generator=g) * 0.1,
         "up_proj.weight": torch.randn(inner, width, generator=g) * 0.1,
         "down_proj.weight": torch.randn(width, inner, generator=g) * 0.1}
    assert {k: v[0] for k, v in mlp.tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    mlp.load(w)
    x = torch.randn(9, width, generator=g).to(dtype)
    h = PartHarness([mlp], [], dtype)
    out = h.run([("a", 9)], lambda ctx, b: mlp.forward(x.to(DEV), ctx).clone())
    want = plain.plain_mlp(x.float(), w["gate_proj.weight"], w["up_proj.weight"],
                           w["down_proj.weight"], dtype)
    assert_close(out, want, dtype, "gated mlp")
    with pytest.raises(ValueError, match="gelu"):
        build_feed_forward(PartSpec.of("gated_mlp", width=8, inner=8, activation="gelu"), dtype,
                           torch.device(DEV))


def _attention(dtype, width, heads, kv_heads, d, rot, window, theta=5000.0):
    from distengine_b200.parts import build_mixer
    PartSpec = _specs()
    spec = PartSpec.of("attention", width=width, heads=heads, kv_heads=kv_heads, head_dim=d,
                       scale=d ** -0.5, window=window,
                       position=PartSpec.of("rope", rotary_dim=rot, theta=theta))
    return build_mixer(spec, dtype, torch.device(DEV))


def _plain_attention_part(x, w, heads, kv_heads, d, rot, window, theta, dtype):
    T = x.shape[0]
    pos = torch.arange(T)
    q = plain.plain_linear(x, w["q_proj.weight"], dtype).view(T, heads, d)
    k = plain.plain_linear(x, w["k_proj.weight"], dtype).view(T, kv_heads, d)
    v = plain.plain_linear(x, w["v_proj.weight"], dtype).view(T, kv_heads, d)
    q = torch.cat((plain.plain_rope(q[..., :rot], pos, theta, dtype), q[..., rot:]), -1)
    k = torch.cat((plain.plain_rope(k[..., :rot], pos, theta, dtype), k[..., rot:]), -1)
    ctx = plain.plain_attention(q, k, v, pos, window, dtype)
    return plain.plain_linear(ctx.reshape(T, heads * d), w["o_proj.weight"], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,rot,window,page", [(6, 2, 48, 48, None, 16),
                                                              (5, 5, 32, 16, None, 8),
                                                              (4, 1, 64, 64, 20, 4)])
def test_attention_part_in_portions(dtype, heads, kv_heads, d, rot, window, page):
    width, theta = 120, 5000.0
    mixer = _attention(dtype, width, heads, kv_heads, d, rot, window, theta)
    g = torch.Generator().manual_seed(d)
    w = {"q_proj.weight": torch.randn(heads * d, width, generator=g) * 0.1,
         "k_proj.weight": torch.randn(kv_heads * d, width, generator=g) * 0.1,
         "v_proj.weight": torch.randn(kv_heads * d, width, generator=g) * 0.1,
         "o_proj.weight": torch.randn(width, heads * d, generator=g) * 0.1}
    mixer.load(w)
    spec = mixer.cache_spec()
    assert (spec.kv_heads, spec.head_dim, spec.window) == (kv_heads, d, window)
    xs = {"a": torch.randn(75 + 7, width, generator=g).to(dtype),
          "b": torch.randn(40 + 6, width, generator=g).to(dtype)}
    want = {rid: _plain_attention_part(x.float(), w, heads, kv_heads, d, rot, window, theta, dtype)
            for rid, x in xs.items()}
    h = PartHarness([mixer], [spec], dtype, page_size=page, num_pages=40)
    fed = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    # portions of a beside portions and single tokens of b; then steps of single tokens only
    # (the one-launch decode kernel in bfloat16: rotation, cache write, window, pages that are
    # gone from the table)
    for na, nb in [(30, 1), (2, 1), (1, 17), (25, 0), (17, 21)] + [(1, 1)] * 6 + [(1, 0)]:
        entries = [(rid, n) for rid, n in (("a", na), ("b", nb)) if n]
        x = torch.cat([xs[rid][fed[rid]: fed[rid] + n] for rid, n in entries]).to(DEV)
        out = h.run(entries, lambda ctx, b: mixer.forward(x, ctx, b[0]).clone()).cpu()
        at = 0
        for rid, n in entries:
            got[rid].append(out[at: at + n])
            at += n
            fed[rid] += n
    for rid in xs:
        assert_close(torch.cat(got[rid]), want[rid], dtype, f"attention part {rid}")
    if window is not None:      # pages behind the window went back to the pool
        held = sum(p >= 0 for p in h.cache.paged[0].tables["a"])
        assert held <= (window + page - 1) // page + 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block(dtype):
    """The arrangement: x += mixer(norm(x)); x += feed_forward(norm(x)), sums in 32-bit."""
    from distengine_b200.parts import (ResidualStream, build_block, build_feed_forward,
                                       build_norm)
    PartSpec = _specs()
    width, heads, kv_heads, d, inner, eps, theta = 72, 3, 1, 32, 100, 1e-5, 1e4
    dev = torch.device(DEV)
    mixer = _attention(dtype, width, heads, kv_heads, d, d, None, theta)
    ffn = build_feed_forward(PartSpec.of("gated_mlp", width=width, inner=inner, activation="silu"),
                             dtype, dev)
    norms = [build_norm(PartSpec.of("rmsnorm", width=width, eps=eps), dtype, dev) for _ in range(3)]
    block = build_block("prenorm", mixer, ffn, norms[0], norms[1])
    g = torch.Generator().manual_seed(3)
    w = {"model.layers.0.self_attn.q_proj.weight": torch.randn(heads * d, width, generator=g) * 0.1,
         "model.layers.0.self_attn.k_proj.weight": torch.randn(kv_heads * d, width, generator=g) * 0.1,
         "model.layers.0.self_attn.v_proj.weight": torch.randn(kv_heads * d, width, generator=g) * 0.1,
         "model.layers.0.self_attn.o_proj.weight": torch.randn(width, heads * d, generator=g) * 0.1,
         "model.layers.0.mlp.gate_proj.weight": torch.randn(inner, width, generator=g) * 0.1,
         "model.layers.0.mlp.up_proj.weight": torch.randn(inner, width, generator=g) * 0.1,
         "model.layers.0.mlp.down_proj.weight": torch.randn(width, inner, generator=g) * 0.1,
         "model.layers.0.input_layernorm.weight": torch.rand(width, generator=g) + 0.5,
         "model.layers.0.post_attention_layernorm.weight": torch.rand(width, generator=g) + 0.5}
    p = "model.layers.0."
    mixer.load({k[len(p + "self_attn."):]: v for k, v in w.items() if "self_attn" in k})
    ffn.load({k[len(p + "mlp."):]: v for k, v in w.items() if ".mlp." in k})
    norms[0].load({"weight": w[p + "input_layernorm.weight"]})
    norms[1].load({"weight": w[p + "post_attention_layernorm.weight"]})
    norms[2].load({"weight": torch.ones(width)})
    x = torch.randn(21, width, generator=g)
    config = dict(rms_norm_eps=eps, num_attention_heads=heads, num_key_value_heads=kv_heads,
                  head_dim=d, rope_theta=theta, hidden_size=width)
    want = plain.plain_decoder_layer(x, torch.arange(21), w, 0, config, dtype)
    h = PartHarness(list(block.parts().values()), [mixer.cache_spec()], dtype)

    def fn(ctx, bindings):
        stream = ResidualStream(x.to(DEV))
        block.forward(stream, ctx, bindings[0])
        norms[2].forward(stream, ctx)                       # folds the last branch in
        return stream.resid.clone()

    got = h.run([("a", 21)], fn)
    assert_close(got, want, dtype, "prenorm block")
