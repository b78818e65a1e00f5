"""Each part alone, built from its spec through the registries, against the plain function of the same
formula, at sizes that no tiny configuration uses."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def ctx(dtype=torch.float32, max_positions=256):
    from sleuth_b200.parts import BuildContext
    return BuildContext(device=DEV, dtype=dtype, max_positions=max_positions)


def batch_for(pasts, counts, cache, slots):
    """A StepBatch for sequences that already hold ``pasts`` tokens and bring ``counts`` more."""
    from sleuth_b200.engine.batch import MetaStager
    book = cache.book
    new = [p + c for p, c in zip(pasts, counts)]
    book.grow(slots, new)
    stager = MetaStager(DEV, cache.n_groups, cache.stride)
    T = sum(counts)
    b = stager.upload(slots, pasts, counts, np.zeros(T, dtype=np.int32), np.zeros(0, dtype=np.int32),
                      book.tables_for(slots))
    b.stream = torch.cuda.current_stream().cuda_stream
    book.commit(slots, new)
    return b


def test_norm_part():
    from sleuth_b200.parts import build_norm
    from sleuth_b200.parts.spec import NormSpec
    for dtype in (torch.float32, torch.bfloat16):
        part = build_norm(NormSpec(dim=70, eps=1e-4), ctx(dtype))
        assert list(part.declare()) == ["weight"] and part.declare()["weight"].shape == (70,)
        g = torch.Generator().manual_seed(0)
        x, w = torch.randn(9, 70, generator=g), 1 + 0.2 * torch.randn(70, generator=g)
        part.bind({"weight": w.to(DEV)})
        out = part.forward(x.to(DEV), torch.empty(9, 70, dtype=dtype, device=DEV))
        tl = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out.cpu().float(), plain.rms_norm(x, w, 1e-4), **tl)


def test_position_part_builds_the_reference_tables():
    from sleuth_b200.parts import build_position
    from sleuth_b200.parts.spec import PositionSpec
    c = ctx(max_positions=300)
    part = build_position(PositionSpec(head_dim=24, theta=1e6), c)
    cos, sin = plain.rope_tables(24, 300, 1e6)
    assert torch.equal(part.cos.cpu(), cos[:, :12]) and torch.equal(part.sin.cpu(), sin[:, :12])
    assert build_position(PositionSpec(head_dim=24, theta=1e6), c) is part          # equal specs share one part
    partial = build_position(PositionSpec(head_dim=24, theta=1e4, rotary_dim=8), c)
    assert partial.cos.shape == (300, 4) and partial.rot_dim == 8
    none = build_position(PositionSpec(head_dim=24, kind="none"), c)
    assert none.tables() is None and none.rot_dim == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ffn_part(dtype):
    from sleuth_b200.parts import Workspace, build_ffn
    from sleuth_b200.parts.spec import GatedMLPSpec
    part = build_ffn(GatedMLPSpec(hidden=72, intermediate=200), ctx(dtype))
    assert {k: v.shape for k, v in part.declare().items()} == {"gate.weight": (200, 72), "up.weight": (200, 72),
                                                                "down.weight": (72, 200)}
    g = torch.Generator().manual_seed(1)
    w = {"gate.weight": torch.randn(200, 72, generator=g) * 0.1, "up.weight": torch.randn(200, 72, generator=g) * 0.1,
         "down.weight": torch.randn(72, 200, generator=g) * 0.1}
    if dtype == torch.bfloat16:
        w = {k: v.to(dtype).float() for k, v in w.items()}
    part.bind({k: v.to(DEV).to(dtype) for k, v in w.items()})
    h = torch.randn(11, 72, generator=g).to(dtype)
    x = torch.ones(11, 72, device=DEV)

    class B:
        stream = torch.cuda.current_stream().cuda_stream
    part.forward(h.to(DEV), x, B, Workspace(DEV))
    ref = 1.0 + plain.swiglu(h.float(), {"p.gate_proj.weight": w["gate.weight"], "p.up_proj.weight": w["up.weight"],
                                         "p.down_proj.weight": w["down.weight"]}, "p.")
    tl = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(x.cpu(), ref, **tl)


@pytest.mark.parametrize("dtype,hd", [(torch.float32, 40), (torch.bfloat16, 40), (torch.bfloat16, 64)])
@pytest.mark.parametrize("window,bias", [(0, False), (37, True)])
def test_attention_part(dtype, hd, window, bias):
    """The mixer alone: a prompt step for three sequences, then one token each, against plain attention."""
    from sleuth_b200.cache.paged import PagedCache
    from sleuth_b200.parts import Workspace, build_mixer
    from sleuth_b200.parts.spec import AttentionSpec, PositionSpec
    hidden, heads, kvh, eps, theta = 56, 6, 2, 1e-5, 5e4
    spec = AttentionSpec(hidden=hidden, heads=heads, kv_heads=kvh, head_dim=hd, position=PositionSpec(hd, theta),
                         qk_norm=True, qk_norm_eps=eps, qkv_bias=bias, window=window)
    part = build_mixer(spec, ctx(dtype, 256))
    g = torch.Generator().manual_seed(hd + window)
    w = {}
    for n, d in part.declare().items():
        t = torch.randn(d.shape, generator=g) * (0.15 if d.role == "matrix" else 0.05)
        if d.init == "gain":
            t = 1 + t
        w[n] = t.to(dtype).float() if d.role == "matrix" else t
    part.bind({n: (t.to(DEV).to(dtype) if part.declare()[n].role == "matrix" else t.to(DEV)) for n, t in w.items()})
    cache = PagedCache([part.cache_request()], max_tokens=1024, max_seq_len=256, dtype=dtype, device=DEV)
    lens = [70, 5, 130]
    hs = [torch.randn(n + 1, hidden, generator=g).to(dtype) for n in lens]
    pw = {"p." + k: v for k, v in w.items()}
    s = dict(heads=heads, kv_heads=kvh, head_dim=hd, eps=eps)
    cos, sin = plain.rope_tables(hd, 256, theta)
    refs = [plain.attention(h.float(), pw, "p.", s, window, cos[:len(h)], sin[:len(h)]) for h in hs]
    slots = cache.open(3)
    ws = Workspace(DEV)
    view = cache.view(0, writes=True)
    tl = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    b = batch_for([0, 0, 0], lens, cache, slots)
    x = torch.zeros(sum(lens), hidden, device=DEV)
    part.forward(torch.cat([h[:-1] for h in hs]).to(DEV), x, b, view, ws)
    torch.testing.assert_close(x.cpu(), torch.cat([r[:-1] for r in refs]), **tl)
    b = batch_for(lens, [1, 1, 1], cache, slots)
    x = torch.zeros(3, hidden, device=DEV)
    part.forward(torch.stack([h[-1] for h in hs]).to(DEV), x, b, view, ws)
    torch.testing.assert_close(x.cpu(), torch.stack([r[-1] for r in refs]), **tl)


def test_layer_embedding_and_head_parts():
    from sleuth_b200.cache.paged import PagedCache
    from types import SimpleNamespace

    from sleuth_b200.parts import Workspace, build_embedding, build_head, build_layer
    from sleuth_b200.parts.spec import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, NormSpec,
                                        PositionSpec)
    d, heads, kvh, hd, inter, eps, theta, vocab = 40, 4, 4, 10, 56, 1e-6, 1e4, 61
    c = ctx(torch.float32, 128)
    spec = LayerSpec(mixer=AttentionSpec(hidden=d, heads=heads, kv_heads=kvh, head_dim=hd, position=PositionSpec(hd, theta),
                                         qk_norm=True, qk_norm_eps=eps),
                     ffn=GatedMLPSpec(hidden=d, intermediate=inter), norm1=NormSpec(d, eps), norm2=NormSpec(d, eps))
    layer = build_layer(spec, c)
    g = torch.Generator().manual_seed(5)
    local = {n: (1 + 0.1 * torch.randn(dd.shape, generator=g)) if dd.init == "gain" else torch.randn(dd.shape, generator=g) * 0.2
             for n, dd in layer.declare().items()}
    layer.bind({n: t.to(DEV) for n, t in local.items()})
    rename = {"norm1.weight": "input_layernorm.weight", "norm2.weight": "post_attention_layernorm.weight"}
    pw = {}
    for n, t in local.items():
        if n in rename:
            pw["model.layers.0." + rename[n]] = t
        elif n.startswith("mixer."):
            pw["model.layers.0.self_attn." + n[6:]] = t
        else:
            pw["model.layers.0.mlp." + n[4:].replace(".weight", "_proj.weight")] = t
    cache = PagedCache([layer.cache_request()], max_tokens=256, max_seq_len=128, dtype=torch.float32, device=DEV)
    (slot,) = cache.open(1)
    x0 = torch.randn(33, d, generator=g)
    x = x0.clone().to(DEV)
    layer.forward(x, batch_for([0], [33], cache, [slot]), cache.view(0, True), Workspace(DEV))
    s = dict(d=d, heads=heads, kv_heads=kvh, head_dim=hd, eps=eps, windows=[0])
    cos, sin = plain.rope_tables(hd, 33, theta)
    torch.testing.assert_close(x.cpu(), plain.block(x0, pw, 0, s, cos, sin), rtol=1e-4, atol=1e-5)

    stream = torch.cuda.current_stream().cuda_stream
    emb = build_embedding(EmbeddingSpec(vocab=vocab, dim=d, scale=2.0), c)       # by kind, as the model builds it
    table = torch.randn(vocab, d, generator=g)
    emb.bind({"weight": table.to(DEV)})
    ids = torch.tensor([0, 60, 7, 7], dtype=torch.int32)
    out = torch.empty(4, d, device=DEV)
    emb.forward(SimpleNamespace(token_ids=ids.to(DEV), ids_map=None, stream=stream), out)
    torch.testing.assert_close(out.cpu(), table[ids.long()] * 2.0)
    back = torch.tensor([3, 3, 0, 1], dtype=torch.int32)                          # through a device-side index map
    emb.forward(SimpleNamespace(token_ids=ids.to(DEV), ids_map=back.to(DEV), stream=stream), out)
    torch.testing.assert_close(out.cpu(), table[ids[back.long()].long()] * 2.0)

    for tied in (True, False):
        head = build_head(HeadSpec(vocab=vocab, dim=d, norm=NormSpec(d, eps), tied=tied), c)
        assert ("weight" in head.declare()) == (not tied)
        gain, wout = 1 + 0.1 * torch.randn(d, generator=g), torch.randn(vocab, d, generator=g)
        head.bind({"norm.weight": gain.to(DEV), **({} if tied else {"weight": wout.to(DEV)})}, embedding_table=table.to(DEV))
        rows = torch.tensor([32, 0, 5], dtype=torch.int32, device=DEV)
        logits = torch.empty(3, vocab, device=DEV)
        head.forward(x, SimpleNamespace(rows=rows, stream=stream), logits, Workspace(DEV))
        ref = plain.rms_norm(x.cpu()[[32, 0, 5]], gain, eps) @ (table if tied else wout).T
        torch.testing.assert_close(logits.cpu(), ref, rtol=1e-4, atol=1e-4)
