"""The tcgen05/TMA matrix product against a float64 product of the same bfloat16 inputs: full tiles, ragged
edges in every dimension, every epilogue."""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run(M, N, K, mode, seed=0):
    from sleuth_b200.kernels import ops as o
    g = torch.Generator().manual_seed(seed + M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    rows = 2 * N if mode == "swiglu" else N
    w = (torch.randn(rows, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    if mode == "swiglu":
        a, b = x.double() @ w[:N].double().T, x.double() @ w[N:].double().T
        ref = a * torch.sigmoid(a) * b
    else:
        ref = x.double() @ w.double().T
    dt = torch.float32 if mode in ("f32", "add") else torch.bfloat16
    base = torch.randn(M, N, generator=g) if mode == "add" else torch.full((M, N), float("nan"))
    out = base.to(dt).to(DEV)
    o.gemm_tc(x.to(DEV), w.to(DEV), out, mode)
    o.gemm_tc_check(DEV)
    if mode == "add":
        ref = ref + base.double()
    tl = dict(rtol=1.5e-2, atol=1.5e-2) if dt == torch.bfloat16 else dict(rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(out.cpu().double(), ref, **tl)


def test_one_tile_first():
    run(128, 128, 64, "f32")


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 256, 64), (256, 512, 128), (129, 200, 72), (77, 136, 96),
                                   (17, 503, 160), (300, 1024, 3072), (2048, 4096, 1024), (1000, 2000, 1000)])
@pytest.mark.parametrize("mode", ["f32", "bf16", "add"])
def test_gemm_tc(M, N, K, mode):
    run(M, N, K, mode)


@pytest.mark.parametrize("M,N,K,mode", [(4100, 300, 136, "f32"), (4096, 512, 64, "bf16"), (4500, 1024, 200, "add"),
                                         (4200, 136, 96, "swiglu"), (5000, 520, 72, "swiglu")])
def test_gemm_tc_many_rows_take_pairs_of_blocks(M, N, K, mode):
    """From 4,096 rows on two blocks of a cluster share tiles of 256 rows (cta_group::2): each loads its rows of X and
    half of the tile's rows of W; row counts that end inside the upper or the lower half of the last tile."""
    run(M, N, K, mode)


@pytest.mark.parametrize("M,inter,K", [(128, 128, 64), (256, 3072, 1024), (77, 136, 96), (2048, 200, 72)])
def test_gemm_tc_gated_activation(M, inter, K):
    run(M, inter, K, "swiglu")


def test_refusals():
    from sleuth_b200.kernels import ops as o
    assert not o.tc_supported(64, 64, 20)
    x = torch.zeros(32, 20, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        o.gemm_tc(x, torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV), torch.zeros(32, 8, dtype=torch.bfloat16, device=DEV), "bf16")


@pytest.mark.parametrize("M,N,K,mode", [(64, 4096, 1024, "bf16"), (64, 1024, 3072, "add"), (40, 3072, 1024, "swiglu"),
                                         (17, 1024, 2048, "add"), (100, 151936, 64, "f32"), (33, 96, 64, "swiglu")])
def test_gemm_tc_few_rows_take_narrow_tiles(M, N, K, mode):
    run(M, N, K, mode)


@pytest.mark.parametrize("heads,kv_heads,hd,bias,norm,rot", [(4, 2, 128, False, True, True), (3, 1, 128, True, True, True),
                                                              (5, 2, 64, True, False, True), (16, 8, 128, False, True, False),
                                                              (2, 0, 128, False, True, True)])
def test_gemm_tc_with_qkv_post_in_the_epilogue(heads, kv_heads, hd, bias, norm, rot):
    """The fused q/k/v projection: product, bias, per-head RMSNorm, rotation, and the stores of q and of k/v into
    scrambled cache pages, against the same steps in float64. kv_heads = 0: a layer that reads another layer's cache."""
    import numpy as np
    from sleuth_b200.kernels import ops as o
    g = torch.Generator().manual_seed(heads * hd + kv_heads)
    pasts, counts = [0, 100, 63], [150, 2, 70]
    lens = [p + c for p, c in zip(pasts, counts)]
    T, K = sum(counts), 96
    rows = heads + 2 * kv_heads
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(rows * hd, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = (torch.randn(rows * hd, generator=g) * 0.1) if bias else None
    qg = (1 + 0.1 * torch.randn(hd, generator=g)) if norm else None
    kg = (1 + 0.1 * torch.randn(hd, generator=g)) if norm else None
    eps = 1e-5
    inv = 1.0 / (1e4 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(256, dtype=torch.float32), inv)
    cos, sin = (ang.cos().contiguous(), ang.sin().contiguous()) if rot else (None, None)
    stride = max((l + 63) // 64 for l in lens)
    n_pages = sum((l + 63) // 64 for l in lens)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), stride), -1, dtype=torch.int32)
    for i, l in enumerate(lens):
        for pg in range((l + 63) // 64):
            table[i, pg] = perm.pop()
    tok_seq = np.repeat(np.arange(3), counts).astype(np.int32)
    tok_pos = np.concatenate([np.arange(p, p + c) for p, c in zip(pasts, counts)]).astype(np.int32)
    d = lambda a: None if a is None else torch.as_tensor(a).to(DEV)
    q_out = torch.full((T, heads, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    k_pool = torch.zeros(n_pages, max(kv_heads, 1), 64, hd, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    o.gemm_tc_qkv(d(x), d(w), heads, kv_heads, hd, d(b), d(qg), d(kg), d(cos), d(sin), eps, q_out,
                  k_pool if kv_heads else None, v_pool if kv_heads else None, d(tok_seq), d(tok_pos), d(table))
    o.gemm_tc_check(DEV)
    y = (x.double() @ w.double().T).view(T, rows, hd)
    if bias:
        y = y + b.double().view(rows, hd)

    def normed(v, gain):
        return v if gain is None else v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * gain.double()

    def rope(v):
        if not rot:
            return v
        c, s = cos[tok_pos].double()[:, None, :], sin[tok_pos].double()[:, None, :]
        a, bb = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([a * c - bb * s, bb * c + a * s], dim=-1)

    tl = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q_out.cpu().double(), rope(normed(y[:, :heads], qg)), **tl)
    if kv_heads:
        k_ref, v_ref = rope(normed(y[:, heads:heads + kv_heads], kg)), y[:, heads + kv_heads:]
        kp, vp = k_pool.cpu().double(), v_pool.cpu().double()
        for t in range(T):
            page = int(table[tok_seq[t], tok_pos[t] // 64])
            torch.testing.assert_close(kp[page, :, tok_pos[t] % 64], k_ref[t], **tl)
            torch.testing.assert_close(vp[page, :, tok_pos[t] % 64], v_ref[t], **tl)
