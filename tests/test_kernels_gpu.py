"""Each CUDA kernel alone against a plain float64 computation of the same formula, at sizes other than
the engine's: odd widths, head sizes 16..256, groups of 1..8 heads, windows, pages in scrambled order."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from sleuth_b200.kernels import ops as o
    return o


def tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------ row-wise kernels ----

@pytest.mark.parametrize("dim", [64, 96, 1000, 1024, 2050])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(dim, dtype):
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(7, dim, generator=g) * 3
    w = 1 + 0.1 * torch.randn(dim, generator=g)
    eps = 1e-5
    ref = (x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * w.double())
    out = torch.empty(7, dim, dtype=dtype, device=DEV)
    ops().rmsnorm(x.to(DEV), w.to(DEV), out, eps)
    torch.testing.assert_close(out.cpu().double(), ref, **tol(dtype))
    # chosen rows only
    rows = torch.tensor([5, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, dim, dtype=dtype, device=DEV)
    ops().rmsnorm(x.to(DEV), w.to(DEV), out2, eps, rows)
    torch.testing.assert_close(out2.cpu().double(), ref[[5, 0, 3]], **tol(dtype))


@pytest.mark.parametrize("dim", [1024, 1000, 2048, 4100])
def test_rmsnorm_many_rows(dim):
    """Prompts bring a thousand rows and more; the bfloat16 run then takes another block shape."""
    g = torch.Generator().manual_seed(dim + 1)
    n = 1100
    x = torch.randn(n, dim, generator=g) * 3
    w = 1 + 0.1 * torch.randn(dim, generator=g)
    eps = 1e-6
    ref = (x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * w.double())
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((n, dim), float("nan"), dtype=dtype, device=DEV)
        ops().rmsnorm(x.to(DEV), w.to(DEV), out, eps)
        torch.testing.assert_close(out.cpu().double(), ref, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_add_swiglu(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(37, 50, generator=g).to(dtype)
    ids = torch.tensor([3, 36, 0, 3, 17], dtype=torch.int32)
    x = torch.empty(5, 50, dtype=torch.float32, device=DEV)
    ops().embed(ids.to(DEV), table.to(DEV), x, 1.5)
    torch.testing.assert_close(x.cpu(), table[ids.long()].float() * 1.5)
    delta = torch.randn(5, 50, generator=g).to(dtype)
    ops().add(x, delta.to(DEV))
    torch.testing.assert_close(x.cpu(), table[ids.long()].float() * 1.5 + delta.float())
    gu = torch.randn(6, 2 * 77, generator=g).to(dtype)
    act = torch.empty(6, 77, dtype=dtype, device=DEV)
    ops().swiglu(gu.to(DEV), act)
    gd, ud = gu[:, :77].double(), gu[:, 77:].double()
    torch.testing.assert_close(act.cpu().double(), gd * torch.sigmoid(gd) * ud, **tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 33, 17), (5, 64, 96), (16, 503, 160), (17, 100, 1000), (130, 257, 75), (96, 40, 36),
                                   (300, 1024, 1024), (257, 130, 1030)])
def test_gemm_f32_exact_and_row_independent(M, N, K):
    g = torch.Generator().manual_seed(M * N)
    a, w, bias = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g)
    out = torch.empty(M, N, device=DEV)
    ops().gemm_f32(a.to(DEV), w.to(DEV), out, bias.to(DEV))
    ref = a.double() @ w.double().T + bias.double()
    torch.testing.assert_close(out.cpu().double(), ref, rtol=1e-5, atol=1e-4)
    # a row computed alone equals the same row computed in the batch, bit for bit
    one = torch.empty(1, N, device=DEV)
    ops().gemm_f32(a[M - 1:M].contiguous().to(DEV), w.to(DEV), one, bias.to(DEV))
    assert torch.equal(one.cpu()[0], out.cpu()[M - 1])
    # accumulate adds to what is there
    acc = torch.full((M, N), 2.0, device=DEV)
    ops().gemm_f32(a.to(DEV), w.to(DEV), acc, None, accumulate=True)
    torch.testing.assert_close(acc.cpu().double(), a.double() @ w.double().T + 2.0, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("M,N,K,mode", [(1, 96, 256, "bf16"), (8, 2560, 1024, "add"), (16, 1000, 2560, "f32"), (5, 520, 384, "swiglu")])
def test_gemm_skinny_features_per_block_change_no_bit(M, N, K, mode):
    """How many output features a block takes (the launcher's rule, or 8, 16, 32 as the engine measures and chooses per
    shape) decides which block computes which feature, never the order of a sum: every choice gives the same bits."""
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn((2 * N if mode == "swiglu" else N), K, generator=g) / 8).bfloat16().to(DEV)
    base = torch.randn(M, N, generator=g).to(DEV)
    outs = []
    for f in (0, 8, 16) + (() if mode == "swiglu" else (32,)):
        out = base.clone() if mode == "add" else torch.empty(M, N, device=DEV, dtype=torch.float32 if mode == "f32" else torch.bfloat16)
        ops().gemm_skinny(x, w, out, mode, features=f)
        outs.append(out.cpu())
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    if mode != "swiglu":
        ref = x.float().cpu() @ w.float().cpu().T + (base.cpu() if mode == "add" else 0)
        torch.testing.assert_close(outs[0].float(), ref, rtol=2e-2, atol=2e-2)


# ------------------------------------------------------------------ cache layout helpers ----

def make_cache(seq_lens, kv_heads, hd, dtype, gen, scramble=True):
    """Random keys/values for sequences of the given lengths, laid out in pages in scrambled order.
    Returns (k_pool, v_pool, table [n, stride], dense keys, dense values) with dense [n][len, K, hd]."""
    n = len(seq_lens)
    stride = max(1, max((l + 63) // 64 for l in seq_lens))
    total = sum((l + 63) // 64 for l in seq_lens) + 3
    order = torch.randperm(total, generator=gen).tolist() if scramble else list(range(total))
    k_pool = torch.full((total, kv_heads, 64, hd), float("nan")).to(dtype)
    v_pool = torch.full((total, kv_heads, 64, hd), float("nan")).to(dtype)
    table = torch.full((n, stride), -1, dtype=torch.int32)
    ks, vs = [], []
    for i, l in enumerate(seq_lens):
        k = torch.randn(l, kv_heads, hd, generator=gen).to(dtype)
        v = torch.randn(l, kv_heads, hd, generator=gen).to(dtype)
        ks.append(k)
        vs.append(v)
        for pg in range((l + 63) // 64):
            page = order.pop()
            table[i, pg] = page
            a, b = pg * 64, min(l, pg * 64 + 64)
            k_pool[page, :, :b - a] = k[a:b].transpose(0, 1)
            v_pool[page, :, :b - a] = v[a:b].transpose(0, 1)
    return k_pool, v_pool, table, ks, vs


def plain_attention(q, k, v, pos, window, scale):
    """q [T, H, hd] at positions pos[t]; k, v [L, K, hd] of the same sequence; float64."""
    T, H, hd = q.shape
    K = k.shape[1]
    out = torch.zeros(T, H, hd, dtype=torch.float64)
    for t in range(T):
        lo = max(0, pos[t] - window + 1) if window else 0
        for h in range(H):
            kk = k[lo:pos[t] + 1, h // (H // K)].double()
            vv = v[lo:pos[t] + 1, h // (H // K)].double()
            s = (kk @ q[t, h].double()) * scale
            out[t, h] = torch.softmax(s, 0) @ vv
    return out


def run_attention(kind, dtype, heads, kv_heads, hd, pasts, counts, window, seed, next_read=None):
    o = ops()
    gen = torch.Generator().manual_seed(seed)
    lens = [p + c for p, c in zip(pasts, counts)]
    k_pool, v_pool, table, ks, vs = make_cache(lens, kv_heads, hd, dtype, gen)
    T = sum(counts)
    q = torch.randn(T, heads, hd, generator=gen).to(dtype)
    # make one far key decisive for some query: scale a key and the matching query channel up
    scale = 1.0 / math.sqrt(hd)
    tok_seq = np.repeat(np.arange(len(counts)), counts).astype(np.int32)
    starts = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    tok_pos = np.concatenate([np.arange(p, p + c) for p, c in zip(pasts, counts)]).astype(np.int32)
    ref = torch.cat([plain_attention(q[starts[i]:starts[i + 1]].float(), ks[i].float(), vs[i].float(),
                                     tok_pos[starts[i]:starts[i + 1]], window, scale) for i in range(len(counts))])
    d = lambda a: torch.as_tensor(a).to(DEV)
    out = torch.full((T, heads * hd), float("nan")).to(dtype).to(DEV)
    if kind == "generic":
        o.attention(d(q), d(k_pool), d(v_pool), out, d(tok_seq), d(tok_pos), d(table), heads, kv_heads, hd, window, scale)
    elif kind == "prefill":
        o.attention_prefill(d(q), d(k_pool), d(v_pool), out, d(starts), d(np.asarray(pasts, dtype=np.int32)),
                            d(np.asarray(counts, dtype=np.int32)), d(table), max(counts), heads, kv_heads, hd, window, scale)
    elif kind in ("tc", "tc one page a step", "tc two pages a step"):
        o.attention_tc(d(q), d(k_pool), d(v_pool), out, d(starts), d(np.asarray(pasts, dtype=np.int32)),
                       d(np.asarray(counts, dtype=np.int32)), d(table), max(counts), heads, kv_heads, hd, window, scale,
                       wide=None if kind == "tc" else kind == "tc two pages a step")
        o.gemm_tc_check(DEV)
    else:
        splits = kind
        floats = o.decode_scratch_floats(len(counts), heads, hd, splits)
        scratch = torch.full((max(floats, 1),), float("nan"), device=DEV)
        o.attention_decode(d(q), d(k_pool), d(v_pool), out, d(starts), d(np.asarray(pasts, dtype=np.int32)), d(table),
                           heads, kv_heads, hd, window, scale, splits, scratch if floats else None, next_read=next_read)
    got = out.cpu().double().view(T, heads, hd)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, ref, **(dict(rtol=2e-2, atol=1.5e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 16), (6, 3, 24), (5, 1, 64), (8, 8, 40), (2, 1, 256), (16, 2, 128)])
def test_attention_generic(dtype, heads, kv_heads, hd):
    run_attention("generic", dtype, heads, kv_heads, hd, pasts=[0, 70, 0, 129], counts=[5, 1, 67, 3], window=0, seed=hd)
    run_attention("generic", dtype, heads, kv_heads, hd, pasts=[0, 100], counts=[90, 2], window=33, seed=hd + 1)


@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 128), (5, 1, 64), (8, 8, 64), (16, 2, 128), (6, 2, 128), (32, 1, 64)])
def test_attention_prefill_tensor_cores(heads, kv_heads, hd):
    bf = torch.bfloat16
    run_attention("prefill", bf, heads, kv_heads, hd, pasts=[0, 0, 0], counts=[1, 64, 200], window=0, seed=1)
    run_attention("prefill", bf, heads, kv_heads, hd, pasts=[70, 0, 129, 5], counts=[33, 5, 1, 130], window=0, seed=2)
    run_attention("prefill", bf, heads, kv_heads, hd, pasts=[0, 150], counts=[170, 40], window=50, seed=3)
    run_attention("prefill", bf, heads, kv_heads, hd, pasts=[300], counts=[7], window=64, seed=4)


@pytest.mark.parametrize("kind", ["tc one page a step", "tc two pages a step"])
@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 128), (4, 1, 64), (8, 8, 64), (16, 2, 128), (2, 2, 128), (32, 1, 64)])
def test_attention_tcgen05(heads, kv_heads, hd, kind):
    """Both tcgen05 kernels on the cases of the mma.sync kernel (pools are NaN outside the sequences), and on
    longer prompts that cross many pages and tiles, with even and odd numbers of pages, windows that end inside a
    step's first or second page, and sequences that end in either."""
    bf = torch.bfloat16
    run_attention(kind, bf, heads, kv_heads, hd, pasts=[0, 0, 0], counts=[1, 64, 200], window=0, seed=1)
    run_attention(kind, bf, heads, kv_heads, hd, pasts=[70, 0, 129, 5], counts=[33, 5, 1, 130], window=0, seed=2)
    run_attention(kind, bf, heads, kv_heads, hd, pasts=[0, 150], counts=[170, 40], window=50, seed=3)
    run_attention(kind, bf, heads, kv_heads, hd, pasts=[300], counts=[7], window=64, seed=4)
    run_attention(kind, bf, heads, kv_heads, hd, pasts=[0, 37], counts=[700, 450], window=0, seed=5)
    run_attention(kind, bf, heads, kv_heads, hd, pasts=[64, 0, 500], counts=[321, 128, 90], window=200, seed=6)


def test_attention_tcgen05_chooses_by_shape():
    """Left to itself the library takes the two-page kernel where one round of blocks holds the step or the longest
    tile outweighs an SM's share of all pages, the one-page kernel where many short tiles fill the GPU."""
    bf = torch.bfloat16
    run_attention("tc", bf, 4, 2, 128, pasts=[0, 10], counts=[511, 60], window=0, seed=7)          # few blocks
    run_attention("tc", bf, 16, 8, 128, pasts=[0] * 12, counts=[200] * 12, window=0, seed=8)       # many short tiles


def test_attention_tcgen05_choice_follows_the_measurements():
    """The shapes at which the two kernels were timed on a B200 (16 query heads, 8 kv heads), and which of them won."""
    o = ops()
    two = lambda n, count, past=0: o.attention_tc_takes_two_pages(n, count, past + count, 16, 8)
    assert two(1, 256) and two(1, 512) and two(1, 1024) and two(1, 1536) and two(1, 2048)        # one round of blocks, or long tiles
    assert not two(1, 3072) and not two(1, 4096) and not two(1, 8192)                              # several rounds
    assert not two(8, 2048) and not two(16, 300) and not two(64, 100) and not two(4, 512)          # many tiles
    assert two(1, 256, past=4096) and two(1, 512, past=8192)                                       # a chunk after a long past
    assert not two(2, 1024, past=1024)


def test_attention_tcgen05_growing_scores():
    """Scores that grow along the sequence force the running maximum up page after page, so the accumulator in
    tensor memory is rescaled many times; scores that shrink never rescale it. Both must agree with the reference."""
    o = ops()
    bf = torch.bfloat16
    H, K, hd, L = 4, 2, 128, 600
    for direction in (1.0, -1.0):
        gen = torch.Generator().manual_seed(11)
        k_pool, v_pool, table, ks, vs = make_cache([L], K, hd, bf, gen)
        q = torch.randn(L, H, hd, generator=gen).to(bf)
        # key t gets an extra component along a fixed direction, growing (or shrinking) with t; every query has that component
        ramp = (torch.arange(L, dtype=torch.float32) / L * 12.0 * direction)
        for t in range(L):
            page, row = int(table[0, t // 64]), t % 64
            k_pool[page, :, row, 0] = ramp[t].to(bf)
            ks[0][t, :, 0] = ramp[t].to(bf)
        q[:, :, 0] = 8.0
        d = lambda a: torch.as_tensor(a).to(DEV)
        i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device=DEV)
        ref = plain_attention(q.double(), ks[0].double(), vs[0].double(), list(range(L)), 0, 1.0)
        for wide in (False, True):
            out = torch.empty(L, H * hd, dtype=bf, device=DEV)
            o.attention_tc(d(q), d(k_pool), d(v_pool), out, i32(0, L), i32(0), i32(L), d(table), L, H, K, hd, 0, 1.0, wide=wide)
            o.gemm_tc_check(DEV)
            got = out.cpu().double().view(L, H, hd)
            assert torch.isfinite(got).all()
            torch.testing.assert_close(got, ref, rtol=2e-2, atol=1.5e-2)


@pytest.mark.parametrize("splits", [1, 2, 5, 32])
@pytest.mark.parametrize("heads,kv_heads,hd", [(4, 2, 128), (5, 1, 64), (8, 8, 64), (16, 2, 128), (40, 2, 64)])
def test_attention_decode_tensor_cores(splits, heads, kv_heads, hd):
    bf = torch.bfloat16
    run_attention(splits, bf, heads, kv_heads, hd, pasts=[0, 63, 64, 300, 1000], counts=[1] * 5, window=0, seed=5)
    run_attention(splits, bf, heads, kv_heads, hd, pasts=[10, 200, 700], counts=[1] * 3, window=100, seed=6)


def test_attention_decode_with_two_page_buffers():
    """Between two and three blocks per SM the launcher takes the form with two page buffers (three blocks fit an SM
    then): twenty sequences of eight kv heads in two slices are 320 blocks."""
    bf = torch.bfloat16
    pasts = [0, 63, 64, 300, 1000, 129, 700, 5, 450, 999] * 2
    run_attention(2, bf, 16, 8, 128, pasts=pasts, counts=[1] * 20, window=0, seed=12)
    run_attention(2, bf, 16, 8, 128, pasts=pasts, counts=[1] * 20, window=200, seed=13)
    run_attention(1, bf, 8, 8, 64, pasts=pasts * 2, counts=[1] * 40, window=0, seed=14)       # 320 blocks of one slice


def test_attention_far_key_decides():
    """One key far back gets a score that dominates: a kernel that drops or misplaces it fails loudly."""
    o = ops()
    for dtype, kind in ((torch.float32, "generic"), (torch.bfloat16, "decode"), (torch.bfloat16, "prefill")):
        gen = torch.Generator().manual_seed(9)
        H, K, hd, L = 4, 2, 128, 700
        k_pool, v_pool, table, ks, vs = make_cache([L], K, hd, dtype, gen)
        far = 37
        page, row = int(table[0, far // 64]), far % 64
        q = torch.randn(1, H, hd, generator=gen).to(dtype)
        k_pool[page, :, row] = (q[0, ::2] * 4).to(dtype)            # key 37 of each kv head lines up with its first query head
        v_pool[page, :, row] = 7.0
        d = lambda a: torch.as_tensor(a).to(DEV)
        out = torch.empty(1, H * hd, dtype=dtype, device=DEV)
        i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device=DEV)
        if kind == "generic":
            o.attention(d(q), d(k_pool), d(v_pool), out, i32(0), i32(L - 1), d(table), H, K, hd, 0, 1.0)
        elif kind == "decode":
            scratch = torch.empty(o.decode_scratch_floats(1, H, hd, 4), device=DEV)
            o.attention_decode(d(q), d(k_pool), d(v_pool), out, i32(0, 1), i32(L - 1), d(table), H, K, hd, 0, 1.0, 4, scratch)
        else:
            # two tokens so that the prefill kernel is the one that fits; look at the last one
            q2 = torch.cat([q, q]).contiguous()
            out2 = torch.empty(2, H * hd, dtype=dtype, device=DEV)
            o.attention_prefill(d(q2), d(k_pool), d(v_pool), out2, i32(0, 2), i32(L - 2), i32(2), d(table), 2, H, K, hd, 0, 1.0)
            out = out2[1:]
        got = out.cpu().float().view(H, hd)
        assert (got[0] - 7.0).abs().max() < 0.05 and (got[2] - 7.0).abs().max() < 0.05


# ------------------------------------------------------------------ qkv_post ----

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,hd,rot", [(4, 2, 16, 16), (6, 3, 24, 24), (5, 1, 64, 32), (2, 2, 128, 128), (3, 1, 256, 0)])
def test_qkv_post(dtype, heads, kv_heads, hd, rot):
    o = ops()
    gen = torch.Generator().manual_seed(hd + heads)
    pasts, counts = [0, 100, 63], [3, 2, 70]
    lens = [p + c for p, c in zip(pasts, counts)]
    T = sum(counts)
    rows = heads + 2 * kv_heads
    qkv = torch.randn(T, rows * hd, generator=gen).to(dtype)
    bias = torch.randn(rows * hd, generator=gen) * 0.1
    qg, kg = 1 + 0.1 * torch.randn(hd, generator=gen), 1 + 0.1 * torch.randn(hd, generator=gen)
    eps, theta, maxpos = 1e-5, 1e4, 256
    cos = sin = None
    if rot:
        inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
        ang = torch.outer(torch.arange(maxpos, dtype=torch.float32), inv)
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    stride = max((l + 63) // 64 for l in lens)
    n_pages = sum((l + 63) // 64 for l in lens)
    perm = torch.randperm(n_pages, generator=gen).tolist()
    table = torch.full((len(lens), stride), -1, dtype=torch.int32)
    for i, l in enumerate(lens):
        for pg in range((l + 63) // 64):
            table[i, pg] = perm.pop()
    tok_seq = np.repeat(np.arange(3), counts).astype(np.int32)
    tok_pos = np.concatenate([np.arange(p, p + c) for p, c in zip(pasts, counts)]).astype(np.int32)
    d = lambda a: None if a is None else torch.as_tensor(a).to(DEV)
    q_out = torch.empty(T, heads, hd, dtype=dtype, device=DEV)
    k_pool = torch.zeros(n_pages, kv_heads, 64, hd, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    o.qkv_post(d(qkv), d(bias), d(qg), d(kg), d(cos), d(sin), q_out, k_pool, v_pool, d(tok_seq), d(tok_pos), d(table),
               heads, kv_heads, hd, rot, eps)
    x = qkv.double().view(T, rows, hd) + bias.double().view(rows, hd)

    def norm(v, gain):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * gain.double()

    def rope(v):
        if not rot:
            return v
        c, s = cos[tok_pos].double()[:, None, :], sin[tok_pos].double()[:, None, :]
        a, b = v[..., :rot // 2], v[..., rot // 2:rot]
        return torch.cat([a * c - b * s, b * c + a * s, v[..., rot:]], dim=-1)

    q_ref = rope(norm(x[:, :heads], qg))
    k_ref = rope(norm(x[:, heads:heads + kv_heads], kg))
    v_ref = x[:, heads + kv_heads:]
    tl = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(q_out.cpu().double(), q_ref, **tl)
    kp, vp = k_pool.cpu().double(), v_pool.cpu().double()
    for t in range(T):
        page = int(table[tok_seq[t], tok_pos[t] // 64])
        torch.testing.assert_close(kp[page, :, tok_pos[t] % 64], k_ref[t], **tl)
        torch.testing.assert_close(vp[page, :, tok_pos[t] % 64], v_ref[t], **tl)


# ------------------------------------------------------------------ few-rows product ----

@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 32, 40, 64])
@pytest.mark.parametrize("N,K", [(1024, 1024), (1000, 2048), (4096, 1024), (40, 96), (33000, 64), (1024, 3072)])
def test_gemm_skinny(M, N, K):
    o = ops()
    assert o.skinny_supported(M, N, K)
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    for mode, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        out = torch.full((M, N), float("nan"), dtype=dt, device=DEV)
        o.gemm_skinny(x.to(DEV), w.to(DEV), out, mode)
        torch.testing.assert_close(out.cpu().double(), ref, rtol=1e-2 if dt == torch.bfloat16 else 1e-4,
                                   atol=1e-2 if dt == torch.bfloat16 else 1e-4)
    base = torch.randn(M, N, generator=g)
    acc = base.clone().to(DEV)
    o.gemm_skinny(x.to(DEV), w.to(DEV), acc, "add")
    torch.testing.assert_close(acc.cpu().double(), base.double() + ref, rtol=1e-4, atol=1e-4)
    # twice the same call gives the same bits (the warps' partial sums are added in a fixed order)
    again = base.clone().to(DEV)
    o.gemm_skinny(x.to(DEV), w.to(DEV), again, "add")
    assert torch.equal(acc, again)


@pytest.mark.parametrize("M,inter,K", [(1, 3072, 1024), (8, 200, 64), (16, 4100, 128), (5, 136, 96), (24, 3072, 1024), (64, 200, 64)])
def test_gemm_skinny_gated_activation(M, inter, K):
    o = ops()
    g = torch.Generator().manual_seed(inter)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=g) / math.sqrt(K) * 2).to(torch.bfloat16)
    gate, up = x.double() @ w[:inter].double().T, x.double() @ w[inter:].double().T
    act = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.gemm_skinny(x.to(DEV), w.to(DEV), act, "swiglu")
    torch.testing.assert_close(act.cpu().double(), gate * torch.sigmoid(gate) * up, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("next_elems", [8, 72000, 4 << 20, 1001])
def test_kernels_told_what_is_read_next_compute_the_same(next_elems):
    """A kernel that is handed the next kernel's weights asks the cache for them and nothing else: its own result is
    the same bits, whatever the size of the range (a few bytes, no multiple of a cache line, megabytes) and for a
    range that is not 16-byte aligned (which is not passed on)."""
    o = ops()
    g = torch.Generator().manual_seed(next_elems)
    nxt = torch.randn(next_elems + 1, generator=g).to(torch.bfloat16).to(DEV)
    nxt = nxt[1:] if next_elems == 1001 else nxt[:next_elems]
    keep = nxt.clone()
    for M, N, K in ((3, 40, 96), (8, 4096, 1024)):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
        plain = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        told = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        o.gemm_skinny(x, w, plain, "bf16")
        o.gemm_skinny(x, w, told, "bf16", next_read=nxt)
        assert torch.equal(plain, told)
        gain = torch.ones(K, device=DEV)
        o.gemm_skinny_norm(x.float(), gain, 1e-6, w, plain, "bf16")
        o.gemm_skinny_norm(x.float(), gain, 1e-6, w, told, "bf16", next_read=nxt)
        assert torch.equal(plain, told)
    # the same for the cache pages of an attention kernel that follows: sequences of 1, 64 and 700 keys, with and
    # without a window, more slices than pages, a table with unused entries
    kv_heads, hd = 2, 64
    lens = [1, 64, 700]
    pool = torch.randn(16, kv_heads, 64, hd, generator=g).to(torch.bfloat16).to(DEV)
    vpool = pool.clone()
    table = torch.full((3, 12), 15, dtype=torch.int32)
    table[0, 0], table[1, :2], table[2, :11] = 0, torch.tensor([1, 2]), torch.arange(3, 14)
    past = torch.tensor([n - 1 for n in lens], dtype=torch.int32).to(DEV)
    for splits, window in ((1, 0), (5, 0), (16, 100)):
        pages = o.next_pages(pool, vpool, table.to(DEV), past, splits, window)
        o.gemm_skinny(x, w, told, "bf16", next_pages=pages)
        o.gemm_skinny(x, w, plain, "bf16")
        assert torch.equal(plain, told)
    torch.cuda.synchronize()
    assert torch.equal(pool, vpool)
    run_attention(3, torch.bfloat16, 4, 2, 64, pasts=[5, 300, 64], counts=[1] * 3, window=0, seed=3, next_read=nxt)
    run_attention(1, torch.bfloat16, 16, 8, 128, pasts=[700], counts=[1], window=0, seed=4, next_read=nxt)
    torch.cuda.synchronize()
    assert torch.equal(nxt, keep)


def test_gemm_skinny_refuses_what_it_cannot_run():
    o = ops()
    assert not o.skinny_supported(65, 64, 64) and not o.skinny_supported(4, 64, 40)
    x = torch.zeros(4, 40, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of 32"):
        o.gemm_skinny(x, torch.zeros(8, 40, dtype=torch.bfloat16, device=DEV), torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV), "bf16")


@pytest.mark.parametrize("rows,vocab,limit", [(1, 503, 503), (5, 151936, 151936), (64, 1000, 777), (3, 70, 64)])
def test_argmax_first_index_on_ties(rows, vocab, limit):
    o = ops()
    g = torch.Generator().manual_seed(rows)
    logits = torch.randn(rows, vocab, generator=g)
    logits[0, limit // 3] = 50.0
    logits[0, limit - 1] = 50.0                      # a tie: the lower index wins
    if rows > 1:
        logits[1, limit:] = 99.0                     # beyond the limit: never chosen
        logits[1, 5] = logits[1, :limit].max()       # ties with a later maximum
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    scratch = torch.empty(o.argmax_scratch_words(rows), dtype=torch.int32, device=DEV)
    o.argmax(logits.to(DEV), limit, out, scratch)
    want = [int(torch.nonzero(r[:limit] == r[:limit].max())[0]) for r in logits]
    assert out.cpu().tolist() == want


@pytest.mark.parametrize("M,N,K,mode", [(1, 4096, 1024, "bf16"), (8, 1024, 2048, "f32"), (16, 200, 96, "bf16"),
                                         (5, 3072, 1024, "swiglu"), (3, 136, 64, "swiglu")])
def test_gemm_skinny_with_the_norm_fused_in(M, N, K, mode):
    """The product that normalises its input rows itself equals norm then product: the rows are normalised in
    float32 and rounded to bfloat16 once, as the norm kernel does."""
    o = ops()
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(M, K, generator=g) * 2
    gain = 1 + 0.2 * torch.randn(K, generator=g)
    eps = 1e-5
    rows = 2 * N if mode == "swiglu" else N
    w = (torch.randn(rows, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    inv = torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float()
    hb = ((x * inv) * gain).to(torch.bfloat16).double()
    if mode == "swiglu":
        a, b = hb @ w[:N].double().T, hb @ w[N:].double().T
        ref = a * torch.sigmoid(a) * b
    else:
        ref = hb @ w.double().T
    dt = torch.float32 if mode == "f32" else torch.bfloat16
    out = torch.full((M, N), float("nan"), dtype=dt, device=DEV)
    o.gemm_skinny_norm(x.to(DEV), gain.to(DEV), eps, w.to(DEV), out, mode)
    tl = dict(rtol=2e-2, atol=2e-2) if dt == torch.bfloat16 else dict(rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(out.cpu().double(), ref, **tl)


@pytest.mark.parametrize("heads,kv_heads,hd,splits,bias,rot", [(4, 2, 128, 1, False, True), (16, 8, 128, 5, False, True),
                                                                 (5, 1, 64, 3, True, True), (40, 2, 64, 2, True, False)])
def test_attention_decode_with_qkv_post_fused(heads, kv_heads, hd, splits, bias, rot):
    """The decode kernel given the raw projection of the new token: it must normalise, rotate, append to the
    cache and attend exactly as qkv_post followed by attention do."""
    o = ops()
    bf = torch.bfloat16
    gen = torch.Generator().manual_seed(heads * hd + splits)
    pasts = [0, 63, 64, 300, 1000]
    n = len(pasts)
    lens = [p + 1 for p in pasts]
    k_pool, v_pool, table, ks, vs = make_cache(lens, kv_heads, hd, bf, gen)
    rows = heads + 2 * kv_heads
    qkv = torch.randn(n, rows * hd, generator=gen).to(bf)
    b = (torch.randn(rows * hd, generator=gen) * 0.1) if bias else None
    qg, kg = 1 + 0.1 * torch.randn(hd, generator=gen), 1 + 0.1 * torch.randn(hd, generator=gen)
    eps, theta = 1e-5, 1e4
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(1100, dtype=torch.float32), inv)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    x = qkv.double().view(n, rows, hd) + (b.double().view(rows, hd) if bias else 0)

    def norm(v, gain):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * gain.double()

    def rope(v):
        if not rot:
            return v
        c, s = cos[pasts].double()[:, None, :], sin[pasts].double()[:, None, :]
        a, bb = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([a * c - bb * s, bb * c + a * s], dim=-1)

    q_ref = rope(norm(x[:, :heads], qg))
    k_new = rope(norm(x[:, heads:heads + kv_heads], kg)).to(bf)           # what the cache will hold
    v_new = x[:, heads + kv_heads:].to(bf)
    scale = 1.0 / math.sqrt(hd)
    ref = []
    for i in range(n):
        kk = torch.cat([ks[i][:pasts[i]].float(), k_new[i:i + 1].float()])
        vv = torch.cat([vs[i][:pasts[i]].float(), v_new[i:i + 1].float()])
        ref.append(plain_attention(q_ref[i:i + 1].to(bf).float(), kk, vv, [pasts[i]], 0, scale))
    ref = torch.cat(ref)
    d = lambda a: None if a is None else torch.as_tensor(a).to(DEV)
    kp, vp = d(k_pool), d(v_pool)                 # the newest row of every sequence is still random rubbish here
    out = torch.full((n, heads * hd), float("nan")).to(bf).to(DEV)
    floats = o.decode_scratch_floats(n, heads, hd, splits)
    scratch = torch.full((max(floats, 1),), float("nan"), device=DEV)
    starts = np.arange(n + 1, dtype=np.int32)
    o.attention_decode(None, kp, vp, out, d(starts), d(np.asarray(pasts, dtype=np.int32)), d(table), heads, kv_heads, hd,
                       0, scale, splits, scratch if floats else None, qkv=d(qkv), qkv_kv_heads=kv_heads, bias=d(b),
                       q_gain=d(qg), k_gain=d(kg), cos=d(cos) if rot else None, sin=d(sin) if rot else None, eps=eps)
    torch.testing.assert_close(out.cpu().double().view(n, heads, hd), ref, rtol=2e-2, atol=1.5e-2)
    for i in range(n):
        page = int(table[i, pasts[i] // 64])
        torch.testing.assert_close(kp[page, :, pasts[i] % 64].cpu().float(), k_new[i].float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(vp[page, :, pasts[i] % 64].cpu().float(), v_new[i].float(), rtol=2e-2, atol=2e-2)
