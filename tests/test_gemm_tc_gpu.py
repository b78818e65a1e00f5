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
