"""Times of the two tcgen05 prompt-attention kernels over step shapes, and which one the library would take.

    python -m sleuth_b200.kernels.prompt_attention_times [--heads 16 --kv-heads 8 --head-dim 128]

Each shape (sequences x new tokens after a number of cached tokens) runs ten times inside a CUDA graph, five replays,
timed with CUDA events: the kernel that walks one page a step (two blocks an SM), the one that walks two (one block
an SM, four threads a row), and the library's own choice (``csrc/attention_tc.cu``: ``wide_pays``).
"""

from __future__ import annotations

import argparse

SHAPES = [([256], 0), ([512], 0), ([1024], 0), ([1536], 0), ([2048], 0), ([3072], 0), ([4096], 0), ([8192], 0),
          ([2048] * 8, 0), ([300] * 16, 0), ([100] * 64, 0), ([512] * 4, 0), ([256], 4096), ([512], 8192), ([1024] * 2, 1024)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    a = ap.parse_args(argv)
    import numpy as np
    import torch

    from . import ops
    dev, bf = "cuda:0", torch.bfloat16
    H, K, hd = a.heads, a.kv_heads, a.head_dim
    scale = hd ** -0.5

    def run(lens, past, wide):
        n, T = len(lens), sum(lens)
        pages_each = [(past + L + 63) // 64 for L in lens]
        pages = sum(pages_each)
        kp = torch.randn(pages, K, 64, hd, device=dev).to(bf)
        vp = torch.randn(pages, K, 64, hd, device=dev).to(bf)
        q = torch.randn(T, H, hd, device=dev).to(bf)
        out = torch.empty(T, H * hd, dtype=bf, device=dev)
        table = torch.full((n, max(pages_each)), -1, dtype=torch.int32)
        at = 0
        for i, pe in enumerate(pages_each):
            table[i, :pe] = torch.arange(at, at + pe, dtype=torch.int32)
            at += pe
        table = table.to(dev)
        starts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
        pasts = torch.full((n,), past, dtype=torch.int32, device=dev)
        counts = torch.tensor(lens, dtype=torch.int32, device=dev)

        def call():
            ops.attention_tc(q, kp, vp, out, starts, pasts, counts, table, max(lens), H, K, hd, 0, scale, wide=wide,
                             max_keys=past + max(lens))
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(10):
                    call()
            graph.replay()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(5):
                graph.replay()
            t1.record(stream)
            torch.cuda.synchronize()
        ops.gemm_tc_check(dev)
        return t0.elapsed_time(t1) / 50 * 1000

    print(f"{H} heads, {K} kv heads, head size {hd}; microseconds a call")
    print("sequences x tokens (after cached) | one page a step | two pages a step | the library's choice")
    for lens, past in SHAPES:
        one, two, chosen = run(lens, past, False), run(lens, past, True), run(lens, past, None)
        print(f"{len(lens):3d} x {lens[0]:5d} ({past:5d}) | {one:8.1f} | {two:8.1f} | {chosen:8.1f}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
