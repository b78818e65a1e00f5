"""Where a single-token step spends its time inside the persistent kernel (``csrc/decode_layers.cu``).

    python -m sleuth_b200.kernels.decode_trace --config config.json --batch 8 [--prompt 2048] [--layers N]

builds the model of ``config.json`` with random weights, gives it ``--batch`` prompts of ``--prompt`` tokens, runs a few
single-token steps through the persistent kernel and hands the last one a trace buffer: every block then stamps the
global nanosecond timer at each phase boundary of every layer and counts the clock cycles each phase waited for its
data. Printed: per phase the mean over blocks and layers, and the smallest and largest per-block mean (a phase that
ends in a grid barrier shows the waiting for the slowest block there, not in the phase itself).
"""

from __future__ import annotations

import argparse
import json

PHASES = ["norm 1 + staging", "q/k/v product", "barrier", "attention", "barrier", "staging y", "o-proj", "barrier",
          "norm 2 + staging", "gate/up product", "barrier", "staging act", "down product", "barrier"]
WAITED = ["q/k/v product", "attention", "o-proj", "gate/up product", "down product"]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--config", required=True, help="a config.json (python bench.py --print-config writes the benchmark's)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    a = ap.parse_args(argv)
    import numpy as np
    import torch

    from ..engine import model as model_mod
    from ..engine.engine import Engine
    from . import ops
    cfg = json.load(open(a.config))
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    model_mod.DECODE_CHOICE = "fused"
    ctx = a.prompt + 64
    eng = Engine.from_config(cfg, seed=0, dtype="bf16", max_seq_len=ctx, max_tokens=a.batch * (ctx + 64), use_graphs=False)
    rng = np.random.default_rng(1)
    vocab = eng.vocab
    slots = eng.open(a.batch)
    eng.prefill(slots, [rng.integers(0, vocab, size=a.prompt).tolist() for _ in range(a.batch)])
    if not eng.model._fused_runs(type("B", (), dict(max_count=1, T=a.batch, n=a.batch))(), eng.cache):
        print("this model or batch does not go through the persistent kernel (see Model._fused_runs)")
        return 1
    layers = cfg["num_hidden_layers"]
    blocks = ops.sm_count(eng.device)
    trace = torch.zeros((blocks, layers, 24), dtype=torch.int64, device=eng.device)
    for k in range(6):
        if k == 5:
            eng.model.decode_trace = trace
        eng.decode(slots, rng.integers(0, vocab, size=a.batch).tolist())
    torch.cuda.synchronize()
    eng.model.decode_trace = None
    t = trace.cpu().numpy().astype(np.float64)
    first = 1 if layers > 1 else 0                          # the first layer of the run also starts the pipeline
    d = (t[:, first:, 1:15] - t[:, first:, 0:14]) / 1000.0
    mhz = torch.cuda.clock_rate() if hasattr(torch.cuda, "clock_rate") else 1965
    print(f"batch {a.batch}, {a.prompt} keys, {layers} layers, {blocks} blocks: a layer takes "
          f"{float((t[0, first:, 14] - t[0, first:, 0]).mean() / 1000.0):.1f} us (block 0)")
    print(f"{'phase':18s} {'mean':>7s} {'least':>7s} {'most':>7s}   (us; least and most: per-block means)")
    for i, name in enumerate(PHASES):
        per_block = d[:, :, i].mean(axis=1)
        print(f"{name:18s} {d[:, :, i].mean():7.2f} {per_block.min():7.2f} {per_block.max():7.2f}")
    w = t[:, first:, 15:20] / float(mhz)
    for i, name in enumerate(WAITED):
        print(f"waited for data in {name:16s} {w[:, :, i].mean():6.2f} us (most: {w[:, :, i].mean(axis=1).max():.2f})")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
