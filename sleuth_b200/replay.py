"""Trace replay: feed given token ids through a model step by step and write the logits.

It samples nothing and owns nothing: the model, the step function, the cache and the kernels are
the ones generation uses (``Engine``). Steps arrive on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives each request's next tokens and the places among them whose logits are wanted;
a request seen for the first time takes a slot, ``end`` lists the requests whose slot and pages go
back after the step. A step with wanted places writes ``<out>/<step>.f32``: float32 little-endian
``[wanted, vocab]`` in the order of the entries and of ``want``. After every step ``done <step>`` is
printed and flushed. The reference has no such program; its closest relatives are the schedule tests
tests/test_model.py:61-69 and tests/test_generate.py:15-25.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description="replay token traces through a model and write logits")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    p.add_argument("--device", default="cuda:0")
    return p


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    import numpy as np
    import torch

    from .config.base import read_config_json
    from .engine.engine import Engine
    from .kernels import ops
    from .engine.stepper import StepEntry

    if a.max_tokens <= 0:
        print("--max-tokens must be positive", file=sys.stderr)
        return 2
    max_pos = int(read_config_json(a.model).get("max_position_embeddings", a.max_tokens))
    max_tokens = -(-a.max_tokens // 64) * 64
    engine = Engine.from_pretrained(a.model, dtype=a.dtype, max_seq_len=min(max_tokens, max_pos),
                                    max_tokens=max_tokens, device=a.device)
    slot_of: dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step = msg["step"]
        entries = []
        fresh = [str(e["id"]) for e in msg.get("entries", []) if str(e["id"]) not in slot_of]
        if fresh:
            for rid, s in zip(fresh, engine.open(len(fresh))):
                slot_of[rid] = s
        for e in msg.get("entries", []):
            entries.append(StepEntry(slot_of[str(e["id"])], e["tokens"], tuple(e.get("want", ()))))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                host = logits.to("cpu", torch.float32).contiguous().numpy()
                with open(out / f"{step}.f32", "wb") as f:
                    f.write(host.astype("<f4", copy=False).tobytes())
            else:
                torch.cuda.synchronize()
            ops.gemm_tc_check(engine.device)     # the step is complete: did a tensor-memory kernel give up a wait?
        ended = [str(r) for r in msg.get("end", [])]
        if ended:
            engine.close([slot_of.pop(r) for r in ended if r in slot_of])
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
