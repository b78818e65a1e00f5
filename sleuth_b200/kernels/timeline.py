"""Reads the timeline that a library built with ``-DSLB_TIMELINE`` records (``csrc/common.cuh``: one record
per block with the time it entered, up to three marks, and the time it left, in nanoseconds of the GPU's
global timer). The ordinary build records nothing and ``start`` says so.

    SLEUTH_B200_NVCC_FLAGS=-DSLB_TIMELINE SLEUTH_B200_BUILD_DIR=/tmp/slb_timeline python my_script.py

    from sleuth_b200.kernels import timeline
    timeline.start(1 << 20); ...run steps...; records = timeline.read()
"""

from __future__ import annotations

import torch

from . import library

FILES = ("gemm_skinny", "attention_flash", "elementwise", "sampling", "gemm_tc", "attention_tc")
KINDS = {1: "embed", 2: "rmsnorm", 3: "gemm_skinny", 4: "attention_decode", 5: "argmax_partial", 6: "argmax_final",
         7: "sample", 8: "other", 9: "gemm_tc", 10: "attention_tc"}
_buffer = None


def start(records: int = 1 << 20, device="cuda:0") -> None:
    """Give every instrumented file a fresh buffer for ``records`` records."""
    global _buffer
    lib = library.load()
    _buffer = torch.zeros(1 + 6 * records, dtype=torch.int64, device=device)
    for f in FILES:
        try:
            fn = getattr(lib.dll, f"slb_timeline_set_{f}")
        except AttributeError:
            raise RuntimeError("this build of the kernel library records no timeline: build one with "
                               "SLEUTH_B200_NVCC_FLAGS=-DSLB_TIMELINE (and SLEUTH_B200_BUILD_DIR set to a folder of its own)") from None
        fn.argtypes = [library.P, library.ctypes.c_uint]
        fn.restype = library.ctypes.c_int
        if fn(_buffer.data_ptr(), records) != 0:
            raise RuntimeError(f"could not hand the timeline buffer to {f}")


def read() -> list[dict]:
    """The records so far, sorted by the time their block entered: ``kind, block, sm, enter, marks (3), leave``."""
    torch.cuda.synchronize()
    host = _buffer.cpu()
    n = min(int(host[0]) & 0xFFFFFFFF, (host.numel() - 1) // 6)
    out = []
    for r in host[1:1 + 6 * n].view(n, 6).tolist():
        head = r[0] & 0xFFFFFFFFFFFFFFFF
        out.append({"kind": KINDS.get(head & 0xFFFF, "?"), "block": (head >> 16) & 0xFFFFFFFF, "sm": head >> 48,
                    "enter": r[1], "marks": r[2:5], "leave": r[5]})
    out.sort(key=lambda d: d["enter"])
    return out


def clear() -> None:
    _buffer[0] = 0


def launches(records: list[dict]) -> list[dict]:
    """Groups block records into kernel launches (a block number seen again, or a pause, starts a new one) and
    gives for each: kind, blocks, the first and last entry, the first and last time a block got past its wait
    (mark 1), the last mark 2, and the first and last exit."""
    out, open_by_kind = [], {}
    for r in records:
        cur = open_by_kind.get(r["kind"])
        if cur is None or r["block"] in cur["seen"] or r["enter"] > cur["last_leave"] + 20000:
            cur = {"kind": r["kind"], "seen": set(), "records": [], "last_leave": 0}
            open_by_kind[r["kind"]] = cur
            out.append(cur)
        cur["seen"].add(r["block"])
        cur["records"].append(r)
        cur["last_leave"] = max(cur["last_leave"], r["leave"])
    for L in out:
        rs = L["records"]
        go = [r["marks"][0] for r in rs if r["marks"][0]]
        m2 = [r["marks"][1] for r in rs if r["marks"][1]]
        L.update(blocks=len(rs), first_enter=min(r["enter"] for r in rs), last_enter=max(r["enter"] for r in rs),
                 first_go=min(go) if go else 0, last_go=max(go) if go else 0, last_mark2=max(m2) if m2 else 0,
                 first_leave=min(r["leave"] for r in rs))
        del L["seen"]
    out.sort(key=lambda L: L["last_leave"])
    return out


def main(argv=None) -> int:
    """``python -m sleuth_b200.kernels.timeline --config config.json --batch 8``: single-token steps of a model with
    random weights, and where one of them spends its time, launch by launch (needs the -DSLB_TIMELINE build).
    With ``--prompt-step`` the step looked at is the prompts' own (``--batch`` prompts of ``--prompt`` tokens)."""
    import argparse
    import json

    import numpy as np

    from ..engine.engine import Engine
    from ..sampling.config import SamplingConfig
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--config", required=True, help="a config.json (the model gets random weights)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048, help="tokens of each prompt")
    ap.add_argument("--layer", type=int, default=None, help="the layer to print launch by launch (default: the middle one)")
    ap.add_argument("--prompt-step", action="store_true", help="look at the step that brings the prompts")
    args = ap.parse_args(argv)
    cfg = json.load(open(args.config))
    eng = Engine.from_config(cfg, seed=0, dtype="bf16", max_seq_len=args.prompt + 64, max_tokens=args.batch * (args.prompt + 64))
    rng = np.random.default_rng(0)
    V, B = cfg["vocab_size"], args.batch
    greedy = SamplingConfig(temperature=0.0)
    if args.prompt_step:
        return _prompt_step(eng, cfg, args, rng)
    slots = eng.open(B)
    eng.sampler.choose(eng.prefill(slots, [rng.integers(0, V, size=args.prompt).tolist() for _ in range(B)]), greedy)
    for _ in range(6):
        eng.sampler.choose(eng.decode(slots, rng.integers(0, V, size=B).tolist()), greedy)
    start(1 << 18)
    steps = 3
    for _ in range(steps):
        eng.sampler.choose(eng.decode(slots, rng.integers(0, V, size=B).tolist()), greedy)
    all_launches = launches(read())
    step = all_launches[-(len(all_launches) // steps):]
    t0 = step[0]["first_enter"]
    print(f"one step: {len(step)} launches, {(step[-1]['last_leave'] - t0) / 1e3:.1f} us from the first entry to the last exit "
          f"(the marks themselves cost some 5 % of a step)")
    total, prev = {}, t0
    for L in step:
        n, us = total.get(L["kind"], (0, 0.0))
        total[L["kind"]] = (n + 1, us + (L["last_leave"] - prev) / 1e3)
        prev = L["last_leave"]
    for kind, (n, us) in sorted(total.items(), key=lambda kv: -kv[1][1]):
        print(f"  {kind:18s} {n:4d} launches end {us:8.1f} us after the launch before them ended ({us / n:.2f} each)")
    layers = cfg["num_hidden_layers"]
    per_layer = (len(step) - 5) // layers if layers else 0
    if per_layer:
        layer = args.layer if args.layer is not None else layers // 2
        first = 1 + per_layer * layer
        base = prev = step[first - 1]["last_leave"]
        print(f"layer {layer}, times in us after the launch in front of it ended:")
        print("  kind               blocks  enter first..last   past the wait first..last   products done   exit first..last   after the launch in front: go, end")
        for L in step[first:first + per_layer]:
            f = lambda v: f"{(v - base) / 1e3:7.2f}" if v else "      -"
            print(f"  {L['kind']:18s} {L['blocks']:5d}  {f(L['first_enter'])} {f(L['last_enter'])}   {f(L['first_go'])} {f(L['last_go'])}"
                  f"   {f(L['last_mark2'])}   {f(L['first_leave'])} {f(L['last_leave'])}   {(L['last_go'] - prev) / 1e3:6.2f} {(L['last_leave'] - prev) / 1e3:6.2f}")
            prev = L["last_leave"]
    eng.close(slots)
    return 0



def _prompt_step(eng, cfg, args, rng) -> int:
    """The step that brings ``--batch`` prompts of ``--prompt`` tokens, four times (the shape repeats, so the later
    ones are replayed graphs); the last one is printed launch by launch for one layer."""
    V, B = cfg["vocab_size"], args.batch
    prompts = [rng.integers(0, V, size=args.prompt).tolist() for _ in range(B)]
    for _ in range(3):
        slots = eng.open(B)
        eng.prefill(slots, prompts)
        eng.close(slots)
    start(1 << 18)
    slots = eng.open(B)
    eng.prefill(slots, prompts)
    step = launches(read())
    eng.close(slots)
    t0 = step[0]["first_enter"]
    print(f"one prompt step: {len(step)} launches, {(step[-1]['last_leave'] - t0) / 1e3:.1f} us from the first entry to the last exit")
    total, prev = {}, t0
    for L in step:
        n, us = total.get(L["kind"], (0, 0.0))
        total[L["kind"]] = (n + 1, us + (L["last_leave"] - prev) / 1e3)
        prev = L["last_leave"]
    for kind, (n, us) in sorted(total.items(), key=lambda kv: -kv[1][1]):
        print(f"  {kind:18s} {n:4d} launches end {us:8.1f} us after the launch before them ended ({us / n:.2f} each)")
    layers = cfg["num_hidden_layers"]
    per_layer = (len(step) - 3) // layers if layers else 0
    if per_layer:
        layer = args.layer if args.layer is not None else layers // 2
        first = 1 + per_layer * layer
        base = prev = step[first - 1]["last_leave"]
        print(f"layer {layer}, times in us after the launch in front of it ended ({per_layer} launches a layer):")
        print("  kind               blocks  enter first..last   past the wait first..last   loads/scores issued   exit first..last   after the launch in front: go, end")
        for L in step[first:first + per_layer]:
            f = lambda v: f"{(v - base) / 1e3:7.2f}" if v else "      -"
            print(f"  {L['kind']:18s} {L['blocks']:5d}  {f(L['first_enter'])} {f(L['last_enter'])}   {f(L['first_go'])} {f(L['last_go'])}"
                  f"   {f(L['last_mark2'])}   {f(L['first_leave'])} {f(L['last_leave'])}   {(L['last_go'] - prev) / 1e3:6.2f} {(L['last_leave'] - prev) / 1e3:6.2f}")
            prev = L["last_leave"]
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
