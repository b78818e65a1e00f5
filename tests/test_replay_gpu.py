"""bin/trace_run as a user runs it: a subprocess fed JSON steps, writing <step>.f32 files."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import tiny
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(folder, dtype, steps, out, max_tokens):
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                             "--out", str(out), "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for msg in steps:
        proc.stdin.write(json.dumps(msg) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {msg['step']}", line          # the next step is sent only after this one is done
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_trace_run_schedules(name, dtype, model_folders, tmp_path):
    cfg, w = plain.read_model(model_folders[name])
    V = cfg["vocab_size"]
    rng = np.random.default_rng(7)
    reqs = {r: rng.integers(0, V, size=n).tolist() for r, n in (("a", 90), ("b", 33), ("c", 5), ("d", 64))}
    ref = {r: plain.logits(cfg, w, ids, round_weights_to_bf16=(dtype == "bfloat16")) for r, ids in reqs.items()}
    steps, expect = [], {}
    # a and b and c start together with unequal prompts, then go on one token each; c ends first, then b
    cut = {"a": 50, "b": 30, "c": 3}
    steps.append({"step": 0, "entries": [{"id": r, "tokens": reqs[r][:cut[r]], "want": [cut[r] - 1] + ([0] if r == "a" else [])}
                                         for r in "abc"], "end": []})
    expect[0] = [("a", 49), ("a", 0), ("b", 29), ("c", 2)]
    k, live = 1, ["a", "b", "c"]
    while live:
        entries, wanted, ended = [], [], []
        for r in live:
            pos = cut[r] + k - 1
            want = [0] if (pos % 2 == 0 or pos == len(reqs[r]) - 1) else []
            entries.append({"id": r, "tokens": [reqs[r][pos]], "want": want})
            wanted += [(r, pos)] * len(want)
            if pos == len(reqs[r]) - 1:
                ended.append(r)
        steps.append({"step": k, "entries": entries, "end": ended})
        if wanted:
            expect[k] = wanted
        live = [r for r in live if r not in ended]
        k += 1
        if k == 12:          # a new request takes freed room while a is still running? no: a batch takes no newcomers
            pass
    # after the batch has ended, d runs whole in the room that was given back
    steps.append({"step": k, "entries": [{"id": "d", "tokens": reqs["d"], "want": list(range(64))}], "end": ["d"]})
    expect[k] = [("d", i) for i in range(64)]
    # the most tokens live at once: a, b and c grown to their ends, each rounded up to 64
    out = tmp_path / "out"
    replay(model_folders[name], dtype, steps, out, max_tokens=128 + 64 + 64)
    # the bounds of tests/test_engine_gpu.py: bfloat16 at twice the largest difference a B200 showed there
    tol = dict(rtol=1e-4, atol=2e-5) if dtype == "float32" else dict(rtol=0.0, atol=1.7e-2)
    for step, rows in expect.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), V)
        want = torch.stack([ref[r][p] for r, p in rows])
        torch.testing.assert_close(torch.from_numpy(got), want, **tol)
    assert not (out / "1.f32").exists() or 1 in expect
    produced = {int(p.name[:-4]) for p in out.iterdir()}
    assert produced == set(expect)


def test_trace_run_refuses_more_tokens_than_it_was_sized_for(model_folders, tmp_path):
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": list(range(70)), "want": []}], "end": []}]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folders["A"], "--dtype",
                           "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                          input=json.dumps(steps[0]) + "\n", capture_output=True, text=True, timeout=120)
    assert proc.returncode != 0 and "64" in proc.stderr
