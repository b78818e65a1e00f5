"""Comparison of engine results with the plain implementation that also remembers the largest difference seen.

``check`` is ``torch.testing.assert_close`` plus a record: per label the largest absolute difference and the
largest magnitude of the expected values. At the end of a session the records are printed (``pytest -s`` or the
terminal summary) and, when ``SLEUTH_B200_ERRORS_FILE`` names a file, written there as JSON, so that the
tolerances in the tests can be set from what a B200 actually shows instead of from a guess."""

from __future__ import annotations

import json
import os

import torch

OBSERVED: dict[str, dict] = {}


def check(got: torch.Tensor, want: torch.Tensor, tol: dict, label: str) -> None:
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    rec = OBSERVED.setdefault(label, {"max_abs_diff": 0.0, "max_abs_value": 0.0, "comparisons": 0})
    if got.shape == want.shape and got.numel():
        rec["max_abs_diff"] = max(rec["max_abs_diff"], float((got - want).abs().max()))
        rec["max_abs_value"] = max(rec["max_abs_value"], float(want.abs().max()))
    rec["comparisons"] += 1
    torch.testing.assert_close(got, want, **tol)


def report(write=print) -> None:
    if not OBSERVED:
        return
    write("largest differences from the plain implementation (label: difference / largest expected value):")
    for label in sorted(OBSERVED):
        r = OBSERVED[label]
        write(f"  {label}: {r['max_abs_diff']:.3g} / {r['max_abs_value']:.3g}  ({r['comparisons']} comparisons)")
    path = os.environ.get("SLEUTH_B200_ERRORS_FILE")
    if path:
        with open(path, "w") as f:
            json.dump(OBSERVED, f, indent=1, sort_keys=True)
