"""Putting a checkpoint's tensors into a model's parts, by name.

The model says which tensors it expects (name -> shape and role); the checkpoint says which it
holds (name -> dtype and shape, from the headers alone). Any disagreement is reported before a
byte of tensor data is read, in ONE error that lists the missing tensors, the unexpected ones and
the ones of the wrong shape. (The reference raises on the first unknown name, the first wrong shape,
and then on missing ones: sleuth/formats/hf.py:289-300.)

Dtypes on the device follow the role (see ``parts/base.py``): matrices in the run dtype, gains and
biases in float32, integer tables in int32. bfloat16 and float16 widen exactly; a 32-bit matrix is
narrowed only by the bfloat16 run, which cannot hold it otherwise.
"""

from __future__ import annotations

import re

import torch

from ..parts.base import ParamDecl
from .safetensors import Checkpoint


class WeightError(ValueError):
    """The checkpoint does not fit the model. ``missing``, ``unexpected`` and ``wrong_shape`` hold the details."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, have, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(have)} in the file, the model needs {list(want)}")
        for name, have in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {have} in the file, which is not a weight dtype")
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def check(expected: dict[str, ParamDecl], ckpt: Checkpoint, ignored=()) -> None:
    have = set(ckpt.names())
    patterns = [re.compile(p) for p in ignored]
    missing = sorted(n for n, d in expected.items() if n not in have and not d.optional)
    unexpected = sorted(n for n in have if n not in expected and not any(p.fullmatch(n) for p in patterns))
    wrong_shape, wrong_dtype = [], []
    for n, d in expected.items():
        if n in have:
            dtype, shape = ckpt.describe(n)
            if tuple(shape) != tuple(d.shape):
                wrong_shape.append((n, shape, d.shape))
            if (d.role == "table" and dtype not in _INTS) or (d.role != "table" and dtype not in _FLOATS):
                wrong_dtype.append((n, str(dtype).replace("torch.", "")))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)


def to_device(t: torch.Tensor, role: str, run_dtype: torch.dtype, device) -> torch.Tensor:
    if role == "table":
        return t.to(device=device, dtype=torch.int32)
    if role == "vector":
        return t.to(device=device, dtype=torch.float32)
    if t.dtype == run_dtype:
        return t.to(device=device).contiguous()
    # widen or narrow on the device: the host copy stays in the stored dtype
    return t.to(device=device).to(run_dtype).contiguous()


def load_into(expected: dict[str, ParamDecl], ckpt: Checkpoint, run_dtype: torch.dtype, device, ignored=()):
    """Check, then read every expected tensor onto the device. Returns ``{name: tensor}``."""
    check(expected, ckpt, ignored)
    out = {}
    for n, d in expected.items():
        if n in ckpt.where:
            out[n] = to_device(ckpt.tensor(n), d.role, run_dtype, device)
    return out
