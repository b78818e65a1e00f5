"""Normalisation parts. ``rmsnorm``: y = x * rsqrt(mean(x^2) + eps) * gain, float32 arithmetic on the
float32 stream, output in the run dtype (sleuth/forge/model/norm.py:34-50)."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import BuildContext, ParamDecl, Part, register_norm
from .spec import NormSpec


class RMSNorm(Part):
    fusable = True      # a product kernel may apply this norm itself from ``weight`` and ``eps``

    def __init__(self, spec: NormSpec, ctx: BuildContext):
        self.dim, self.eps, self.dtype = spec.dim, spec.eps, ctx.dtype
        self.weight = None

    def declare(self):
        return {"weight": ParamDecl((self.dim,), "vector", init="gain")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def fused_decode(self):
        return {"gain": self.weight, "eps": self.eps} if self.weight is not None else None

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None, stream=None):
        """out[r] = norm(x[rows[r]]) (or x[r] without ``rows``); ``out`` has the run dtype."""
        ops.rmsnorm(x, self.weight, out, self.eps, rows, stream)
        return out


register_norm("rmsnorm", RMSNorm)
