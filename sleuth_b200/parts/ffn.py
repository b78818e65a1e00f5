"""Feed-forward parts. ``gated_mlp``: down(act(gate(h)) * up(h)) without biases
(sleuth/forge/model/mlp.py:25-41). Gate and up matrices are stacked at load time into one
``[2 * intermediate, hidden]`` matrix, so one product feeds the activation kernel."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import BuildContext, Normed, ParamDecl, Part, register_ffn
from . import linear
from .linear import Linear
from .spec import GatedMLPSpec


# Measured on a B200 at batch 1 and 8: the norm kernel plus the plain product take less time than the product
# with the norm fused in for this shape (1.101 against 1.233 ms a step at batch 8, 0.845 against 0.895 ms at
# batch 1): each of the 384 blocks would normalise all rows again before its first product, and nothing hides that
# in front of so short a block.
FUSE_NORM = False


class GatedMLP(Part):
    accepts_normed = True

    def __init__(self, spec: GatedMLPSpec, ctx: BuildContext):
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation {spec.activation!r} is not supported (silu)")
        self.spec, self.ctx = spec, ctx
        self.gate_up = self.down = None

    def declare(self):
        s = self.spec
        return {"gate.weight": ParamDecl((s.intermediate, s.hidden)), "up.weight": ParamDecl((s.intermediate, s.hidden)),
                "down.weight": ParamDecl((s.hidden, s.intermediate))}

    def bind(self, t):
        self.gate_up = Linear(torch.cat([t["gate.weight"], t["up.weight"]], dim=0), self.ctx.dtype)
        self.down = Linear(t["down.weight"], self.ctx.dtype)

    def lead_weight(self):
        return self.gate_up.weight if self.gate_up is not None else None

    def fused_decode(self):
        if self.ctx.dtype != torch.bfloat16 or self.gate_up is None or self.spec.intermediate % 32 or self.spec.hidden % 128:
            return None
        return {"w_gu": self.gate_up.weight, "w_down": self.down.weight, "inter": self.spec.intermediate}

    def forward(self, h, x, b, ws):
        T = h.shape[0]
        mark = ws.mark()
        act = ws.take((T, self.spec.intermediate), self.ctx.dtype)
        if self.ctx.dtype == torch.bfloat16 and linear.use_skinny(T, self.spec.intermediate, self.spec.hidden):
            # norm in the product's prologue (when handed the stream), activation in its epilogue
            if (isinstance(h, Normed) and h.gain is not None and FUSE_NORM
                    and ops.skinny_supported(T, self.spec.intermediate, self.spec.hidden, norm=True)):
                ops.gemm_skinny_norm(h.x, h.gain, h.eps, self.gate_up.weight, act, "swiglu", b.stream, self.down.weight)
            else:
                hh = h.tensor() if isinstance(h, Normed) else h
                f = linear.tuned_features("swiglu", T, self.spec.intermediate, self.spec.hidden,
                                          lambda f: ops.gemm_skinny(hh, self.gate_up.weight, act, "swiglu", b.stream, features=f))
                ops.gemm_skinny(hh, self.gate_up.weight, act, "swiglu", b.stream, self.down.weight, features=f)
        elif self.ctx.dtype == torch.bfloat16 and linear.use_tc(T, self.spec.intermediate, self.spec.hidden):
            ops.gemm_tc(h.tensor() if isinstance(h, Normed) else h, self.gate_up.weight, act, "swiglu", b.stream)
        else:
            gu = self.gate_up.forward(h, ws=ws, stream=b.stream)
            ops.swiglu(gu, act, b.stream)
        self.down.forward(act, into=x, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None))
        ws.release(mark)


register_ffn("gated_mlp", GatedMLP)
