"""Position encodings of queries and keys.

``rotary``: rotate-half pairs (i, i + rot/2) by the angle position * theta^(-2i/rot). The cos and
sin tables ``[positions, rot/2]`` are built once, on the host, in float32, with the reference's own
order of operations (sleuth/forge/model/rope.py:30-38: ``1 / theta ** (arange(0, rot, 2) / rot)``,
``outer(positions, inv_freq)``), so the angles are the reference's to the bit. The kernels that
apply them live in ``csrc/qkv_post.cu``. ``none``: no tables, nothing is rotated.
"""

from __future__ import annotations

import torch

from .base import BuildContext, Part, register_position
from .spec import PositionSpec


class Rotary(Part):
    def __init__(self, spec: PositionSpec, ctx: BuildContext):
        self.rot_dim = spec.rotary_dim or spec.head_dim
        if self.rot_dim % 2 or self.rot_dim > spec.head_dim:
            raise ValueError(f"rotary_dim {self.rot_dim} must be even and at most head_dim {spec.head_dim}")
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim))
        pos = torch.arange(ctx.max_positions, dtype=torch.float32)
        ang = torch.outer(pos, inv_freq)                       # [positions, rot/2], float32
        self.cos = ang.cos().contiguous().to(ctx.device)
        self.sin = ang.sin().contiguous().to(ctx.device)

    def tables(self):
        return self.cos, self.sin


class NoPosition(Part):
    rot_dim = 0

    def __init__(self, spec, ctx: BuildContext):
        pass

    def tables(self):
        return None


register_position("rotary", Rotary)
register_position("none", NoPosition)
