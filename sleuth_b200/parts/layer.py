"""Arrangements of a mixer, a feed-forward and their norms in one layer.

``prenorm``: x += mixer(norm1(x)); x += ffn(norm2(x)) (sleuth/forge/model/transformer.py:78,87-88,96,99).
The layer owns the residual arrangement only; the parts it is given decide everything else. The sum
itself is a float32 accumulation into the stream, done by the last product of the mixer or ffn.
"""

from __future__ import annotations

from .base import BuildContext, Normed, Part, build_ffn, build_mixer, build_norm, lead_weight_of, register_layer
from .spec import LayerSpec


class PreNormLayer(Part):
    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.ctx = ctx
        self.norm1 = build_norm(spec.norm1, ctx)
        self.mixer = build_mixer(spec.mixer, ctx)
        self.norm2 = build_norm(spec.norm2, ctx)
        self.ffn = build_ffn(spec.ffn, ctx)
        self.children = {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "ffn": self.ffn}
        self.capturable = all(getattr(p, "capturable", True) for p in self.children.values())

    def declare(self):
        out = {}
        for prefix, part in self.children.items():
            for name, decl in part.declare().items():
                out[f"{prefix}.{name}"] = decl
        return out

    def bind(self, tensors):
        for prefix, part in self.children.items():
            part.bind({k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")})

    def cache_request(self):
        return self.mixer.cache_request()

    def lead_weight(self):
        return lead_weight_of(self.mixer)

    def fused_decode(self):
        """x += mixer(norm1(x)); x += ffn(norm2(x)) is what the persistent single-token kernel runs: offered when all
        four parts offer their share."""
        shares = {name: getattr(part, "fused_decode", lambda: None)() for name, part in self.children.items()}
        if any(v is None for v in shares.values()):
            return None
        if "w_qkv" not in shares["mixer"] or "w_gu" not in shares["ffn"] or "gain" not in shares["norm1"] or "gain" not in shares["norm2"]:
            return None
        return shares

    def forward(self, x, b, view, ws):
        mark = ws.mark()
        after = getattr(b, "next_read", None)    # what follows this layer
        b.next_read = lead_weight_of(self.ffn)
        self.mixer.forward(self._input(self.norm1, self.mixer, x, b, ws), x, b, view, ws)
        ws.release(mark)
        b.next_read = after
        self.ffn.forward(self._input(self.norm2, self.ffn, x, b, ws), x, b, ws)
        ws.release(mark)

    def _input(self, norm, part, x, b, ws):
        """What ``part`` reads: the normalised tensor, or, for a part that can normalise inside its first
        product, a ``Normed`` that runs the norm kernel only if asked for the tensor."""
        n = Normed(norm, x, ws, b.stream, self.ctx.dtype)
        return n if part.accepts_normed else n.tensor()


register_layer("prenorm", PreNormLayer)
