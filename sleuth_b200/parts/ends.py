"""The two ends of the model: token embedding and the output head."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import BuildContext, ParamDecl, Part, build_norm, register_embedding, register_head
from .linear import Linear
from .spec import EmbeddingSpec, HeadSpec


class TokenEmbedding(Part):
    """x[t] = table[ids[t]] * scale into the float32 stream (sleuth/forge/model/transformer.py:345-348)."""

    def __init__(self, spec: EmbeddingSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.table = None

    def declare(self):
        return {"weight": ParamDecl((self.spec.vocab, self.spec.dim))}

    def bind(self, t):
        self.table = t["weight"]

    def forward(self, b, x):
        """``b``: the step's batch; its token ids sit in ``b.token_ids`` (read through ``b.ids_map`` in a step that
        takes its tokens from the device-side feed)."""
        ops.embed(b.token_ids, self.table, x, self.spec.scale, b.stream, b.ids_map)


class LMHead(Part):
    """Final norm on the chosen rows, then logits = h @ W^T in float32
    (sleuth/forge/model/transformer.py:301-302). A tied head uses the embedding table (:129-130)."""

    def __init__(self, spec: HeadSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.norm = build_norm(spec.norm, ctx)
        self.proj = None

    def declare(self):
        d = {"norm.weight": ParamDecl((self.spec.dim,), "vector", init="gain")}
        if not self.spec.tied:
            d["weight"] = ParamDecl((self.spec.vocab, self.spec.dim))
        return d

    def bind(self, t, embedding_table: torch.Tensor | None = None):
        self.norm.bind({"weight": t["norm.weight"]})
        w = embedding_table if self.spec.tied else t["weight"]
        self.proj = Linear(w, self.ctx.dtype)

    def forward(self, x, b, logits, ws):
        """logits[r] = head(x[b.rows[r]]); ``logits`` is float32 [len(b.rows), vocab]."""
        mark = ws.mark()
        h = ws.take((logits.shape[0], self.spec.dim), self.ctx.dtype)
        self.norm.forward(x, h, b.rows, b.stream)
        self.proj.forward(h, out=logits, stream=b.stream)
        ws.release(mark)


register_embedding("token_embedding", TokenEmbedding)
register_head("lm_head", LMHead)
