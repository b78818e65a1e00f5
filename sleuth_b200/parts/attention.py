"""Causal grouped-query attention over the paged cache, as a mixer part.

One fused q/k/v projection (the three matrices are stacked at load time into one
``[(H + 2K) * head_dim, hidden]`` matrix), then bias, per-head RMSNorm of q and k, rotation and the
cache write in one kernel, then attention over the cache, then the output projection added into
the residual stream. Formulas and their order: sleuth/forge/model/attention.py:101-157 (projections
:106-108, QK-norm before RoPE :121-126, cache update :129-130, scale 1/sqrt(head_dim) :84, GQA
head mapping :197-199, window mask :160-169, output projection without bias :155-157).

With ``reads_shared_kv`` the part has no k/v projections and reads the cache entry another layer
application wrote.
"""

from __future__ import annotations

import math
import os

import torch

from ..cache.paged import KVRequest
from ..kernels import ops
from .base import BuildContext, ParamDecl, Part, build_position, register_mixer
from .base import Normed
from .linear import Linear, use_tc
from .spec import AttentionSpec


# Which kernel serves a step that brings several tokens per sequence: "auto" takes the tcgen05 kernel once a
# sequence fills at least one of its 128-row tiles, "mma" always the mma.sync kernel, "tc" the tcgen05 kernel
# whenever it takes the shape.
ATTENTION_CHOICE = os.environ.get("SLEUTH_B200_ATTENTION", "auto")


def use_tc_attention(heads: int, kv_heads: int, head_dim: int, dtype, max_count: int, scale: float = 1.0) -> bool:
    if ATTENTION_CHOICE == "mma" or scale <= 0 or not ops.attention_tc_supported(heads, kv_heads, head_dim, dtype):
        return False
    return ATTENTION_CHOICE == "tc" or max_count * (heads // kv_heads) >= 128


class GQAAttention(Part):
    accepts_normed = True

    def __init__(self, spec: AttentionSpec, ctx: BuildContext):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads ({spec.heads}) must be a multiple of kv_heads ({spec.kv_heads})")
        if spec.head_dim % 2 or spec.head_dim > 256:
            raise ValueError(f"head_dim {spec.head_dim} is not supported: it must be even and at most 256")
        self.spec = spec
        self.ctx = ctx
        self.position = build_position(spec.position, ctx)
        self.scale = spec.scale or 1.0 / math.sqrt(spec.head_dim)
        self.qkv = self.o = None
        self.bias = self.q_gain = self.k_gain = None

    # ---- weights ----
    def declare(self):
        s = self.spec
        d = {"q_proj.weight": ParamDecl((s.heads * s.head_dim, s.hidden)),
             "o_proj.weight": ParamDecl((s.hidden, s.heads * s.head_dim))}
        if not s.reads_shared_kv:
            d["k_proj.weight"] = ParamDecl((s.kv_heads * s.head_dim, s.hidden))
            d["v_proj.weight"] = ParamDecl((s.kv_heads * s.head_dim, s.hidden))
        if s.qkv_bias:
            d["q_proj.bias"] = ParamDecl((s.heads * s.head_dim,), "vector")
            if not s.reads_shared_kv:
                d["k_proj.bias"] = ParamDecl((s.kv_heads * s.head_dim,), "vector")
                d["v_proj.bias"] = ParamDecl((s.kv_heads * s.head_dim,), "vector")
        if s.qk_norm:
            d["q_norm.weight"] = ParamDecl((s.head_dim,), "vector", init="gain")
            if not s.reads_shared_kv:
                d["k_norm.weight"] = ParamDecl((s.head_dim,), "vector", init="gain")
        return d

    def bind(self, t):
        s = self.spec
        names = ["q_proj"] if s.reads_shared_kv else ["q_proj", "k_proj", "v_proj"]
        self.qkv = Linear(torch.cat([t[n + ".weight"] for n in names], dim=0), self.ctx.dtype)
        self.o = Linear(t["o_proj.weight"], self.ctx.dtype)
        if s.qkv_bias:
            self.bias = torch.cat([t[n + ".bias"] for n in names]).contiguous()
        if s.qk_norm:
            self.q_gain = t["q_norm.weight"]
            self.k_gain = t["q_norm.weight"] if s.reads_shared_kv else t["k_norm.weight"]

    def cache_request(self):
        s = self.spec
        return KVRequest(s.kv_heads, s.head_dim, s.window)

    # ---- one step ----
    def _attend(self, q, y, b, view, table, ws):
        """Attention of the step's (post-processed) queries over the cache into ``y``; the kernel by dtype and step shape."""
        s = self.spec
        flash = ops.flash_supported(s.head_dim, self.ctx.dtype)
        if not flash:
            ops.attention(q, view.k_pool, view.v_pool, y, b.tok_seq, b.tok_pos, table, s.heads, s.kv_heads,
                          s.head_dim, view.window, self.scale, b.stream)
        elif b.max_count == 1:
            splits = ops.decode_splits(b.n, s.kv_heads, s.heads // s.kv_heads, table.shape[1])
            floats = ops.decode_scratch_floats(b.n, s.heads, s.head_dim, splits)
            scratch = ws.take((floats,), torch.float32) if floats else None
            ops.attention_decode(q, view.k_pool, view.v_pool, y, b.seq_start, b.past, table, s.heads, s.kv_heads,
                                 s.head_dim, view.window, self.scale, splits, scratch, b.stream)
        elif use_tc_attention(s.heads, s.kv_heads, s.head_dim, self.ctx.dtype, b.max_count, self.scale):
            ops.attention_tc(q, view.k_pool, view.v_pool, y, b.seq_start, b.past, b.counts, table, b.max_count,
                             s.heads, s.kv_heads, s.head_dim, view.window, self.scale, b.stream, max_keys=b.max_len)
        else:
            ops.attention_prefill(q, view.k_pool, view.v_pool, y, b.seq_start, b.past, b.counts, table, b.max_count,
                                  s.heads, s.kv_heads, s.head_dim, view.window, self.scale, b.stream)

    def lead_weight(self):
        return self.qkv.weight if self.qkv is not None else None

    def fused_decode(self):
        s = self.spec
        rot = self.position.rot_dim
        if (self.ctx.dtype != torch.bfloat16 or self.qkv is None or s.reads_shared_kv or s.head_dim not in (64, 128)
                or rot not in (0, s.head_dim) or s.heads // s.kv_heads > 8 or s.hidden % 128
                or (s.qk_norm and (self.q_gain is None or self.k_gain is None))):
            return None
        tables = self.position.tables() if rot else None
        return {"w_qkv": self.qkv.weight, "w_o": self.o.weight, "bias": self.bias, "q_gain": self.q_gain if s.qk_norm else None,
                "k_gain": self.k_gain if s.qk_norm else None, "cos": tables[0] if tables else None,
                "sin": tables[1] if tables else None, "heads": s.heads, "kv_heads": s.kv_heads, "head_dim": s.head_dim,
                "window": s.window, "qk_eps": s.qk_norm_eps, "scale": self.scale, "hidden": s.hidden}

    def forward(self, h, x, b, view, ws):
        s = self.spec
        T = h.shape[0]
        writes = view.writes and not s.reads_shared_kv
        kvh = 0 if s.reads_shared_kv else s.kv_heads
        table = b.tables[view.group]
        mark = ws.mark()
        tables = self.position.tables()
        cos, sin = tables if tables is not None else (None, None)
        rot = self.position.rot_dim
        flash = ops.flash_supported(s.head_dim, self.ctx.dtype)
        fused_post = (flash and rot in (0, s.head_dim) and b.max_count > 1 and (writes or s.reads_shared_kv)
                      and use_tc(T, self.qkv.out_features, self.qkv.in_features))
        if fused_post:
            # many tokens: the projection's epilogue post-processes q/k/v on its float32 accumulators
            q = ws.take((T, s.heads, s.head_dim), self.ctx.dtype)
            hh = h.tensor() if isinstance(h, Normed) else h
            ops.gemm_tc_qkv(hh, self.qkv.weight, s.heads, kvh, s.head_dim, self.bias, self.q_gain, self.k_gain,
                            cos if rot else None, sin if rot else None, s.qk_norm_eps, q,
                            view.k_pool if kvh else None, view.v_pool if kvh else None, b.tok_seq, b.tok_pos, table,
                            b.stream)
            y = ws.take((T, s.heads * s.head_dim), self.ctx.dtype)
            self._attend(q, y, b, view, table, ws)
            self.o.forward(y, into=x, ws=ws, stream=b.stream)
            ws.release(mark)
            return
        single = flash and b.max_count == 1 and rot in (0, s.head_dim) and (writes or s.reads_shared_kv)
        pages = None
        if single:
            splits = ops.decode_splits(b.n, s.kv_heads, s.heads // s.kv_heads, table.shape[1])
            # the attention kernel gets onto the SMs too late to fetch ahead: the projection asks L2 for its first pages
            pages = ops.next_pages(view.k_pool, view.v_pool, table, b.past, splits, view.window)
        qkv = self.qkv.forward(h, ws=ws, stream=b.stream, next_pages=pages)
        y = ws.take((T, s.heads * s.head_dim), self.ctx.dtype)
        if single:
            # one token per sequence: the attention kernel post-processes q/k/v itself and appends to the cache
            floats = ops.decode_scratch_floats(b.n, s.heads, s.head_dim, splits)
            scratch = ws.take((floats,), torch.float32) if floats else None
            ops.attention_decode(None, view.k_pool, view.v_pool, y, b.seq_start, b.past, table, s.heads, s.kv_heads,
                                 s.head_dim, view.window, self.scale, splits, scratch, b.stream, qkv=qkv,
                                 qkv_kv_heads=kvh, bias=self.bias, q_gain=self.q_gain, k_gain=self.k_gain,
                                 cos=cos if rot else None, sin=sin if rot else None, eps=s.qk_norm_eps,
                                 next_read=self.o.weight)
            self.o.forward(y, into=x, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None))
            ws.release(mark)
            return
        q = ws.take((T, s.heads, s.head_dim), self.ctx.dtype)
        ops.qkv_post(qkv, self.bias, self.q_gain, self.k_gain, cos, sin, q,
                     view.k_pool if writes else None, view.v_pool if writes else None,
                     b.tok_seq, b.tok_pos, table, s.heads, kvh, s.head_dim, rot, s.qk_norm_eps, b.stream)
        self._attend(q, y, b, view, table, ws)
        self.o.forward(y, into=x, ws=ws, stream=b.stream)
        ws.release(mark)


register_mixer("gqa_attention", GQAAttention)
