"""Plain Qwen3 dense decoder: whole sequences, no cache, one function per part.

Written from the formulas of tbertha35/Sleuth's model code (paths are relative to that project).
``tests/golden/make_golden.py`` compared it once with the reference's own ``Transformer`` on the
two tiny configurations; ``tests/test_plain.py`` checks it against those committed outputs.

Everything runs on the CPU with ordinary tensor operations, in the dtype of ``work`` (float32 or
float64). Nothing here is imported by the product path, and nothing of the product path is
imported here.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
              "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """All tensors of one file. Layout: u64 LE header length, JSON header, raw little-endian
    row-major data with offsets relative to the data section (sleuth/formats/safetensors.py:3-12)."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    header.pop("__metadata__", None)
    out = {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        buf = bytearray(raw[8 + n + b: 8 + n + e])
        if len(buf) == 0:
            out[name] = torch.empty(info["shape"], dtype=dt)
        else:
            out[name] = torch.frombuffer(buf, dtype=torch.uint8).view(dt).reshape(info["shape"]).clone()
    return out


def read_model(folder) -> tuple[dict, dict[str, torch.Tensor]]:
    """(config.json as a dict, tensors by name) of a model folder."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors = read_safetensors(folder / "model.safetensors")
    return cfg, tensors


def settings(cfg: dict) -> dict:
    """The numbers the formulas need, with the reference's defaults (sleuth/formats/hf.py:92-116)."""
    d = cfg["hidden_size"]
    heads = cfg["num_attention_heads"]
    n_layers = cfg["num_hidden_layers"]
    windows = [0] * n_layers
    if cfg.get("sliding_window") and (cfg.get("use_sliding_window") or cfg.get("layer_types")):
        kinds = cfg.get("layer_types")
        if kinds is None:
            first = cfg.get("max_window_layers", 0)
            kinds = ["sliding_attention" if i >= first else "full_attention" for i in range(n_layers)]
        windows = [cfg["sliding_window"] if k == "sliding_attention" else 0 for k in kinds]
    return dict(
        d=d, heads=heads, kv_heads=cfg.get("num_key_value_heads", heads),
        head_dim=cfg.get("head_dim") or d // heads, layers=n_layers,
        eps=cfg.get("rms_norm_eps", 1e-6), theta=float(cfg.get("rope_theta", 10000.0)),
        tied=bool(cfg.get("tie_word_embeddings", False)), windows=windows,
    )


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dimension; the gain multiplies directly
    (sleuth/forge/model/norm.py:50; the fused form sleuth/forge/model/fused_ops.py:47-51)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight.to(x.dtype)


def rope_tables(head_dim: int, length: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin [length, head_dim], built in float32: inv_freq[i] = theta^(-2i/head_dim),
    angle[p, i] = p * inv_freq[i], the half table repeated twice (sleuth/forge/model/rope.py:30-38)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    pos = torch.arange(length, dtype=torch.float32)
    ang = torch.outer(pos, inv_freq)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [heads, T, head_dim]; pairs channel i with i + head_dim/2:
    x' = x*cos + rotate_half(x)*sin, rotate_half(x) = cat(-x2, x1)
    (sleuth/forge/model/rope.py:41-43,55)."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos.to(x.dtype) + rot * sin.to(x.dtype)


def causal_mask(T: int, window: int) -> torch.Tensor:
    """True where query i may see key j: j <= i, and i - j < window when a window is set
    (sleuth/forge/model/attention.py:160-169)."""
    q = torch.arange(T)[:, None]
    k = torch.arange(T)[None, :]
    mask = k <= q
    if window:
        mask &= (q - k) < window
    return mask


def attention(h: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, s: dict, window: int,
              cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention of one layer over a whole sequence h [T, d].

    q/k/v projections with optional bias (sleuth/forge/model/attention.py:106-108); per-head RMSNorm
    of q and k with the layer's shared gain, before the rotation (:121-122); rotation of q and k
    (:125-126); scores * 1/sqrt(head_dim), query head h reads KV head h // (H/K), masked softmax and
    the weighted sum in the working precision (:195-206); output projection without bias (:155-157).
    """
    T = h.shape[0]
    H, K, hd = s["heads"], s["kv_heads"], s["head_dim"]

    def lin(name):
        y = h @ w[prefix + name + ".weight"].to(h.dtype).T
        b = w.get(prefix + name + ".bias")
        return y + b.to(h.dtype) if b is not None else y

    q = lin("q_proj").view(T, H, hd).transpose(0, 1)      # [H, T, hd]
    k = lin("k_proj").view(T, K, hd).transpose(0, 1)      # [K, T, hd]
    v = lin("v_proj").view(T, K, hd).transpose(0, 1)
    if prefix + "q_norm.weight" in w:
        q = rms_norm(q, w[prefix + "q_norm.weight"], s["eps"])
        k = rms_norm(k, w[prefix + "k_norm.weight"], s["eps"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    rep = H // K
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    scores = (q @ k.transpose(-2, -1)) * (1.0 / math.sqrt(hd))
    scores = scores.masked_fill(~causal_mask(T, window), float("-inf"))
    probs = scores.softmax(dim=-1)
    y = (probs @ v).transpose(0, 1).reshape(T, H * hd)
    return y @ w[prefix + "o_proj.weight"].to(h.dtype).T


def swiglu(h: torch.Tensor, w: dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)), silu(z) = z * sigmoid(z), no biases
    (sleuth/forge/model/mlp.py:37-41)."""
    g = h @ w[prefix + "gate_proj.weight"].to(h.dtype).T
    u = h @ w[prefix + "up_proj.weight"].to(h.dtype).T
    return ((g * torch.sigmoid(g)) * u) @ w[prefix + "down_proj.weight"].to(h.dtype).T


def block(x: torch.Tensor, w: dict[str, torch.Tensor], i: int, s: dict, cos, sin) -> torch.Tensor:
    """Pre-norm residual block: x += attn(norm1(x)); x += mlp(norm2(x))
    (sleuth/forge/model/transformer.py:78,87-88,96,99)."""
    p = f"model.layers.{i}."
    a = attention(rms_norm(x, w[p + "input_layernorm.weight"], s["eps"]), w, p + "self_attn.", s,
                  s["windows"][i], cos, sin)
    x = x + a
    m = swiglu(rms_norm(x, w[p + "post_attention_layernorm.weight"], s["eps"]), w, p + "mlp.")
    return x + m


def logits(cfg: dict, w: dict[str, torch.Tensor], tokens, work: torch.dtype = torch.float32,
           round_weights_to_bf16: bool = False, rows=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence: embedding lookup without scaling
    (sleuth/forge/model/transformer.py:345-348), the blocks, the final norm and the output
    matrix, which is the embedding when tied (:122,129-130,301-302).

    round_weights_to_bf16: every matrix and vector is first rounded to bfloat16 (what a
    bfloat16 engine holds), the arithmetic stays in ``work``. rows: the positions whose logits are
    returned (all of them when None); a large vocabulary makes the others expensive.
    """
    s = settings(cfg)
    if round_weights_to_bf16:
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    w = {k: v.to(work) for k, v in w.items()}
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["model.embed_tokens.weight"][ids]
    cos, sin = rope_tables(s["head_dim"], len(ids), s["theta"])
    for i in range(s["layers"]):
        x = block(x, w, i, s, cos, sin)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    h = rms_norm(x, w["model.norm.weight"], s["eps"])
    out = w["model.embed_tokens.weight"] if (s["tied"] or "lm_head.weight" not in w) else w["lm_head.weight"]
    return h @ out.T


# --------------------------------------------------------------------------- sampling ----

def final_logits(row: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
                 repetition_penalty: float = 1.0, recent: list[int] | None = None,
                 banned: list[int] | None = None) -> torch.Tensor:
    """The logits a token is drawn from, for one row [V]: ban list, repetition penalty on the recent
    tokens (positive logits divided, others multiplied), then for temperature > 0: divide by it,
    top-k, top-p (a token goes when the mass before it reaches p), min-p
    (sleuth/forge/infer/sampling.py:67-96,110-127)."""
    lo = torch.finfo(torch.float32).min
    x = row.float().clone()
    if banned:
        masked = x.clone()
        masked[[b for b in banned if b < x.numel()]] = lo
        if bool((masked > lo).any()):
            x = masked
    if recent and repetition_penalty != 1.0:
        idx = torch.as_tensor(sorted(set(recent)), dtype=torch.long)
        seen = x[idx]
        x[idx] = torch.where(seen > 0, seen / repetition_penalty, seen * repetition_penalty)
    if temperature <= 0:
        return x
    x = x / temperature
    if 0 < top_k < x.numel():
        kth = torch.topk(x, top_k).values[-1]
        x = x.masked_fill(x < kth, lo)
    if top_p < 1.0:
        p = x.softmax(-1)
        order = torch.argsort(x, descending=True, stable=True)
        before = p[order].cumsum(-1) - p[order]
        drop = torch.zeros_like(x, dtype=torch.bool)
        drop[order] = before >= top_p
        x = x.masked_fill(drop, lo)
    if min_p > 0.0:
        p = x.softmax(-1)
        x = x.masked_fill(p < min_p * p.max(), lo)
    return x


def draw(row: torch.Tensor, u: float) -> int:
    """Inverse-CDF draw in token order from softmax(row) with the uniform number u in [0, 1).
    (The reference draws with torch.multinomial, sleuth/forge/infer/sampling.py:106-107; the
    distribution is the same, the random stream is ours.)"""
    p = row.double().softmax(-1)
    cdf = p.cumsum(-1)
    target = u * float(cdf[-1])
    idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
    return min(idx, row.numel() - 1)


def greedy_generate(cfg: dict, w: dict[str, torch.Tensor], prompt: list[int], max_new_tokens: int,
                    stop_ids=(), work: torch.dtype = torch.float32) -> list[int]:
    """Cache-less greedy decoding: the whole sequence is recomputed for every token; argmax with
    the first index on ties; the stop token is kept (sleuth/forge/infer/generate.py:107-124,
    sleuth/forge/infer/sampling.py:104-105)."""
    ids = list(prompt)
    new = []
    for _ in range(max_new_tokens):
        row = logits(cfg, w, ids, work, rows=[len(ids) - 1])[0]
        tok = int(row.argmax())
        new.append(tok)
        ids.append(tok)
        if tok in stop_ids:
            break
    return new
