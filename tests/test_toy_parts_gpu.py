"""The framework's generality, shown with toy parts that exist only here: a mixer with per-sequence
state of its own, a layer named twice in the schedule, a layer that reads another layer's cache, a
feed-forward that routes every token to one of three experts, and another position encoding (positions
scaled down, only half of each head rotated). They are registered, built, loaded and stepped through the
public registries without touching a file of the package."""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from closeness import check
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

HID, HEADS, KVH, HD, INTER, VOCAB, EPS, THETA = 48, 4, 2, 16, 80, 97, 1e-5, 10000.0


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    variant: str = "state"
    head_dim: int = 16
    model_type: str = "toy"


@dataclass(frozen=True)
class RunningMeanSpec:
    hidden: int
    kind: str = "running_mean"


@dataclass(frozen=True)
class Top1ExpertsSpec:
    hidden: int
    inner: int
    experts: int
    kind: str = "top1_experts"


@dataclass(frozen=True)
class ScaledRotarySpec:
    head_dim: int
    theta: float
    factor: float
    rotary_dim: int
    kind: str = "scaled_rotary"


EXPERTS, EXPERT_INNER, POS_FACTOR, ROT = 3, 40, 4.0, 8
SOFTCAP, MAX_POS = 0.5, 256


@dataclass(frozen=True)
class LearnedPositionEmbeddingSpec:
    """Token table plus a learned table of absolute positions: a position encoding that lives in the embedding."""
    vocab: int
    dim: int
    positions: int
    name: str = "model.embed_tokens.weight"
    names: tuple = (("positions.weight", "model.embed_positions.weight"),)
    kind: str = "learned_position_embedding"


@dataclass(frozen=True)
class SoftcapHeadSpec:
    """Final norm, output matrix with a bias, logits squashed to (-cap, cap)."""
    vocab: int
    dim: int
    norm: object
    tied: bool
    cap: float
    norm_name: str = "model.norm.weight"
    name: str = "lm_head.weight"
    names: tuple = (("bias", "lm_head.bias"),)
    kind: str = "softcap_head"


def toy_spec(cfg: ToyConfig, tensor_names=None):
    from sleuth_b200.parts.spec import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelSpec,
                                        NormSpec, PositionSpec, ScheduleEntry)
    d = cfg.hidden_size
    HD = cfg.head_dim
    pos = PositionSpec(head_dim=HD, theta=THETA)
    ffn = GatedMLPSpec(hidden=d, intermediate=INTER)

    def names(i, mixer_names):
        p = f"model.layers.{i}."
        n = {"norm1.weight": p + "input_layernorm.weight", "norm2.weight": p + "post_attention_layernorm.weight",
             "ffn.gate.weight": p + "mlp.gate_proj.weight", "ffn.up.weight": p + "mlp.up_proj.weight",
             "ffn.down.weight": p + "mlp.down_proj.weight"}
        n.update({f"mixer.{k}": p + v for k, v in mixer_names.items()})
        return n

    attn_names = {f"{x}_proj.weight": f"self_attn.{x}_proj.weight" for x in "qkvo"}
    attn_names.update({"q_norm.weight": "self_attn.q_norm.weight", "k_norm.weight": "self_attn.k_norm.weight"})
    attn = AttentionSpec(hidden=d, heads=HEADS, kv_heads=KVH, head_dim=HD, position=pos, qk_norm=True, qk_norm_eps=EPS)
    layer0 = LayerSpec(mixer=attn, ffn=ffn, norm1=NormSpec(d, EPS), norm2=NormSpec(d, EPS), names=names(0, attn_names))
    if cfg.variant == "routed":
        # layer 0 rotates with the toy position encoding, layer 1 routes its feed-forward; both are toy kinds
        attn0 = AttentionSpec(hidden=d, heads=HEADS, kv_heads=KVH, head_dim=HD, qk_norm=True, qk_norm_eps=EPS,
                              position=ScaledRotarySpec(head_dim=HD, theta=THETA, factor=POS_FACTOR, rotary_dim=ROT))
        layer0 = LayerSpec(mixer=attn0, ffn=ffn, norm1=NormSpec(d, EPS), norm2=NormSpec(d, EPS), names=names(0, attn_names))
        n1 = names(1, attn_names)
        for k in [k for k in n1 if k.startswith("ffn.")]:
            del n1[k]
        n1["ffn.router.weight"] = "model.layers.1.moe.router.weight"
        for e in range(EXPERTS):
            n1[f"ffn.experts.{e}.up.weight"] = f"model.layers.1.moe.experts.{e}.up.weight"
            n1[f"ffn.experts.{e}.down.weight"] = f"model.layers.1.moe.experts.{e}.down.weight"
        layer1 = LayerSpec(mixer=attn, ffn=Top1ExpertsSpec(d, EXPERT_INNER, EXPERTS), norm1=NormSpec(d, EPS),
                           norm2=NormSpec(d, EPS), names=n1)
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1))
    elif cfg.variant == "learned":
        layer1, schedule = None, None           # built below, with the toy ends
    elif cfg.variant == "state":
        layer1 = LayerSpec(mixer=RunningMeanSpec(d), ffn=ffn, norm1=NormSpec(d, EPS), norm2=NormSpec(d, EPS),
                           names=names(1, {"w.weight": "mean_mixer.w.weight"}))
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2))      # layer 0 runs twice
    else:
        reader = AttentionSpec(hidden=d, heads=HEADS, kv_heads=KVH, head_dim=HD, position=pos, qk_norm=True,
                               qk_norm_eps=EPS, reads_shared_kv=True)
        rn = {"q_proj.weight": "self_attn.q_proj.weight", "o_proj.weight": "self_attn.o_proj.weight",
              "q_norm.weight": "self_attn.q_norm.weight"}
        layer1 = LayerSpec(mixer=reader, ffn=ffn, norm1=NormSpec(d, EPS), norm2=NormSpec(d, EPS), names=names(1, rn))
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 0))                           # layer 1 reads layer 0's cache
    embedding = EmbeddingSpec(vocab=cfg.vocab_size, dim=d)
    head = HeadSpec(vocab=cfg.vocab_size, dim=d, norm=NormSpec(d, EPS), tied=True)
    if cfg.variant == "learned":
        # no rotation anywhere: positions come from a learned table in the embedding; the head is a toy kind too
        nopos = PositionSpec(head_dim=HD, kind="none")
        attn_np = AttentionSpec(hidden=d, heads=HEADS, kv_heads=KVH, head_dim=HD, position=nopos, qk_norm=True, qk_norm_eps=EPS)
        layer0 = LayerSpec(mixer=attn_np, ffn=ffn, norm1=NormSpec(d, EPS), norm2=NormSpec(d, EPS), names=names(0, attn_names))
        layer1 = LayerSpec(mixer=attn_np, ffn=ffn, norm1=NormSpec(d, EPS), norm2=NormSpec(d, EPS), names=names(1, attn_names))
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1))
        embedding = LearnedPositionEmbeddingSpec(vocab=cfg.vocab_size, dim=d, positions=MAX_POS)
        head = SoftcapHeadSpec(vocab=cfg.vocab_size, dim=d, norm=NormSpec(d, EPS), tied=True, cap=SOFTCAP)
    return ModelSpec(embedding=embedding, layers=(layer0, layer1), schedule=schedule, head=head, max_positions=MAX_POS)


def make_running_mean_mixer():
    from sleuth_b200.cache.paged import StateRequest
    from sleuth_b200.parts.base import ParamDecl, Part

    class RunningMean(Part):
        """out[t] = W @ mean(h[0..t]) of the token's own sequence. The sum so far and the count are the
        sequence's state, kept in the cache's state region under the sequence's slot."""
        capturable = False      # it walks the step's sequences on the host

        def __init__(self, spec, ctx):
            self.hidden, self.ctx = spec.hidden, ctx

        def declare(self):
            return {"w.weight": ParamDecl((self.hidden, self.hidden))}

        def bind(self, t):
            self.w = t["w.weight"].float()

        def cache_request(self):
            return StateRequest((self.hidden + 1,), torch.float32)

        def forward(self, h, x, b, view, ws):
            start = 0
            for slot, count in zip(b.host_slots, b.host_counts):
                state = view.state[slot]
                hs = h[start:start + count].float()
                sums = state[:-1] + hs.cumsum(0)
                counts = state[-1] + torch.arange(1, count + 1, device=h.device, dtype=torch.float32)
                x[start:start + count] += (sums / counts[:, None]) @ self.w.T
                state[:-1] = sums[-1]
                state[-1] = counts[-1]
                start += count

    return RunningMean


def make_top1_experts():
    from sleuth_b200.parts.base import ParamDecl, Part

    class Top1Experts(Part):
        """Every token goes to the expert with the largest router logit (float32, first index on ties); the
        expert's output (relu MLP) is weighted by that expert's softmax probability and added to the stream."""
        capturable = False      # which rows go to which expert is read back on the host

        def __init__(self, spec, ctx):
            self.spec = spec

        def declare(self):
            s = self.spec
            d = {"router.weight": ParamDecl((s.experts, s.hidden))}
            for e in range(s.experts):
                d[f"experts.{e}.up.weight"] = ParamDecl((s.inner, s.hidden))
                d[f"experts.{e}.down.weight"] = ParamDecl((s.hidden, s.inner))
            return d

        def bind(self, t):
            self.router = t["router.weight"].float()
            self.up = [t[f"experts.{e}.up.weight"].float() for e in range(self.spec.experts)]
            self.down = [t[f"experts.{e}.down.weight"].float() for e in range(self.spec.experts)]

        def forward(self, h, x, b, ws):
            hf = h.float()
            prob = (hf @ self.router.T).softmax(-1)
            chosen = prob.argmax(-1)
            for e in range(self.spec.experts):
                rows = (chosen == e).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(hf[rows] @ self.up[e].T) @ self.down[e].T
                    x.index_add_(0, rows, y * prob[rows, e][:, None])

    return Top1Experts


def make_scaled_rotary():
    from sleuth_b200.parts.base import Part

    class ScaledRotary(Part):
        """Rotate-half over the first ``rotary_dim`` channels of a head, by the angle (position / factor) * frequency."""

        def __init__(self, spec, ctx):
            self.rot_dim = spec.rotary_dim
            inv = 1.0 / (spec.theta ** (torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim))
            ang = torch.outer(torch.arange(ctx.max_positions, dtype=torch.float32) / spec.factor, inv)
            self.cos, self.sin = ang.cos().contiguous().to(ctx.device), ang.sin().contiguous().to(ctx.device)

        def tables(self):
            return self.cos, self.sin

    return ScaledRotary


def make_learned_position_embedding():
    from sleuth_b200.parts.base import ParamDecl, Part

    class LearnedPositionEmbedding(Part):
        """x[t] = tokens[id of t] + positions[position of t]: it reads the batch's positions beside its token ids."""

        def __init__(self, spec, ctx):
            self.spec = spec

        def declare(self):
            return {"weight": ParamDecl((self.spec.vocab, self.spec.dim)),
                    "positions.weight": ParamDecl((self.spec.positions, self.spec.dim))}

        def bind(self, t):
            self.table, self.positions = t["weight"], t["positions.weight"]       # ``table``: what a tied head reads

        def forward(self, b, x):
            ids = b.token_ids[:x.shape[0]] if b.ids_map is None else b.token_ids[b.ids_map[:x.shape[0]].long()]
            x.copy_(self.table[ids.long()].float() + self.positions[b.tok_pos[:x.shape[0]].long()].float())

    return LearnedPositionEmbedding


def make_softcap_head():
    from sleuth_b200.parts import build_norm
    from sleuth_b200.parts.base import ParamDecl, Part

    class SoftcapHead(Part):
        """logits = cap * tanh((norm(x) @ W^T + bias) / cap) on the wanted rows."""

        def __init__(self, spec, ctx):
            self.spec, self.ctx = spec, ctx
            self.norm = build_norm(spec.norm, ctx)

        def declare(self):
            d = {"norm.weight": ParamDecl((self.spec.dim,), "vector", init="gain"), "bias": ParamDecl((self.spec.vocab,), "vector")}
            if not self.spec.tied:
                d["weight"] = ParamDecl((self.spec.vocab, self.spec.dim))
            return d

        def bind(self, t, embedding_table=None):
            self.norm.bind({"weight": t["norm.weight"]})
            self.weight = embedding_table if self.spec.tied else t["weight"]
            self.bias = t["bias"]

        def forward(self, x, b, logits, ws):
            h = torch.empty((logits.shape[0], self.spec.dim), dtype=self.ctx.dtype, device=x.device)
            self.norm.forward(x, h, b.rows, b.stream)
            raw = h.float() @ self.weight.float().T + self.bias
            logits.copy_(self.spec.cap * torch.tanh(raw / self.spec.cap))

    return SoftcapHead


@pytest.fixture()
def toy_registered():
    from sleuth_b200.config import register_architecture, unregister_architecture
    from sleuth_b200.parts import (register_embedding, register_ffn, register_head, register_mixer, register_position,
                                   unregister)
    register_mixer("running_mean", make_running_mean_mixer())
    register_ffn("top1_experts", make_top1_experts())
    register_position("scaled_rotary", make_scaled_rotary())
    register_embedding("learned_position_embedding", make_learned_position_embedding())
    register_head("softcap_head", make_softcap_head())
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec, model_types=("toy",))
    yield
    unregister_architecture("ToyForCausalLM")
    unregister("mixer", "running_mean")
    unregister("ffn", "top1_experts")
    unregister("position", "scaled_rotary")
    unregister("embedding", "learned_position_embedding")
    unregister("head", "softcap_head")


def settings(HD):
    return dict(d=HID, heads=HEADS, kv_heads=KVH, head_dim=HD, layers=2, eps=EPS, theta=THETA, tied=True, windows=[0, 0])


def plain_state_model(w, ids, HD=HD):
    s = settings(HD)
    x = w["model.embed_tokens.weight"][torch.as_tensor(ids)]
    cos, sin = plain.rope_tables(HD, len(ids), THETA)
    x = plain.block(x, w, 0, s, cos, sin)
    h = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], EPS)
    mean = h.cumsum(0) / torch.arange(1, len(ids) + 1)[:, None]
    x = x + mean @ w["model.layers.1.mean_mixer.w.weight"].T
    x = x + plain.swiglu(plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], EPS), w, "model.layers.1.mlp.")
    x = plain.block(x, w, 0, s, cos, sin)
    return plain.rms_norm(x, w["model.norm.weight"], EPS) @ w["model.embed_tokens.weight"].T


def plain_shared_kv_model(w, ids, HD=HD):
    s = settings(HD)
    T = len(ids)
    x = w["model.embed_tokens.weight"][torch.as_tensor(ids)]
    cos, sin = plain.rope_tables(HD, T, THETA)
    # keys and values of layer 0, as it stores them
    h0 = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], EPS)
    k = (h0 @ w["model.layers.0.self_attn.k_proj.weight"].T).view(T, KVH, HD).transpose(0, 1)
    v = (h0 @ w["model.layers.0.self_attn.v_proj.weight"].T).view(T, KVH, HD).transpose(0, 1)
    k = plain.apply_rope(plain.rms_norm(k, w["model.layers.0.self_attn.k_norm.weight"], EPS), cos, sin)
    x = plain.block(x, w, 0, s, cos, sin)
    h1 = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], EPS)
    q = (h1 @ w["model.layers.1.self_attn.q_proj.weight"].T).view(T, HEADS, HD).transpose(0, 1)
    q = plain.apply_rope(plain.rms_norm(q, w["model.layers.1.self_attn.q_norm.weight"], EPS), cos, sin)
    kk, vv = k.repeat_interleave(HEADS // KVH, 0), v.repeat_interleave(HEADS // KVH, 0)
    sc = (q @ kk.transpose(-2, -1)) / math.sqrt(HD)
    sc = sc.masked_fill(~plain.causal_mask(T, 0), float("-inf"))
    y = (sc.softmax(-1) @ vv).transpose(0, 1).reshape(T, HEADS * HD)
    x = x + y @ w["model.layers.1.self_attn.o_proj.weight"].T
    x = x + plain.swiglu(plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], EPS), w, "model.layers.1.mlp.")
    return plain.rms_norm(x, w["model.norm.weight"], EPS) @ w["model.embed_tokens.weight"].T


def plain_routed_model(w, ids, HD=HD):
    s = settings(HD)
    T = len(ids)
    x = w["model.embed_tokens.weight"][torch.as_tensor(ids)]
    # layer 0 by hand: its rotation is the toy one (scaled positions, the first ROT channels of a head only)
    inv = 1.0 / (THETA ** (torch.arange(0, ROT, 2, dtype=torch.float32) / ROT))
    ang = torch.outer(torch.arange(T, dtype=torch.float32) / POS_FACTOR, inv)

    def rotate(v):       # [heads, T, HD]
        a, b, rest = v[..., :ROT // 2], v[..., ROT // 2:ROT], v[..., ROT:]
        return torch.cat([a * ang.cos() - b * ang.sin(), b * ang.cos() + a * ang.sin(), rest], dim=-1)

    p = "model.layers.0.self_attn."
    h = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], EPS)
    q = (h @ w[p + "q_proj.weight"].T).view(T, HEADS, HD).transpose(0, 1)
    k = (h @ w[p + "k_proj.weight"].T).view(T, KVH, HD).transpose(0, 1)
    v = (h @ w[p + "v_proj.weight"].T).view(T, KVH, HD).transpose(0, 1)
    q = rotate(plain.rms_norm(q, w[p + "q_norm.weight"], EPS))
    k = rotate(plain.rms_norm(k, w[p + "k_norm.weight"], EPS))
    kk, vv = k.repeat_interleave(HEADS // KVH, 0), v.repeat_interleave(HEADS // KVH, 0)
    sc = ((q @ kk.transpose(-2, -1)) / math.sqrt(HD)).masked_fill(~plain.causal_mask(T, 0), float("-inf"))
    x = x + (sc.softmax(-1) @ vv).transpose(0, 1).reshape(T, HEADS * HD) @ w[p + "o_proj.weight"].T
    x = x + plain.swiglu(plain.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], EPS), w, "model.layers.0.mlp.")
    # layer 1: ordinary attention, then the routed feed-forward
    cos, sin = plain.rope_tables(HD, T, THETA)
    h = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], EPS)
    x = x + plain.attention(h, w, "model.layers.1.self_attn.", s, 0, cos, sin)
    h = plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], EPS)
    prob = (h @ w["model.layers.1.moe.router.weight"].T).softmax(-1)
    chosen = prob.argmax(-1)
    y = torch.zeros_like(x)
    for t in range(T):
        e = int(chosen[t])
        y[t] = (torch.relu(h[t] @ w[f"model.layers.1.moe.experts.{e}.up.weight"].T)
                @ w[f"model.layers.1.moe.experts.{e}.down.weight"].T) * prob[t, e]
    x = x + y
    return plain.rms_norm(x, w["model.norm.weight"], EPS) @ w["model.embed_tokens.weight"].T


def plain_learned_model(w, ids, HD=HD):
    T = len(ids)
    x = w["model.embed_tokens.weight"][torch.as_tensor(ids)] + w["model.embed_positions.weight"][:T]
    for i in range(2):
        p = f"model.layers.{i}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], EPS)
        q = (h @ w[p + "self_attn.q_proj.weight"].T).view(T, HEADS, HD).transpose(0, 1)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).view(T, KVH, HD).transpose(0, 1)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).view(T, KVH, HD).transpose(0, 1)
        q = plain.rms_norm(q, w[p + "self_attn.q_norm.weight"], EPS)            # normalised, never rotated
        k = plain.rms_norm(k, w[p + "self_attn.k_norm.weight"], EPS)
        kk, vv = k.repeat_interleave(HEADS // KVH, 0), v.repeat_interleave(HEADS // KVH, 0)
        sc = ((q @ kk.transpose(-2, -1)) / math.sqrt(HD)).masked_fill(~plain.causal_mask(T, 0), float("-inf"))
        x = x + (sc.softmax(-1) @ vv).transpose(0, 1).reshape(T, HEADS * HD) @ w[p + "self_attn.o_proj.weight"].T
        x = x + plain.swiglu(plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], EPS), w, p + "mlp.")
    raw = plain.rms_norm(x, w["model.norm.weight"], EPS) @ w["model.embed_tokens.weight"].T + w["lm_head.bias"]
    return SOFTCAP * torch.tanh(raw / SOFTCAP)


# float32: summation order only. bfloat16 (head size 64, so that the tensor-core attention kernels serve the toy
# parts' layers): weights rounded alike on both sides, activations rounded in the engine only; the logits of these
# models are about 1 in magnitude and the largest difference seen on a B200 was 0.0032: the bound is twice that.
TOY_TOL = {"fp32": dict(rtol=1e-4, atol=2e-5), "bf16": dict(rtol=0.0, atol=6.5e-3)}


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("variant,oracle", [("state", plain_state_model), ("shared_kv", plain_shared_kv_model),
                                            ("routed", plain_routed_model), ("learned", plain_learned_model)])
def test_toy_architecture_builds_loads_and_steps(variant, oracle, dtype, toy_registered, tmp_path):
    import functools

    import sleuth_b200 as sb
    from sleuth_b200.cache.paged import KVRequest, StateRequest
    hd = 16 if dtype == "fp32" else 64
    cfg = dict(architectures=["ToyForCausalLM"], model_type="toy", vocab_size=VOCAB, hidden_size=HID, variant=variant,
               head_dim=hd)
    folder = sb.write_random_model(tmp_path / variant, cfg, seed=3, dtype=torch.float32)
    _, w = plain.read_model(folder)
    if dtype == "bf16":
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    w = {k: v.float() for k, v in w.items()}
    oracle = functools.partial(oracle, HD=hd)
    tol = TOY_TOL[dtype]
    eng = sb.load(folder, dtype=dtype, max_seq_len=256, max_tokens=1024)
    reqs = eng.model.cache_requests
    if variant == "state":
        assert "model.layers.1.mean_mixer.w.weight" in w
        assert [type(r) for r in reqs] == [KVRequest, StateRequest, KVRequest]          # the repeated layer has two entries
    elif variant == "routed":
        assert "model.layers.1.moe.experts.2.down.weight" in w and "model.layers.1.mlp.gate_proj.weight" not in w
        assert [type(r) for r in reqs] == [KVRequest, KVRequest]
    elif variant == "learned":
        assert w["model.embed_positions.weight"].shape == (MAX_POS, HID) and w["lm_head.bias"].shape == (VOCAB,)
        assert type(eng.model.embedding).__name__ == "LearnedPositionEmbedding" and type(eng.model.head).__name__ == "SoftcapHead"
    else:
        assert "model.layers.1.self_attn.k_proj.weight" not in w and len(reqs) == 1     # one entry, written by layer 0
    rng = np.random.default_rng(1)
    a, b = rng.integers(0, VOCAB, size=70).tolist(), rng.integers(0, VOCAB, size=9).tolist()
    slots = eng.open(2)
    out = eng.step([(slots[0], a, tuple(range(70))), (slots[1], b, tuple(range(9)))]).cpu()
    want = torch.cat([oracle(w, a), oracle(w, b)])
    check(out, want, tol, "toy parts " + dtype)
    eng.close(slots)
    # a reused slot starts from a zeroed state; prompt then token by token equals the whole sequence
    (slot,) = eng.open(1)
    assert slot in slots
    rows = [eng.step([(slot, a[:40], (39,))]).cpu()]
    rows += [eng.step([(slot, [t], (0,))]).cpu().clone() for t in a[40:]]
    check(torch.cat(rows), oracle(w, a)[39:], tol, "toy parts " + dtype)
    eng.close([slot])
    res = eng.generate([a[:5], b], max_new_tokens=4, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=())
    if dtype == "fp32":
        assert res[0].new_ids[0] == int(oracle(w, a[:5])[-1].argmax())
    # parts that walk the step on the host or route by data are not recorded: no CUDA graph was made of a step
    recorded = variant in ("shared_kv", "learned")
    assert eng.model.capturable == recorded and (recorded or not eng.stepper._graphs)


def test_state_is_sized_by_sequences_not_by_pages(toy_registered):
    """A mixer that keeps a megabyte of state per sequence, in a cache of 4,096 pages: the state region holds as
    many rows as sequences may be live at once, so it takes megabytes, not the 4 GB that a row per page would."""
    from sleuth_b200.cache.paged import KVRequest, PagedCache, StateRequest
    big = StateRequest((512, 512), torch.float32)                    # 1 MiB per sequence
    reqs = [KVRequest(2, 16), big, None]
    before = torch.cuda.memory_allocated()
    cache = PagedCache(reqs, max_tokens=4096 * 64, max_seq_len=1024, dtype=torch.bfloat16, device="cuda:0", max_sequences=12)
    assert cache.n_pages == 4096 and cache.max_slots == 12 and cache.states[1].shape == (12, 512, 512)
    assert cache.book.max_slots == 12 and cache.book.groups[0].table.shape[0] == 12
    default = PagedCache(reqs, max_tokens=4096 * 64, max_seq_len=1024, dtype=torch.bfloat16, device="cuda:0")
    assert default.max_slots == 256 and default.states[1].numel() * 4 == 256 << 20
    assert torch.cuda.memory_allocated() - before < (1 << 30)
    assert PagedCache([KVRequest(2, 16)], 4096 * 64, 1024, torch.bfloat16, "cuda:0").max_slots == 4096    # no state: a slot per page
    slots = cache.open(12)
    with pytest.raises(Exception, match="slots"):
        cache.open(1)
    cache.states[1][slots[3]] += 1.0
    cache.close(slots)
    again = cache.open(12)
    assert float(cache.states[1][again].abs().sum()) == 0.0            # a slot taken again starts from a zeroed state


def test_shared_cache_entry_with_every_kernel_starting_early(toy_registered, tmp_path):
    """SLEUTH_B200_PDL=1 lets every kernel start while the one in front still runs. A layer that reads the cache entry
    another layer application of the same step wrote must then not ask for its pages before that writer has finished:
    single-token steps of the shared-cache toy model, in bfloat16 at head size 64 (the split-KV attention kernel with
    its q/k/v prologue), against the plain implementation."""
    import functools

    import sleuth_b200 as sb
    from sleuth_b200.kernels import ops
    cfg = dict(architectures=["ToyForCausalLM"], model_type="toy", vocab_size=VOCAB, hidden_size=HID, variant="shared_kv",
               head_dim=64)
    folder = sb.write_random_model(tmp_path / "shared", cfg, seed=4, dtype=torch.float32)
    _, w = plain.read_model(folder)
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    oracle = functools.partial(plain_shared_kv_model, HD=64)
    dll = ops.lib().dll
    before = dll.slb_get_pdl()
    dll.slb_set_pdl(1)
    try:
        eng = sb.load(folder, dtype="bf16", max_seq_len=256, max_tokens=1024)
        ids = np.random.default_rng(2).integers(0, VOCAB, size=150).tolist()
        (slot,) = eng.open(1)
        rows = [eng.step([(slot, ids[:100], (99,))]).cpu()]
        rows += [eng.step([(slot, [t], (0,))]).cpu().clone() for t in ids[100:]]      # eager, then recorded and replayed
        eng.close([slot])
        check(torch.cat(rows), oracle(w, ids)[99:], TOY_TOL["bf16"], "toy parts bf16")
    finally:
        dll.slb_set_pdl(before)
