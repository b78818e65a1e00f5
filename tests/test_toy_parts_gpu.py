"""The framework's generality, shown with toy parts that exist only here: a mixer with per-sequence
state of its own, a layer named twice in the schedule, and a layer that reads another layer's cache.
They are registered, built, loaded and stepped through the public registries without touching a
file of the package."""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

HID, HEADS, KVH, HD, INTER, VOCAB, EPS, THETA = 48, 4, 2, 16, 80, 97, 1e-5, 10000.0


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    variant: str = "state"
    model_type: str = "toy"


@dataclass(frozen=True)
class RunningMeanSpec:
    hidden: int
    kind: str = "running_mean"


def toy_spec(cfg: ToyConfig, tensor_names=None):
    from sleuth_b200.parts.spec import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelSpec,
                                        NormSpec, PositionSpec, ScheduleEntry)
    d = cfg.hidden_size
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
    if cfg.variant == "state":
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
    return ModelSpec(embedding=EmbeddingSpec(vocab=cfg.vocab_size, dim=d), layers=(layer0, layer1), schedule=schedule,
                     head=HeadSpec(vocab=cfg.vocab_size, dim=d, norm=NormSpec(d, EPS), tied=True), max_positions=256)


def make_running_mean_mixer():
    from sleuth_b200.cache.paged import StateRequest
    from sleuth_b200.parts.base import ParamDecl, Part

    class RunningMean(Part):
        """out[t] = W @ mean(h[0..t]) of the token's own sequence. The sum so far and the count are the
        sequence's state, kept in the cache's state region under the sequence's slot."""

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


@pytest.fixture()
def toy_registered():
    from sleuth_b200.config import register_architecture, unregister_architecture
    from sleuth_b200.parts import register_mixer, unregister
    register_mixer("running_mean", make_running_mean_mixer())
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec, model_types=("toy",))
    yield
    unregister_architecture("ToyForCausalLM")
    unregister("mixer", "running_mean")


def settings():
    return dict(d=HID, heads=HEADS, kv_heads=KVH, head_dim=HD, layers=2, eps=EPS, theta=THETA, tied=True, windows=[0, 0])


def plain_state_model(w, ids):
    s = settings()
    w = {k: v.float() for k, v in w.items()}
    x = w["model.embed_tokens.weight"][torch.as_tensor(ids)]
    cos, sin = plain.rope_tables(HD, len(ids), THETA)
    x = plain.block(x, w, 0, s, cos, sin)
    h = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], EPS)
    mean = h.cumsum(0) / torch.arange(1, len(ids) + 1)[:, None]
    x = x + mean @ w["model.layers.1.mean_mixer.w.weight"].T
    x = x + plain.swiglu(plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], EPS), w, "model.layers.1.mlp.")
    x = plain.block(x, w, 0, s, cos, sin)
    return plain.rms_norm(x, w["model.norm.weight"], EPS) @ w["model.embed_tokens.weight"].T


def plain_shared_kv_model(w, ids):
    s = settings()
    w = {k: v.float() for k, v in w.items()}
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


@pytest.mark.parametrize("variant,oracle", [("state", plain_state_model), ("shared_kv", plain_shared_kv_model)])
def test_toy_architecture_builds_loads_and_steps(variant, oracle, toy_registered, tmp_path):
    import sleuth_b200 as sb
    from sleuth_b200.cache.paged import KVRequest, StateRequest
    cfg = dict(architectures=["ToyForCausalLM"], model_type="toy", vocab_size=VOCAB, hidden_size=HID, variant=variant)
    folder = sb.write_random_model(tmp_path / variant, cfg, seed=3, dtype=torch.float32)
    _, w = plain.read_model(folder)
    eng = sb.load(folder, dtype="fp32", max_seq_len=256, max_tokens=1024)
    reqs = eng.model.cache_requests
    if variant == "state":
        assert "model.layers.1.mean_mixer.w.weight" in w
        assert [type(r) for r in reqs] == [KVRequest, StateRequest, KVRequest]          # the repeated layer has two entries
    else:
        assert "model.layers.1.self_attn.k_proj.weight" not in w and len(reqs) == 1     # one entry, written by layer 0
    rng = np.random.default_rng(1)
    a, b = rng.integers(0, VOCAB, size=70).tolist(), rng.integers(0, VOCAB, size=9).tolist()
    slots = eng.open(2)
    out = eng.step([(slots[0], a, tuple(range(70))), (slots[1], b, tuple(range(9)))]).cpu()
    torch.testing.assert_close(out, torch.cat([oracle(w, a), oracle(w, b)]), rtol=1e-4, atol=2e-5)
    eng.close(slots)
    # a reused slot starts from a zeroed state; prompt then token by token equals the whole sequence
    (slot,) = eng.open(1)
    assert slot in slots
    rows = [eng.step([(slot, a[:40], (39,))]).cpu()]
    rows += [eng.step([(slot, [t], (0,))]).cpu().clone() for t in a[40:]]
    torch.testing.assert_close(torch.cat(rows), oracle(w, a)[39:], rtol=1e-4, atol=2e-5)
    eng.close([slot])
    res = eng.generate([a[:5], b], max_new_tokens=4, sampling=sb.SamplingConfig(temperature=0.0), stop_ids=())
    assert res[0].new_ids[0] == int(oracle(w, a[:5])[-1].argmax())
