"""The Qwen3 dense decoder (``Qwen3ForCausalLM``): its typed configuration and its model description.

Field names are the keys of the architecture's own ``config.json``. Defaults and refusals follow
sleuth/formats/hf.py:83-118: ``rms_norm_eps`` 1e-6, ``rope_theta`` 10000, ``num_key_value_heads`` =
heads, ``head_dim`` = hidden/heads (an independent ``head_dim`` is allowed, hf.py:94,105), only the
SiLU gate (hf.py:87-88), no RoPE scaling (hf.py:89-91). The model is pre-norm blocks of
GQA attention with per-head QK RMSNorm and rotate-half RoPE plus a SwiGLU feed-forward
(sleuth/forge/model/transformer.py:75-99, attention.py:101-157, mlp.py:37-41).

Two things are read here that the reference infers from tensor names instead (hf.py:113-116):
``attention_bias`` and ``tie_word_embeddings``. The weight loader reports a disagreement between
these keys and the tensors in the file as missing or unexpected tensors.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..parts.spec import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelSpec, NormSpec,
                          PositionSpec, straight_schedule)
from .base import ConfigError


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int | None = None
    head_dim: int | None = None
    hidden_act: str = "silu"
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: dict | None = None
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int | None = None
    layer_types: tuple[str, ...] | None = None
    eos_token_id: int | tuple[int, ...] | None = None
    bos_token_id: int | None = None
    model_type: str = "qwen3"

    def __post_init__(self):
        def need(cond, msg):
            if not cond:
                raise ConfigError("config.json: " + msg)

        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "max_position_embeddings"):
            need(getattr(self, key) > 0, f"{key} must be positive, got {getattr(self, key)}")
        need(self.hidden_act == "silu", f"hidden_act {self.hidden_act!r} is not supported (only the SiLU gate)")
        if self.rope_scaling:
            kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
            need(kind in (None, "default"), f"rope_scaling {dict(self.rope_scaling)} is not supported")
        need(self.kv_heads > 0 and self.num_attention_heads % self.kv_heads == 0,
             f"num_attention_heads ({self.num_attention_heads}) must be a multiple of num_key_value_heads "
             f"({self.kv_heads})")
        if self.head_dim is None:
            need(self.hidden_size % self.num_attention_heads == 0,
                 f"hidden_size ({self.hidden_size}) must be divisible by num_attention_heads "
                 f"({self.num_attention_heads}) when head_dim is not given")
        need(self.head_size > 0 and self.head_size % 2 == 0, f"head_dim must be even for RoPE, got {self.head_size}")
        need(self.rms_norm_eps > 0, f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        need(self.rope_theta > 0, f"rope_theta must be positive, got {self.rope_theta}")
        if self.layer_types is not None:
            need(len(self.layer_types) == self.num_hidden_layers,
                 f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
            bad = sorted(set(self.layer_types) - {"full_attention", "sliding_attention"})
            need(not bad, f"layer_types entries must be 'full_attention' or 'sliding_attention', got {bad}")
        if self.layer_types is not None and "sliding_attention" in self.layer_types:
            need(self.sliding_window is not None and self.sliding_window > 0,
                 "layer_types names sliding_attention layers, which need sliding_window > 0")
        if self.sliding_window is not None:
            need(self.sliding_window > 0, f"sliding_window must be positive, got {self.sliding_window}")

    # ---- derived ----
    @property
    def kv_heads(self) -> int:
        return self.num_key_value_heads if self.num_key_value_heads is not None else self.num_attention_heads

    @property
    def head_size(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_size // self.num_attention_heads

    @property
    def windows(self) -> tuple[int, ...]:
        """Window of each layer, 0 = every earlier key. A layer slides when ``layer_types`` says so,
        or, without ``layer_types``, when ``use_sliding_window`` is set and its index is at least
        ``max_window_layers``. A query sees keys ``p - window + 1 .. p``
        (sleuth/forge/model/attention.py:160-169)."""
        n = self.num_hidden_layers
        w = self.sliding_window or 0
        if self.layer_types is not None:
            return tuple(w if t == "sliding_attention" else 0 for t in self.layer_types)
        if self.use_sliding_window and w:
            first = self.max_window_layers if self.max_window_layers is not None else 0
            return tuple(w if i >= first else 0 for i in range(n))
        return (0,) * n

    @property
    def stop_ids(self) -> tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        return (self.eos_token_id,) if isinstance(self.eos_token_id, int) else tuple(self.eos_token_id)

    def to_json_dict(self) -> dict:
        """The ``config.json`` that reads back as this configuration."""
        d = {
            "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.kv_heads,
            "head_dim": self.head_size, "hidden_act": self.hidden_act,
            "max_position_embeddings": self.max_position_embeddings, "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta, "attention_bias": self.attention_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if any(self.windows):
            d.update(use_sliding_window=True, sliding_window=self.sliding_window,
                     layer_types=["sliding_attention" if w else "full_attention" for w in self.windows])
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id if isinstance(self.eos_token_id, int) else list(self.eos_token_id)
        return d


def qwen3_model_spec(cfg: Qwen3Config, tensor_names=None) -> ModelSpec:
    """The description the engine builds the Qwen3 model from. Tensor names are the checkpoint's own
    (sleuth/formats/hf.py:10-17).

    tensor_names: the names a checkpoint holds, when one is being loaded. The output matrix is tied
    to the embedding when the configuration says so or when the checkpoint has no ``lm_head.weight``
    (sleuth/formats/hf.py:114); a tied model ignores an ``lm_head.weight`` that a file still carries
    (hf.py:285-288)."""
    tied = cfg.tie_word_embeddings or (tensor_names is not None and "lm_head.weight" not in tensor_names)
    d, eps = cfg.hidden_size, cfg.rms_norm_eps
    position = PositionSpec(head_dim=cfg.head_size, theta=cfg.rope_theta)
    ffn = GatedMLPSpec(hidden=d, intermediate=cfg.intermediate_size, activation="silu")
    layers = []
    for i, window in enumerate(cfg.windows):
        p = f"model.layers.{i}."
        names = {"norm1.weight": p + "input_layernorm.weight", "norm2.weight": p + "post_attention_layernorm.weight"}
        for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
            names[f"mixer.{proj}.weight"] = p + f"self_attn.{proj}.weight"
        for proj in ("q_proj", "k_proj", "v_proj"):
            names[f"mixer.{proj}.bias"] = p + f"self_attn.{proj}.bias"
        names["mixer.q_norm.weight"] = p + "self_attn.q_norm.weight"
        names["mixer.k_norm.weight"] = p + "self_attn.k_norm.weight"
        for local, theirs in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
            names[f"ffn.{local}.weight"] = p + f"mlp.{theirs}.weight"
        mixer = AttentionSpec(hidden=d, heads=cfg.num_attention_heads, kv_heads=cfg.kv_heads,
                              head_dim=cfg.head_size, position=position, qk_norm=True, qk_norm_eps=eps,
                              qkv_bias=cfg.attention_bias, window=window)
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm1=NormSpec(d, eps), norm2=NormSpec(d, eps), names=names))
    return ModelSpec(
        embedding=EmbeddingSpec(vocab=cfg.vocab_size, dim=d),
        layers=tuple(layers),
        schedule=straight_schedule(cfg.num_hidden_layers),
        head=HeadSpec(vocab=cfg.vocab_size, dim=d, norm=NormSpec(d, eps), tied=tied),
        max_positions=cfg.max_position_embeddings,
        ignored_tensors=(r".*rotary_emb\.inv_freq$",) + ((r"lm_head\.weight$",) if tied else ()),
    )
