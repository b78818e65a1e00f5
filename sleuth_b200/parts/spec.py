"""Descriptions of a model as data: which parts make up each layer, and in which order layers run.

An architecture turns its typed configuration into one ``ModelSpec``. Everything below the
architecture works from these descriptions alone: the part registries build a part from its spec
(``spec.kind`` names the class), the cache sizes its groups from what the parts ask for, and the
engine runs ``ModelSpec.schedule``. A spec carries every size and constant its part needs; no part
looks at a configuration or knows which model it sits in.

The reference composes its model the same way in spirit: ``make_norm(kind, dim, eps)``
(sleuth/forge/model/norm.py:53-58), ``make_mlp(cfg)`` (sleuth/forge/model/mlp.py:59-60), a per-layer
``attn_spec(i)`` (sleuth/forge/model/config.py:142-147) and ``shared_layers`` for a layer applied
more than once (sleuth/forge/model/config.py:80-86).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping


@dataclass(frozen=True)
class NormSpec:
    dim: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys. ``kind="rotary"``: rotate-half pairs (i, i+rot/2)
    over the first ``rotary_dim`` channels of each head; ``kind="none"``: nothing."""
    head_dim: int
    theta: float = 10000.0
    rotary_dim: int = 0          # 0 = all of head_dim
    kind: str = "rotary"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over the key/value cache."""
    hidden: int                  # width of the input and of the output
    heads: int                   # query heads
    kv_heads: int                # key/value heads; divides ``heads``
    head_dim: int                # independent of ``hidden``
    position: PositionSpec
    qk_norm: bool = False        # per-head RMSNorm of q and k before the position encoding
    qk_norm_eps: float = 1e-6
    qkv_bias: bool = False
    window: int = 0              # 0 = every earlier key; n = the n most recent keys, the query's own included
    scale: float = 0.0           # 0 = 1/sqrt(head_dim)
    reads_shared_kv: bool = False  # no k/v projections: reads the cache another layer application wrote
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(x)) * up(x)), no biases."""
    hidden: int
    intermediate: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``kind``) of a mixer, a feed-forward and their norms.

    ``names`` maps each part-local tensor name ("norm1.weight", "mixer.q_proj.weight",
    "ffn.down.weight", ...) to its name in the weight files."""
    mixer: object
    ffn: object
    norm1: NormSpec
    norm2: NormSpec
    names: Mapping[str, str] = field(default_factory=dict)
    kind: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One application of a layer. ``cache`` numbers the cache entry it uses; the first application
    in schedule order that names an entry owns it (and writes it), later ones only read it."""
    layer: int
    cache: int


@dataclass(frozen=True)
class EmbeddingSpec:
    """The part that fills the stream from token ids. ``name`` is the checkpoint name of its tensor ``weight``; a
    part of another ``kind`` that declares more tensors gives their checkpoint names in a field ``names``
    (local name -> checkpoint name) of its own spec class."""
    vocab: int
    dim: int
    scale: float = 1.0
    name: str = "model.embed_tokens.weight"
    kind: str = "token_embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Final norm and output matrix. ``tied``: the output matrix is the embedding table. ``norm_name`` and ``name``
    are the checkpoint names of the tensors ``norm.weight`` and ``weight``; more tensors of another ``kind`` are
    named by a field ``names`` (local name -> checkpoint name) of its own spec class."""
    vocab: int
    dim: int
    norm: NormSpec
    tied: bool
    norm_name: str = "model.norm.weight"
    name: str = "lm_head.weight"
    kind: str = "lm_head"


@dataclass(frozen=True)
class ModelSpec:
    embedding: EmbeddingSpec
    layers: tuple
    schedule: tuple
    head: HeadSpec
    max_positions: int
    ignored_tensors: tuple = ()   # regular expressions of tensor names a checkpoint may hold and nobody reads

    def __post_init__(self):
        seen = set()
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.layers)}")
            seen.add(e.cache)
        if seen and seen != set(range(len(seen))):
            raise ValueError(f"cache entries must be numbered 0..{len(seen) - 1} without gaps, got {sorted(seen)}")


def straight_schedule(n_layers: int) -> tuple:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(ScheduleEntry(i, i) for i in range(n_layers))
