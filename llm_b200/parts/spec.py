"""Descriptions of a model as data.

A configuration class turns config.json into a `ModelSpec`: one `BlockSpec`
for every layer (its norms, its mixer, its feed-forward, each with all
sizes and constants), a schedule that says in which order layers run and
whose cache each reads, and the names of the tensors that every part
binds. Parts are built from these records through the registries in
`llm_b200.parts`; nothing here knows an architecture.

Any object with a `kind` attribute can stand as a spec: a part registered
under that kind receives it unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    weight: str                      # tensor name
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary encoding: angle = position * inv_freq[pair]."""
    head_dim: int
    theta: float
    max_positions: int
    scaling: Optional[tuple] = None  # sorted (key, value) pairs of rope_scaling, or None
    pairing: str = "half"            # 'half': (p, p + n/2); 'interleaved': (2p, 2p + 1)
    kind: str = "rope"
    rotary_dim: Optional[int] = None # n: how many leading elements of a head rotate (None: all)

    @property
    def scaling_dict(self):
        return dict(self.scaling) if self.scaling is not None else None


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float                     # multiplies q.k
    bias: bool
    window: int                      # 0: every earlier key; w > 0: the last w keys
    position: Optional[PositionSpec]
    names: tuple                     # sorted (role, tensor name): q, k, v, o (+ q_bias, ...)
    kind: str = "attention"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class GatedMlpSpec:
    hidden: int
    intermediate: int
    activation: str                  # 'silu'
    names: tuple                     # sorted (role, tensor name): gate, up, down
    kind: str = "gated_mlp"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class BlockSpec:
    """x += mixer(mixer_norm(x)); x += feed_forward(ffn_norm(x))  ('pre_norm')."""
    mixer_norm: object
    mixer: object
    ffn_norm: object
    feed_forward: object
    kind: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. `cache_of` names an earlier schedule entry whose
    keys and values this run reads instead of writing its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab: int
    hidden: int
    max_positions: int
    embedding: str                   # tensor name of the [vocab, hidden] table
    blocks: tuple                    # BlockSpec per layer
    schedule: tuple                  # ScheduleEntry, in running order
    final_norm: object
    head: Optional[str]              # tensor name of the [vocab, hidden] head; None: tied to the embedding
    stop_tokens: tuple = field(default_factory=tuple)
    embedding_scale: float = 1.0     # multiplies the embedded tokens
    logit_scale: float = 1.0         # multiplies the logits


def names(**roles) -> tuple:
    return tuple(sorted(roles.items()))
