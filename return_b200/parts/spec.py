"""Specifications of the parts a decoder is put together from.

A specification is a frozen record of sizes and constants with a ``kind``.  The registries of
``return_b200/parts/registry.py`` map a kind to the class that runs it.  An architecture
(``return_b200/models``) turns its configuration into a ``DecoderSpec``: one ``BlockSpec`` per
layer, chosen layer by layer, and a ``schedule`` that says in which order layers run.  A
specification never names a model; a part built from it does not know which model it is in.

Anything with a ``kind`` attribute can be a specification, so a test or a later architecture
can define its own records for its own parts.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * (offset + w) over the last ``size`` elements."""
    size: int
    eps: float
    offset: float = 0.0
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Half-split rotary encoding of the first ``rotary_dim`` elements of a head."""
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    window: Optional[int] = None          # None: every earlier key; n: the last n keys
    qk_norm: Optional[NormSpec] = None    # per-head norm of q and k before the rotation
    position: Optional[Any] = None        # a position-encoding spec, e.g. RopeSpec
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down( silu(gate(x)) * up(x) ), dense.  ``interleave``: row layout of the fused gate_up weight:
    0 = all gate rows then all up rows; 8 = blocks of 8 gate rows then their 8 up rows, which lets
    the product's epilogue apply the gate (needs intermediate_size % 8 == 0)."""
    hidden_size: int
    intermediate_size: int
    interleave: int = 0
    kind: str = "swiglu"


@dataclass(frozen=True)
class BlockSpec:
    """The arrangement of one layer: x += mixer(norm(x)); x += feed_forward(norm(x))."""
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    kind: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` None: the run owns a cache of its own; an index: the run
    reads the cache that the schedule entry with that index wrote, and writes none."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class DecoderSpec:
    vocab_size: int
    hidden_size: int
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_embeddings: bool

    @staticmethod
    def in_order(n_layers: int) -> Tuple[ScheduleEntry, ...]:
        return tuple(ScheduleEntry(i) for i in range(n_layers))

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, there are {len(self.layers)}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which owns none")
