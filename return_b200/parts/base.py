"""Interfaces of the parts and the registries that map a specification's ``kind`` to a class.

A part is built from its specification and a ``BuildEnv`` (activation dtype and device), says
which parameters it wants (``params``), receives them (``bind``) and runs (``forward``).  The
five families and what each must offer:

``Norm``              ``forward(x, out)``; ``add_forward(stream, delta, out, rows)``, the residual
                      add fused with the norm (stream is the float32 residual).
``PositionEncoding``  ``rotary_tables()`` -> (cos, sin, rotary_dim) for encodings that rotate pairs
                      of a head, or ``apply(qkv, batch, ...)`` for any other in-place encoding.
``Mixer``             ``cache_need()`` -> ``KVCacheNeed`` | ``StateNeed`` | None and
                      ``forward(x, ctx)`` with x [T, hidden] -> [T, hidden].
``FeedForward``       ``forward(x, ctx)``.
``Block``             ``forward(stream, delta, ctx)`` -> the delta still to be added to the stream.

Parameters have names local to the part ("qkv", "q_norm.weight").  Which checkpoint tensors
fill them is the architecture's knowledge, not the part's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class BuildEnv:
    act_dtype: torch.dtype            # torch.float32 (true 32-bit path) or torch.bfloat16
    device: torch.device


@dataclass(frozen=True)
class ParamSpec:
    """A parameter a part wants.  role "matrix": operand of a matrix product, kept in the
    activation dtype.  role "vector": a norm weight or the like; keeps float32 if stored so."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"              # random-weights law: "normal" N(0, .02) | "ones_normal" 1 + N(0, .1)


@dataclass(frozen=True)
class KVCacheNeed:
    """The mixer wants paged keys and values: all of them, or a window."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """The mixer wants one tensor of fixed shape per request."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class Tiling:
    """A table a part wants in every step's batch: the step's segments of several tokens cut into blocks of
    ``rows`` query rows, as (segment, first row within it) pairs.  ``heaviest_first``: the blocks with the most
    keys before them come first (they take longest, so they are launched first)."""
    rows: int
    heaviest_first: bool = False


@dataclass
class KVView:
    """One cache layer as a mixer sees it."""
    k: torch.Tensor                   # [num_pages, Hkv, page_size, D]
    v: torch.Tensor
    block_table: torch.Tensor         # int32 [segments of the step, blocks]
    page_size: int


@dataclass
class LayerContext:
    """What a part gets beside its input for one run of a layer in one step."""
    batch: Any                        # engine.batch.StepBatch
    kv: Optional[KVView] = None
    state: Optional[torch.Tensor] = None      # [num_slots, *StateNeed.shape]; row = batch.seg_slot
    write_cache: bool = True
    position: int = -1                        # index of this run in the model's schedule
    next_block: Any = None                    # the block that runs after this one in this step, or None (a block may
                                              # prepare what its successor's first norm needs)

    def buffer(self, name: str, shape, dtype, device) -> torch.Tensor:
        """An uninitialised work buffer for the part that asks.  The layers of a step run one after the
        other in one stream, so a buffer of the same name, shape and type is handed to every layer that
        asks for it: the step allocates once, not once per layer.  Whoever asks owns the contents until
        the next layer's part of the same name asks again; a name is unique to one use in one part."""
        held = getattr(self.batch, "scratch", None)
        if held is None:                       # a batch without a map of buffers: allocate each time
            return torch.empty(shape, dtype=dtype, device=device)
        key = (name, shape, dtype)
        t = held.get(key)
        if t is None:
            t = held[key] = torch.empty(shape, dtype=dtype, device=device)
        return t


def work_buffer(ctx: Optional[LayerContext], name: str, shape, dtype, device) -> torch.Tensor:
    """``ctx.buffer(...)``, or a fresh tensor for a part that is run on its own, without a context."""
    if ctx is None:
        return torch.empty(shape, dtype=dtype, device=device)
    return ctx.buffer(name, shape, dtype, device)


class Part:
    # False for a part whose forward looks at the step's tables on the host (its launches then
    # depend on the data, and a step that holds it is never captured in a CUDA graph)
    graph_safe = True

    def __init__(self, spec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def params(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for name, t in tensors.items():
            setattr(self, "p_" + name.replace(".", "_"), t)

    def batch_tilings(self) -> Dict[str, "Tiling"]:
        """Tables of query-row blocks that the part's kernels read, by name; the step's batch then holds
        ``batch.tiles[name]`` (device, int32 [blocks, 2]) and ``batch.host.tiles[name]``.  A name is the
        part's own ("attention.rows256"); the engine knows none of them."""
        return {}

    def graph_variant(self, n_tokens: int, longest_context: int) -> Dict[Any, Any]:
        """What a captured step of ``n_tokens`` single tokens must fix beforehand because a captured launch
        cannot change it (a grid size that follows from the context lengths), as {key: value}.  Steps whose
        variants are equal share a graph; inside the captured step the part finds its value under
        ``batch.variant[key]``.  ``longest_context`` is an upper bound of the step's context lengths."""
        return {}


class Norm(Part):
    def forward(self, x, out):
        raise NotImplementedError

    def add_forward(self, stream, delta, out, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_tables(self):
        return None

    def apply(self, qkv, batch, num_heads, num_kv_heads, head_dim):
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        return None

    def forward(self, x, ctx: LayerContext):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx: LayerContext):
        raise NotImplementedError


class Block(Part):
    def cache_need(self):
        return None

    def first_norm(self):
        """(weight, eps, offset, size) if the block's first act is an RMSNorm of the residual stream, else None."""
        return None

    def forward(self, stream, delta, ctx: LayerContext):
        raise NotImplementedError


# ------------------------------------------------------------------------------- registries

class Registry:
    def __init__(self, family: str):
        self.family = family
        self._classes: Dict[str, Callable] = {}

    def register(self, kind: str, cls=None):
        """``REG.register("kind", Class)`` or ``@REG.register("kind")``."""
        def put(c):
            self._classes[kind] = c
            return c
        return put(cls) if cls is not None else put

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def build(self, spec, env: BuildEnv):
        kind = getattr(spec, "kind", None)
        if kind not in self._classes:
            raise KeyError(f"no {self.family} of kind {kind!r}; registered: {sorted(self._classes)}")
        return self._classes[kind](spec, env)

    def kinds(self):
        return sorted(self._classes)


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
