"""A decoder made of parts: embedding, a schedule of blocks, final norm, output head.

The model knows nothing of Qwen3.  It is built from a ``DecoderSpec`` and asks each block for
its parameters under the names ``layers.<i>.<part>.<param>``, plus ``embed``, ``final_norm.weight``
and ``lm_head`` (an alias of ``embed`` when the specification ties them).  The forward pass of
one step follows the reference's (rollout/monkey_patch/qwen3.py:71-81): embed, run the layers,
final norm; the head is applied to the rows whose logits are wanted only
(rollout/model.py:286-290).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ext import ops
from ..parts.base import BLOCKS, NORMS, BuildEnv, KVCacheNeed, LayerContext, ParamSpec, StateNeed
from ..parts.spec import DecoderSpec


class DecoderModel:
    def __init__(self, spec: DecoderSpec, env: BuildEnv):
        spec.validate()
        self.spec = spec
        self._graph_safe = None
        self.env = env
        self.blocks = [BLOCKS.build(b, env) for b in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, env)
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ parameters
    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"embed": ParamSpec((s.vocab_size, s.hidden_size))}
        for i, block in enumerate(self.blocks):
            for name, ps in block.params().items():
                p[f"layers.{i}.{name}"] = ps
        for name, ps in self.final_norm.params().items():
            p[f"final_norm.{name}"] = ps
        if not s.tie_embeddings:
            p["lm_head"] = ParamSpec((s.vocab_size, s.hidden_size))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embed = tensors["embed"]
        self.lm_head = self.embed if self.spec.tie_embeddings else tensors["lm_head"]
        for i, block in enumerate(self.blocks):
            prefix = f"layers.{i}."
            block.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})
        self.final_norm.bind({k[len("final_norm."):]: v for k, v in tensors.items() if k.startswith("final_norm.")})

    @property
    def graph_safe(self) -> bool:
        if self._graph_safe is None:          # the parts do not change after the model is built
            self._graph_safe = all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe
        return self._graph_safe

    def batch_tilings(self):
        """Every table of query-row blocks that some part of the model reads (``Part.batch_tilings``)."""
        out = {}
        for b in self.blocks:
            for name, tiling in b.batch_tilings().items():
                if out.setdefault(name, tiling) != tiling:
                    raise ValueError(f"two parts ask for different tilings under the name {name!r}")
        return out

    def graph_variant(self, n_tokens: int, longest_context: int):
        """What a captured step of single tokens fixes beforehand, over all parts (``Part.graph_variant``)."""
        out = {}
        for b in self.blocks:
            out.update(b.graph_variant(n_tokens, longest_context))
        return out

    # ------------------------------------------------------------------ caches
    def cache_needs(self) -> List[object]:
        """Per schedule entry: what the run's mixer wants cached (None if it owns no cache)."""
        out = []
        for e in self.spec.schedule:
            out.append(self.blocks[e.layer].cache_need() if e.cache_of is None else None)
        return out

    # ------------------------------------------------------------------ one step
    def forward(self, batch, storage) -> torch.Tensor:
        """Runs the step's tokens through the schedule; returns float32 logits [n_want, vocab]."""
        T = batch.num_tokens
        H = self.spec.hidden_size
        dev = self.env.device
        stream = torch.empty((T, H), dtype=torch.float32, device=dev)
        ops.embedding(self.embed, batch.tokens, stream)
        delta = None
        schedule = self.spec.schedule
        for index, entry in enumerate(schedule):
            owner = index if entry.cache_of is None else entry.cache_of
            ctx = storage.layer_context(owner, batch, write=entry.cache_of is None)
            ctx.position = index
            ctx.next_block = self.blocks[schedule[index + 1].layer] if index + 1 < len(schedule) else None
            delta = self.blocks[entry.layer].forward(stream, delta, ctx)
        n_want = batch.num_want
        logits = torch.empty((n_want, self.spec.vocab_size), dtype=torch.float32, device=dev)
        if n_want:
            hidden = torch.empty((n_want, H), dtype=self.env.act_dtype, device=dev)
            self.final_norm.add_forward(stream, delta, hidden, rows=batch.want_rows)
            ops.linear(hidden, self.lm_head, logits)
        return logits
