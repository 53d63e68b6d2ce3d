"""The pre-norm residual block (rollout/monkey_patch/qwen3.py:59-68).

The residual stream is float32 in both precisions.  A block receives the stream and the
"delta" that the block before it still owes the stream, adds it inside its first norm
kernel, and returns its own feed-forward output as the next delta, so each residual add is
fused with the norm that follows it.
"""
from __future__ import annotations

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.mixer = MIXERS.build(spec.mixer, env)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, env)
        self.mixer_norm = NORMS.build(spec.mixer_norm, env)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, env)
        self._children = {"mixer": self.mixer, "feed_forward": self.feed_forward,
                          "mixer_norm": self.mixer_norm, "feed_forward_norm": self.feed_forward_norm}

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self._children.values())

    def params(self):
        return {f"{child}.{name}": p for child, part in self._children.items()
                for name, p in part.params().items()}

    def bind(self, tensors):
        for child, part in self._children.items():
            prefix = child + "."
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def cache_need(self):
        return self.mixer.cache_need()

    def batch_tilings(self):
        out = {}
        for part in self._children.values():
            out.update(part.batch_tilings())
        return out

    def graph_variant(self, n_tokens, longest_context):
        out = {}
        for part in self._children.values():
            out.update(part.graph_variant(n_tokens, longest_context))
        return out

    def forward(self, stream, delta, ctx):
        T, H = stream.shape
        a = ctx.buffer("block.normed", (T, H), self.env.act_dtype, stream.device)
        self.mixer_norm.add_forward(stream, delta, a)             # stream += delta; a = norm(stream)
        mixed = self.mixer.forward(a, ctx)
        self.feed_forward_norm.add_forward(stream, mixed, a)      # stream += mixed; a = norm(stream)
        return self.feed_forward.forward(a, ctx)
