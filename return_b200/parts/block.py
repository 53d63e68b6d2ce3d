"""The pre-norm residual block (rollout/monkey_patch/qwen3.py:59-68).

The residual stream is float32 in both precisions.  A block receives the stream and the
"delta" that the block before it still owes the stream, adds it inside its first norm
kernel, and returns its own feed-forward output as the next delta, so each residual add is
fused with the norm that follows it.
"""
from __future__ import annotations

import torch

from ..ext import ops
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

    # ------------------------------------------------------------------ few rows: products chained in persistent kernels
    def _chain_plan(self, stream):
        """For a step of few rows in bfloat16 the block runs as three kernels instead of eight: (residual add +
        norm + the mixer's first product), the mixer's middle, (the mixer's last product -> residual add + norm
        -> gated product -> last product), the last a persistent kernel whose weight stream does not stop
        between the products (csrc/gemm_chain.cu).  That needs a mixer and a feed-forward that expose their
        products, RMSNorms, and sizes the kernel takes; anything else runs part by part."""
        if self.env.act_dtype != torch.bfloat16 or stream.shape[0] > ops.CHAIN_MAX_ROWS:
            return None
        plan = getattr(self, "_chain_parts", None)
        if plan is None:
            plan = False
            mixer, ff = self.mixer, self.feed_forward
            norms_ok = all(getattr(n.spec, "kind", None) == "rmsnorm" and hasattr(n, "p_weight")
                           for n in (self.mixer_norm, self.feed_forward_norm))
            if norms_ok and hasattr(mixer, "in_projection") and hasattr(mixer, "core") and hasattr(ff, "gated_projections"):
                (w_in, in_name), w_out = mixer.in_projection(), mixer.out_projection()
                gate_up, down, interleave = ff.gated_projections()
                if interleave == 8 and ops.chain_ok(1, [ops.ChainStep(None, w, None, g) for w, g in
                                                        ((w_in, False), (w_out, False), (gate_up, True), (down, False))]):
                    plan = (w_in, in_name, w_out, gate_up, down)
            self._chain_parts = plan
        return plan or None

    def _forward_chained(self, plan, stream, delta, ctx):
        w_in, in_name, w_out, gate_up, down = plan
        T, H = stream.shape
        dev, dt = stream.device, self.env.act_dtype
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        held = getattr(ctx.batch, "scratch", None)
        # the residual stream goes stream -> other -> stream: every CTA reads one while one CTA writes the other
        other = ctx.buffer("block.stream_other", (T, H), torch.float32, dev)
        proj = ctx.buffer(in_name, (T, w_in.shape[0]), dt, dev)
        ops.gemm_chain(T, [ops.ChainStep(("norm", stream, other, delta, n1.p_weight, n1.spec.eps, n1.spec.offset), w_in, proj)], held)
        mixed = self.mixer.core(proj, ctx)
        inter = gate_up.shape[0] // 2
        y = ctx.buffer("block.mixer_out", (T, H), dt, dev)
        act = ctx.buffer("block.gated_act", (T, (inter + 31) // 32 * 32), dt, dev)      # in the chain kernel's own order of k
        out = ctx.buffer("block.ff_out", (T, H), dt, dev)
        ops.gemm_chain(T, [ops.ChainStep(mixed, w_out, y),
                           ops.ChainStep(("norm", other, stream, y, n2.p_weight, n2.spec.eps, n2.spec.offset), gate_up, act, gated=True),
                           ops.ChainStep("previous", down, out)], held)
        return out

    def forward(self, stream, delta, ctx):
        plan = self._chain_plan(stream)
        if plan is not None:
            return self._forward_chained(plan, stream, delta, ctx)
        T, H = stream.shape
        a = ctx.buffer("block.normed", (T, H), self.env.act_dtype, stream.device)
        self.mixer_norm.add_forward(stream, delta, a)             # stream += delta; a = norm(stream)
        mixed = self.mixer.forward(a, ctx)
        self.feed_forward_norm.add_forward(stream, mixed, a)      # stream += mixed; a = norm(stream)
        return self.feed_forward.forward(a, ctx)
