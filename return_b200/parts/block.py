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

    # ------------------------------------------------------------------ few rows: norms and residual adds inside the products
    def first_norm(self):
        """(weight, eps, offset, size) of the RMSNorm that this block applies to the residual stream first, or None.
        The block that runs before this one may then prepare the normed rows in the epilogue of its last product."""
        n = self.mixer_norm
        if getattr(n.spec, "kind", None) == "rmsnorm" and hasattr(n, "p_weight"):
            return n.p_weight, n.spec.eps, n.spec.offset, n.spec.size
        return None

    def _fused_plan(self, stream):
        """For a step of few rows in bfloat16 the two norms and the two residual adds of the block cost no kernel of
        their own: the product before a norm (the mixer's last, the feed-forward's last) adds into the stream
        and leaves v * w and sum(v^2); the product after it (the gated one, the next block's first) scales by
        rstd (csrc/gemm_skinny.cu).  Six launches a layer instead of eight.  That needs a mixer and a feed-forward
        that expose their products, RMSNorms, and sizes the kernel takes; anything else runs part by part."""
        if self.env.act_dtype != torch.bfloat16 or stream.shape[0] > ops.SKINNY_MAX_ROWS:
            return None
        plan = getattr(self, "_fused_parts", None)
        if plan is None:
            plan = False
            mixer, ff = self.mixer, self.feed_forward
            n2 = self.feed_forward_norm
            norms_ok = self.first_norm() is not None and getattr(n2.spec, "kind", None) == "rmsnorm" and hasattr(n2, "p_weight")
            if norms_ok and hasattr(mixer, "in_projection") and hasattr(mixer, "core") and hasattr(ff, "gated_projections"):
                (w_in, in_name), w_out = mixer.in_projection(), mixer.out_projection()
                gate_up, down, interleave = ff.gated_projections()
                weights = (w_in, w_out, gate_up, down)
                if (interleave == 8 and gate_up.shape[0] % 16 == 0 and w_out.shape[0] == stream.shape[1] == down.shape[0]
                        and all(w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0
                                and w.data_ptr() % 16 == 0 for w in weights)):
                    plan = (w_in, in_name, w_out, gate_up, down)
            self._fused_parts = plan
        return plan or None

    def _forward_fused(self, plan, stream, delta, ctx):
        w_in, in_name, w_out, gate_up, down = plan
        T, H = stream.shape
        dev, dt = stream.device, self.env.act_dtype
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        held = ctx.batch.scratch
        # what the block before this one left for this block's first norm (made for this position of the schedule)
        pre = held.pop("block.prenormed", None)
        proj = ctx.buffer(in_name, (T, w_in.shape[0]), dt, dev)
        if delta is None and pre is not None and pre["position"] == ctx.position:
            ops.gemm_skinny_fused(pre["rows"], w_in, proj, scale=(pre["sums"], n1.spec.eps))
        else:
            a = ctx.buffer("block.normed", (T, H), dt, dev)
            n1.add_forward(stream, delta, a)                   # stream += delta; a = norm(stream)
            ops.gemm_skinny(a, w_in, proj)
        mixed = self.mixer.core(proj, ctx)
        rows2 = ctx.buffer("block.rows_mid", (T, H), dt, dev)
        sums2 = ops.RowSums(ctx.buffer("block.sums_mid", (8, ops.RowSums.WIDTH), torch.float32, dev), H)
        ops.gemm_skinny_fused(mixed, w_out, rows2, residual=(stream, (n2.p_weight, n2.spec.offset), sums2))
        act = ctx.buffer("block.gated_act", (T, gate_up.shape[0] // 2), dt, dev)
        ops.gemm_skinny_fused(rows2, gate_up, act, gated=True, scale=(sums2, n2.spec.eps))
        nxt = ctx.next_block.first_norm() if ctx.next_block is not None and hasattr(ctx.next_block, "first_norm") else None
        if nxt is not None and nxt[3] != H:
            nxt = None
        if nxt is None:
            ops.gemm_skinny_fused(act, down, None, residual=(stream, None, None))
        else:
            rows3 = ctx.buffer("block.rows_out", (T, H), dt, dev)
            sums3 = ops.RowSums(ctx.buffer("block.sums_out", (8, ops.RowSums.WIDTH), torch.float32, dev), H)
            ops.gemm_skinny_fused(act, down, rows3, residual=(stream, (nxt[0], nxt[2]), sums3))
            held["block.prenormed"] = {"rows": rows3, "sums": sums3, "position": ctx.position + 1}
        return None                                            # the stream already holds this block's output

    def forward(self, stream, delta, ctx):
        plan = self._fused_plan(stream) if getattr(ctx.batch, "scratch", None) is not None else None
        if plan is not None:
            return self._forward_fused(plan, stream, delta, ctx)
        T, H = stream.shape
        a = ctx.buffer("block.normed", (T, H), self.env.act_dtype, stream.device)
        self.mixer_norm.add_forward(stream, delta, a)             # stream += delta; a = norm(stream)
        mixed = self.mixer.forward(a, ctx)
        self.feed_forward_norm.add_forward(stream, mixed, a)      # stream += mixed; a = norm(stream)
        return self.feed_forward.forward(a, ctx)
