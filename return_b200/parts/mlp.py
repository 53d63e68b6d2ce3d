"""Dense SwiGLU feed-forward (rollout/monkey_patch/qwen3.py:20-22,99-105)."""
from __future__ import annotations

import torch

from ..ext import ops
from .base import FEED_FORWARDS, FeedForward, ParamSpec, work_buffer


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """y = down( silu(g) * u ) with [g, u] = x @ gate_up^T.  The reference concatenates gate rows
    and up rows; ``spec.interleave`` may instead ask for blocks of 8 gate rows and 8 up rows, so that
    the product's epilogue applies the gate when a step has few rows."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.interleave not in (0, 8) or (spec.interleave and spec.intermediate_size % spec.interleave):
            raise ValueError("interleave is 0, or 8 with intermediate_size a multiple of 8")

    def params(self):
        s = self.spec
        return {"gate_up": ParamSpec((2 * s.intermediate_size, s.hidden_size)),
                "down": ParamSpec((s.hidden_size, s.intermediate_size))}

    def gated_projections(self):
        """(gate_up weight, down weight, rows of a gate/up block): a feed-forward that is "gated product, then
        product" says so, and a block may then run the two in a kernel of its own choosing."""
        return self.p_gate_up, self.p_down, self.spec.interleave

    def forward(self, x, ctx):
        s = self.spec
        T = x.shape[0]
        act = work_buffer(ctx, "mlp.act", (T, s.intermediate_size), x.dtype, x.device)
        ops.gated_linear(x, self.p_gate_up, act, s.interleave, ctx)
        y = work_buffer(ctx, "mlp.y", (T, s.hidden_size), x.dtype, x.device)
        ops.linear(act, self.p_down, y)
        return y
