"""Dense SwiGLU feed-forward (rollout/monkey_patch/qwen3.py:20-22,99-105)."""
from __future__ import annotations

import torch

from ..ext import ops
from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """y = down( silu(g) * u ) with [g, u] = x @ gate_up^T, gate rows first, as the reference
    concatenates them."""

    def params(self):
        s = self.spec
        return {"gate_up": ParamSpec((2 * s.intermediate_size, s.hidden_size)),
                "down": ParamSpec((s.hidden_size, s.intermediate_size))}

    def forward(self, x, ctx):
        s = self.spec
        T = x.shape[0]
        gu = torch.empty((T, 2 * s.intermediate_size), dtype=x.dtype, device=x.device)
        ops.linear(x, self.p_gate_up, gu)
        act = torch.empty((T, s.intermediate_size), dtype=x.dtype, device=x.device)
        ops.swiglu(gu, act)
        y = torch.empty((T, s.hidden_size), dtype=x.dtype, device=x.device)
        ops.linear(act, self.p_down, y)
        return y
