"""RMSNorm (rollout/fused.py:6-17 with OFFSET = 0 for Qwen3, rollout/monkey_patch/qwen3.py:15-17)."""
from __future__ import annotations

import torch

from ..ext import ops
from .base import NORMS, Norm, ParamSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * (offset + weight), float32 arithmetic, one rounding."""

    def params(self):
        return {"weight": ParamSpec((self.spec.size,), role="vector", init="ones_normal")}

    def forward(self, x, out):
        ops.rmsnorm_rows(x, self.p_weight, self.spec.eps, out, offset=self.spec.offset)
        return out

    def add_forward(self, stream, delta, out, rows=None):
        """stream (float32 residual) += delta, then out = norm(stream).  With ``rows`` only those rows
        are normalised and the stream is left as it is."""
        ops.add_rmsnorm(stream, delta, self.p_weight, self.spec.eps, out, rows=rows, offset=self.spec.offset)
        return out
