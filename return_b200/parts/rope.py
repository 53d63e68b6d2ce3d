"""Rotary position encoding: tables of cos and sin, float32.

inv_freq[i] = theta^(-i / (R/2)), angle = position * inv_freq[i]
(rollout/monkey_patch/qwen3.py:121-127; rollout/utils/test_decode.py:14-17).  The reference
rounds its tables to bfloat16; these stay float32 in both precisions, because the rotation
angles belong to the arithmetic that is kept in 32-bit.  The rotation itself is fused into the
kernel that writes the cache (csrc/rope_cache.cu).
"""
from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

# every layer of a model asks for the same tables: one copy per (rotary width, theta, positions, device)
_TABLES = {}


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim={spec.rotary_dim} must be even")
        self._tables = None

    def rotary_tables(self):
        """(cos, sin, rotary_dim); cos and sin are float32 [max_positions, rotary_dim/2] on the device."""
        if self._tables is None:
            s = self.spec
            key = (s.rotary_dim, float(s.theta), s.max_positions, str(self.env.device))
            shared = _TABLES.get(key)
            if shared is None:
                half = s.rotary_dim // 2
                # made on the CPU in float32 so that every device sees the same angles
                inv_freq = 1.0 / (s.theta ** (torch.arange(0, half, dtype=torch.float32) / half))
                ang = torch.outer(torch.arange(s.max_positions, dtype=torch.float32), inv_freq)
                shared = _TABLES[key] = (ang.cos().contiguous().to(self.env.device),
                                         ang.sin().contiguous().to(self.env.device), s.rotary_dim)
            self._tables = shared
        return self._tables


def drop_shared_tables() -> None:
    """Forgets the shared tables (models that still hold them keep them alive)."""
    _TABLES.clear()
