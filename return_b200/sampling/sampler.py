"""Sampling of next tokens on the device, with the reference's options and meanings.

Options per request (rollout/engine.py:17-21, rollout/model.py:15-61): ``temperature`` (<= 0:
greedy), ``top_k`` (0: off), ``top_p``; the log-probability of the chosen token comes from the raw
logits (rollout/model.py:64-67).  The kernel is csrc/sampling.cu.  The reference draws from torch's
global generator, so its samples depend on what else is in the batch; here each draw is one
uniform number computed on the host from (seed, index of the output token), the same whatever
the batch is.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from ..ext import ops

_MASK = (1 << 64) - 1


def uniform_draw(seed: int, index: int) -> float:
    """A number in [0, 1) from (seed, index): the splitmix64 finaliser, 24 bits kept so that it is
    exact in float32."""
    x = (seed * 0x9E3779B97F4A7C15 + (index + 1) * 0xBF58476D1CE4E5B9) & _MASK
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK
    x ^= x >> 31
    return (x >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device, max_rows: int = 256):
        self.device = torch.device(device)
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        self._cap = n
        self._host = torch.empty(4 * n, dtype=torch.float32).pin_memory()
        self._dev = torch.empty(4 * n, dtype=torch.float32, device=self.device)
        self._out_dev = torch.empty(2 * n, dtype=torch.float32, device=self.device)
        self._out_host = torch.empty(2 * n, dtype=torch.float32).pin_memory()

    def sample(self, logits: torch.Tensor, params: Sequence[Tuple[float, int, float, float]]) -> Tuple[List[int], List[float]]:
        """``params``: per row (temperature, top_k, top_p, uniform draw).  Returns tokens and log-probs."""
        n = logits.shape[0]
        assert n == len(params)
        if n == 0:
            return [], []
        if n > self._cap:
            self._grow(max(n, 2 * self._cap))
        h = self._host.numpy()
        arr = np.asarray(params, dtype=np.float64)
        h[0:n] = arr[:, 0]
        h[n:2 * n].view(np.int32)[:] = arr[:, 1].astype(np.int32)
        h[2 * n:3 * n] = arr[:, 2]
        h[3 * n:4 * n] = arr[:, 3]
        d = self._dev
        d[:4 * n].copy_(self._host[:4 * n], non_blocking=True)
        toks = self._out_dev[:n].view(torch.int32)
        lps = self._out_dev[n:2 * n]
        ops.sample(logits, d[0:n], d[n:2 * n].view(torch.int32), d[2 * n:3 * n], d[3 * n:4 * n], toks, lps)
        self._out_host[:2 * n].copy_(self._out_dev[:2 * n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        out = self._out_host.numpy()
        return out[:n].view(np.int32).tolist(), out[n:2 * n].tolist()
