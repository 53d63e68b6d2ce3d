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
    """``sample`` launches the kernel and waits for its result; ``launch`` / ``fetch`` are its two
    halves, with two slots of pinned memory so that one launch may be in flight while the next is
    prepared (the engine's decode loop reads a step's tokens while the next step runs)."""

    SLOTS = 2

    def __init__(self, device, max_rows: int = 256):
        self.device = torch.device(device)
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        self._cap = n
        self._host = [torch.empty(4 * n, dtype=torch.float32).pin_memory() for _ in range(self.SLOTS)]
        self._dev = torch.empty(4 * n, dtype=torch.float32, device=self.device)
        self._out_dev = torch.empty(2 * n, dtype=torch.float32, device=self.device)
        self._out_host = [torch.empty(2 * n, dtype=torch.float32).pin_memory() for _ in range(self.SLOTS)]
        self._done = [torch.cuda.Event() for _ in range(self.SLOTS)]
        self._rows = [0] * self.SLOTS

    def launch(self, logits: torch.Tensor, params: Sequence[Tuple[float, int, float, float]], slot: int = 0) -> torch.Tensor:
        """Starts the sampling of one token per row; ``params``: per row (temperature, top_k, top_p,
        uniform draw).  Returns the tokens as an int32 device tensor (valid in stream order until the
        next launch); ``fetch(slot)`` waits and brings them to the host."""
        n = logits.shape[0]
        assert n == len(params) and n > 0
        if n > self._cap:
            torch.cuda.current_stream().synchronize()       # nothing may still read the old buffers
            self._grow(max(n, 2 * self._cap))
        h = self._host[slot].numpy()
        arr = np.asarray(params, dtype=np.float64)
        h[0:n] = arr[:, 0]
        h[n:2 * n].view(np.int32)[:] = arr[:, 1].astype(np.int32)
        h[2 * n:3 * n] = arr[:, 2]
        h[3 * n:4 * n] = arr[:, 3]
        d = self._dev
        d[:4 * n].copy_(self._host[slot][:4 * n], non_blocking=True)
        toks = self._out_dev[:n].view(torch.int32)
        lps = self._out_dev[n:2 * n]
        ops.sample(logits, d[0:n], d[n:2 * n].view(torch.int32), d[2 * n:3 * n], d[3 * n:4 * n], toks, lps)
        self._out_host[slot][:2 * n].copy_(self._out_dev[:2 * n], non_blocking=True)
        self._done[slot].record()
        self._rows[slot] = n
        return toks

    def fetch(self, slot: int = 0) -> Tuple[List[int], List[float]]:
        """Tokens and log-probabilities of the launch in ``slot``, once they have arrived."""
        n = self._rows[slot]
        self._done[slot].synchronize()
        out = self._out_host[slot].numpy()
        return out[:n].view(np.int32).tolist(), out[n:2 * n].tolist()

    def sample(self, logits: torch.Tensor, params: Sequence[Tuple[float, int, float, float]]) -> Tuple[List[int], List[float]]:
        """``params``: per row (temperature, top_k, top_p, uniform draw).  Returns tokens and log-probs."""
        if logits.shape[0] == 0:
            return [], []
        self.launch(logits, params, 0)
        return self.fetch(0)
