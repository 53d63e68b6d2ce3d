"""Trace replay: given token ids go through the engine's step function, logits come out.

The reference has no such program; its nearest pieces are the duck-typed requests that drive
``model.prefill`` / ``model.decode`` directly (rollout/utils/check_correctness.py:30-39) and the
hooks that record every logits row (rollout/utils/check_chunk_prefill.py:49-57).  ``TraceReplayer``
owns nothing but the loop: the model, the cache manager, the step function and the kernels are
the ones generation uses.  ``bin/trace_run`` is its command line.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ext import ops
from .config import EngineConfig
from .runner import ModelRunner


class TraceReplayer:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, max_reside: int = 8,
                 poison: bool = False, device: str = "cuda:0", use_cuda_graph: bool = False):
        """``use_cuda_graph``: steps that hold single tokens only replay captured graphs, as they do in
        generation (padded batch sizes, fixed key splits, tables at fixed addresses); off, every step is
        launched kernel by kernel.  The reference's check script has the same switch
        (rollout/utils/check_correctness.py:43-50, ``--graph``)."""
        if 64 % page_size:
            raise ValueError("page_size must divide 64")
        # every request's count is rounded up to a multiple of 64, so the pool is a multiple of 64
        max_token = max(64, (max_tokens + 63) // 64 * 64)
        # a trace step may bring any number of tokens, so the longest append is the pool itself
        cfg = EngineConfig(max_token=max_token, max_reside=max_reside, page_size=page_size, dtype=dtype,
                           prefill_chunk=max_token, use_cuda_graph=use_cuda_graph, device=device)
        self.runner = ModelRunner.from_model_dir(model_dir, cfg)
        if poison:
            self.runner.storage.poison()

    def run_step(self, record: dict) -> Optional[torch.Tensor]:
        """One trace step: all entries as one batch; then the requests named in ``end`` give back
        what they hold.  Returns float32 logits [wanted, vocab] or None if nothing was wanted."""
        runner = self.runner
        entries = []
        for e in record.get("entries", []):
            if not e["tokens"]:
                continue
            rid = e["id"]
            if rid not in runner.manager:
                runner.add_request(rid)
            entries.append(runner.reserve(rid, e["tokens"], e.get("want", [])))
        logits = None
        if entries:
            out = runner.step(entries)
            ops.check_status(runner.env.device)           # waits for the step; raises if a kernel's bounded wait gave up
            if out.shape[0]:
                logits = out
        for rid in record.get("end", []):
            if rid in runner.manager:
                runner.free_request(rid)
        return logits
