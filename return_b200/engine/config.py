"""Settings of the engine, with the reference's names where it has them.

``max_token``  capacity of the KV pool in token slots (rollout/server.py:91, rollout/cache.py:16);
``max_reside`` most requests that hold cache at a time = largest batch (rollout/server.py:90);
``page_size``  token slots per page (PAGE_SIZE, rollout/constant.py:1; 64 there, 16 here);
``prefill_chunk`` most tokens one step runs (PREFILL_CHUNK, rollout/constant.py:5);
``use_cuda_graph`` replay captured graphs for steps that only decode (USE_CUDA_GRAPH, :3);
``capture_at_start`` capture them all when the engine is built, as the reference does
(rollout/model.py:346-407), instead of each on its first use;
``keep_sessions`` a request that ends keeps its cache for a follow-up request with the same id, until
``release`` or until the pages are needed (the reference always keeps, rollout/engine.py:286-306).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class EngineConfig:
    max_token: int = 65536
    max_reside: int = 64
    page_size: int = 16
    prefill_chunk: int = 8192
    dtype: str = "bfloat16"               # "bfloat16" | "float32"
    max_model_len: Optional[int] = None   # longest sequence; default min(max_position_embeddings, max_token)
    use_cuda_graph: bool = True
    capture_at_start: bool = False
    keep_sessions: bool = False
    seed: int = 0
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.page_size <= 0 or self.max_token < self.page_size:
            raise ValueError("max_token must hold at least one page")
        if self.max_reside <= 0 or self.prefill_chunk <= 0:
            raise ValueError("max_reside and prefill_chunk must be positive")

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.float32 if self.dtype == "float32" else torch.bfloat16

    @property
    def num_pages(self) -> int:
        return self.max_token // self.page_size
