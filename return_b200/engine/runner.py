"""The step function: runs one batch of (request, next tokens) from the cache and returns the
logits at the wanted places.

The reference has two entry points that also sample, ``Model.prefill`` (which loops over chunk
steps itself) and ``Model.decode`` (rollout/model.py:184-343), and never mixes the two in one
forward.  Here there is one: ``ModelRunner.step(entries)``.  It runs exactly the tokens it is
given, as one packed batch, against the keys and values that earlier steps left in the pages.
Making room in the cache (``reserve``) is separate from running (``step``), so a scheduler can
decide what fits before anything is launched.
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager, KVCapacityError
from ..cache.storage import CacheStorage
from ..config import registry
from ..models.decoder import DecoderModel
from ..parts.base import BuildEnv
from ..weights import loader
from ..ext import ops
from .batch import BatchStaging, StaticDecodeBatch, StepBatch, StepEntry, build_host_batch
from .config import EngineConfig


def graph_batch_size(m: int, max_reside: int) -> int:
    """The batch size of the graph that runs a decode step of ``m`` tokens: ``m`` itself up to 8 (the
    weight-streaming kernels are compiled per row count), then the next of 12, 16, 24, 32, 48, 64, ...
    so that requests which end one by one do not each ask for a capture; the rows between are padding.
    Never more than ``max_reside``."""
    if m <= 8:
        return m
    n = 8
    while n < m:
        n += n // 2 if n & (n - 1) == 0 else n // 3
    return min(n, max(m, max_reside))


class ModelRunner:
    def __init__(self, model: DecoderModel, engine_config: EngineConfig, max_positions: int):
        self.model = model
        self.config = engine_config
        self.env = model.env
        self.max_positions = max_positions
        self.storage = CacheStorage(model.cache_needs(), engine_config.page_size, engine_config.num_pages,
                                    engine_config.max_reside, self.env,
                                    longest_append=min(engine_config.prefill_chunk, max_positions))
        self.manager: CacheManager = self.storage.make_manager()
        self.storage.allocate()
        self.staging = BatchStaging(self.env.device)
        self.vocab_size = model.spec.vocab_size
        self.tilings = model.batch_tilings()   # the tables of row blocks that the model's parts read, by name
        self._graphs = {}                   # (decode batch size, what the parts fixed) -> (graph, static batch, static logits)
        self._graph_keys = {}               # (decode batch size, span of context lengths) -> key of _graphs
        self._graph_pool = None
        self.launches_per_replay = {}       # decode batch size -> kernels of this package in its graph

    # ------------------------------------------------------------------ building
    @classmethod
    def from_model_dir(cls, model_dir: str, engine_config: EngineConfig) -> "ModelRunner":
        """Reads config.json, picks the architecture from the registry and loads the safetensors."""
        if not torch.cuda.is_available():
            raise RuntimeError("return_b200 runs on a CUDA device (B200, sm_100a); none is visible")
        arch, cfg = registry.read_config(model_dir)
        device = torch.device(engine_config.device)
        env = BuildEnv(engine_config.act_dtype, device)
        # like the reference, the position tables are sized by the pool, not by
        # max_position_embeddings (rollout/monkey_patch/qwen3.py:121-127)
        max_positions = engine_config.max_model_len or min(engine_config.max_token, 1 << 20)
        model = DecoderModel(arch.decoder_spec(cfg, max_positions), env)
        expected = {n: shape for n, (shape, _) in loader.checkpoint_shapes(arch, cfg).items()}
        params = loader.load_parameters(model.params(), arch.weight_sources(cfg), expected, model_dir,
                                        env.act_dtype, device, arch.ignorable_tensors(cfg))
        model.bind(params)
        runner = cls(model, engine_config, max_positions)
        runner.model_config = cfg
        return runner

    @classmethod
    def from_random(cls, cfg, engine_config: EngineConfig, seed: int = 0) -> "ModelRunner":
        """A model of configuration ``cfg`` with random weights made on the device (no model folder)."""
        if not torch.cuda.is_available():
            raise RuntimeError("return_b200 runs on a CUDA device (B200, sm_100a); none is visible")
        arch = registry.resolve(cfg.to_dict())
        device = torch.device(engine_config.device)
        env = BuildEnv(engine_config.act_dtype, device)
        max_positions = engine_config.max_model_len or min(engine_config.max_token, 1 << 20)
        model = DecoderModel(arch.decoder_spec(cfg, max_positions), env)
        shapes = loader.checkpoint_shapes(arch, cfg)
        with torch.cuda.device(device):
            params = loader.random_parameters(model.params(), arch.weight_sources(cfg), shapes, seed,
                                              env.act_dtype, device)
        model.bind(params)
        runner = cls(model, engine_config, max_positions)
        runner.model_config = cfg
        return runner

    # ------------------------------------------------------------------ requests
    def add_request(self, rid: Hashable) -> int:
        return self.manager.add(rid)         # the storage zeroes the slot's state (CacheManager.on_slot_taken)

    def free_request(self, rid: Hashable) -> None:
        self.manager.free(rid)

    def reserve(self, rid: Hashable, tokens: Sequence[int], want: Sequence[int] = ()) -> StepEntry:
        """Makes room for the request's next tokens and returns the step entry for them.
        Raises KVCapacityError, changing nothing, if the pages do not suffice."""
        n = len(tokens)
        if self.manager.length(rid) + n > self.max_positions:
            raise ValueError(f"request {rid!r} would reach {self.manager.length(rid) + n} tokens; "
                             f"the engine was set up for {self.max_positions}")
        start = self.manager.append(rid, n)
        return StepEntry(rid=rid, tokens=tokens, want=want, start=start)

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the entries as one batch; float32 logits [wanted places, vocab], in entry order.

        ``device_tokens`` (int32 [n], a step of single decoded tokens through a captured graph only): the
        tokens are taken from this device tensor, in stream order, instead of from the entries; this is
        how a step starts before the host has seen the tokens the step before it sampled."""
        host = build_host_batch(entries, self.manager, self.vocab_size, self.max_positions, self.tilings)
        with torch.cuda.device(self.env.device):
            if self.config.use_cuda_graph and host.num_tokens == host.num_segments and self.model.graph_safe:
                return self._graphed_decode(host, device_tokens)
            if device_tokens is not None:
                raise ValueError("tokens on the device are taken by captured decode steps only")
            batch = StepBatch(host, self.env.device, self.staging)
            return self.model.forward(batch, self.storage)

    # ------------------------------------------------------------------ CUDA graphs for decode steps
    def runs_ahead(self) -> bool:
        """Whether decode steps go through captured graphs, which can take their tokens from the device."""
        return bool(self.config.use_cuda_graph and self.model.graph_safe)

    def _graphed_decode(self, host, device_tokens=None) -> torch.Tensor:
        """A step of single decoded tokens replays a graph captured for its batch size, as the
        reference does (rollout/model.py:346-407); graphs are captured on first use.  A captured
        launch cannot change its grid, so there is one graph per batch size and per set of choices that
        the model's parts make from the context lengths (``Part.graph_variant``: the attention's number
        of key splits).  They are asked with the span of context lengths (the longest request's, rounded
        up to a power of two or one and a half), so that many steps share a graph."""
        m = host.num_tokens
        n = self.graph_batch_size(m)
        key = self._graph_key(n, int(host.seg_kv_len.max()))
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(key)
        graph, static, logits = entry
        static.fill(host)
        if device_tokens is not None:
            static.tokens[:m].copy_(device_tokens[:m], non_blocking=True)     # after the upload, in stream order
        graph.replay()
        if host.num_want == m and (host.want_rows == range(m)).all():
            return logits[:m]
        return logits.index_select(0, torch.as_tensor(host.want_rows, dtype=torch.int64).to(logits.device))

    def graph_batch_size(self, m: int) -> int:
        return graph_batch_size(m, self.config.max_reside)

    @staticmethod
    def _span(longest: int) -> int:
        span = 512
        while span < longest:
            span += span // 2 if span & (span - 1) == 0 else span // 3     # 512, 768, 1024, 1536, 2048, ...
        return span

    def _graph_key(self, n: int, longest: int):
        span = self._span(longest)
        key = self._graph_keys.get((n, span))
        if key is None:                      # asked of every part of every layer: once per (batch size, span), not per step
            variant = self.model.graph_variant(n, span)
            key = self._graph_keys[(n, span)] = (n, tuple(sorted(variant.items(), key=repr)))
        return key

    def _capture(self, key):
        n, variant = key
        max_blocks = [(self.max_positions + g.page_size - 1) // g.page_size for g in self.manager.groups]
        static = StaticDecodeBatch(n, max_blocks, self.env.device, dict(variant), pad_slot=self.config.max_reside,
                                   tilings=self.tilings)
        side = torch.cuda.Stream(device=self.env.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                      # warm-up outside the capture
            self.model.forward(static, self.storage)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.env.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(static, self.storage)
        self.launches_per_replay[n] = ops.launch_count - before
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        self._graphs[key] = (graph, static, logits)
        return self._graphs[key]

    def capture_decode_graphs(self, batch_sizes=None) -> int:
        """Captures the decode graphs ahead of the first request (the reference's ``build_graph``): for every
        batch size that ``graph_batch_size`` can give (or those asked for), one graph per variant that
        a span of context lengths up to the engine's limit leads to.  Returns how many graphs there are."""
        sizes = batch_sizes or sorted({self.graph_batch_size(m) for m in range(1, self.config.max_reside + 1)})
        spans, span = [], self._span(1)
        while True:
            spans.append(span)
            if span >= self.max_positions:
                break
            span = self._span(span + 1)
        for n in sizes:
            for key in sorted({self._graph_key(n, sp) for sp in spans}, key=repr):
                if key not in self._graphs:
                    self._capture(key)
        return len(self._graphs)
