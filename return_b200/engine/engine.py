"""The Python entry point: ``Engine`` generates tokens for requests on one GPU.

In the reference's manner (rollout/engine.py:65-72,127-129,341-348): requests are ``Request``
records with its field names, ``submit`` hands one in, ``stats()`` reports throughput counters,
``KVCapacityError`` reports a pool that is too small.  The reference's engine is an asyncio task
behind Ray actors; this one is a plain object with a synchronous ``generate`` and a step-wise
interface (``add_request`` / ``step`` / ``has_unfinished``); ``AsyncEngine`` wraps it with the
reference's ``start`` / ``await submit`` / ``release`` shape.
"""
from __future__ import annotations

import asyncio
import time
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..cache.manager import KVCapacityError
from ..ext import ops
from ..sampling.sampler import Sampler, uniform_draw
from .config import EngineConfig
from .request import GenerationResult, Request
from .runner import ModelRunner
from .scheduler import Scheduler, StepPlan


class Engine:
    def __init__(self, model: Union[str, ModelRunner], config: Optional[EngineConfig] = None, **overrides):
        """``model``: a folder with config.json and model.safetensors (the model class is chosen by
        config.json), or a ready ``ModelRunner``.  ``overrides`` are EngineConfig fields
        (max_token, max_reside, page_size, prefill_chunk, dtype, seed, ...)."""
        if isinstance(model, ModelRunner):
            self.runner = model
            self.config = model.config
        else:
            import dataclasses
            self.config = dataclasses.replace(config or EngineConfig(), **overrides)
            self.runner = ModelRunner.from_model_dir(model, self.config)
        self.scheduler = Scheduler(self.runner.manager, self.config.prefill_chunk, self.runner.max_positions,
                                   keep_sessions=self.config.keep_sessions)
        self.sampler = Sampler(self.runner.env.device, max(16, self.config.max_reside))
        if self.config.capture_at_start and self.runner.runs_ahead():
            self.runner.capture_decode_graphs()
        self._t_start = time.perf_counter()
        self._acc_decode = self._acc_prefill = 0.0
        self._dc_tok = self._pf_tok = 0
        self._steps = self._preemptions = 0
        self._auto_id = 0

    # ------------------------------------------------------------------ step-wise interface
    def add_request(self, req: Request) -> None:
        if req.seed is None:
            req.seed = (self.config.seed * 1000003 + self.scheduler._arrivals) & 0x7FFFFFFFFFFFFFFF
        self.scheduler.add(req)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    def release(self, rid) -> bool:
        """Gives back the cache that an ended request kept (``keep``), as the reference's ``release`` does
        (rollout/engine.py:276-284)."""
        return self.scheduler.release(rid)

    def step(self) -> List[Request]:
        """One scheduling decision and one step of the model.  Returns the requests that ended in it
        (finished, or failed with ``finish_reason == "error"``)."""
        t0 = time.perf_counter()
        plan: StepPlan = self.scheduler.schedule()
        self._preemptions += len(plan.preempted)
        ended = list(plan.failed)
        if not plan.entries:
            return ended
        from .batch import StepEntry
        entries, samplers = [], []
        for e in plan.entries:
            entries.append(StepEntry(e.request.id, e.tokens, [len(e.tokens) - 1] if e.sample else [], e.start))
            if e.sample:
                r = e.request
                samplers.append((r, (r.temperature, r.top_k, r.top_p, uniform_draw(r.seed, len(r.output)))))
        logits = self.runner.step(entries)
        sampled: Dict[Hashable, tuple] = {}
        if samplers:
            toks, lps = self.sampler.sample(logits, [p for _, p in samplers])
            for (r, _), t, lp in zip(samplers, toks, lps):
                sampled[r.id] = (t, lp)
        else:
            torch.cuda.current_stream().synchronize()
        ops.check_status(self.runner.env.device)           # a kernel whose bounded wait gave up raises here, not garbage
        ended += self.scheduler.commit(plan, sampled)
        dt = time.perf_counter() - t0
        n_dec = sum(1 for e in plan.entries if len(e.tokens) == 1 and e.sample and len(e.request.output) > 1)
        n_pf = plan.num_tokens - n_dec
        if n_pf:
            self._acc_prefill += dt
        else:
            self._acc_decode += dt
        self._dc_tok += n_dec
        self._pf_tok += n_pf
        self._steps += 1
        return ended

    # ------------------------------------------------------------------ decode steps that run ahead of the host
    def _can_run_ahead(self) -> bool:
        """Every running request is decoding, none waits for a slot that is free, and decode steps go
        through captured graphs: the next step can then start before the host has read the last
        step's tokens, because its tokens can come straight from the sampler's device buffer."""
        sch = self.scheduler
        if not sch.running or not self.runner.runs_ahead():
            return False
        if sch.waiting and self.runner.manager.free_slots > 0:
            return False
        return all(r.output and r.num_computed == r.num_tokens - 1 for r in sch.running)

    def _decode_ahead(self, max_steps: Optional[int] = None) -> List[Request]:
        """Consecutive steps of one decoded token per running request, each launched while the step
        before it still runs: the host reads step k's tokens (and sees which requests ended) while
        step k + 1 is on the GPU.  A request that ends on a stop sequence has then run one token too
        many, which is dropped; ends by length are known beforehand and cost nothing.  Returns the
        requests that ended; stops at the first end, when pages run short (the ordinary step then
        decides who gives way), or after ``max_steps`` steps."""
        from .batch import StepEntry
        sch, mgr = self.scheduler, self.runner.manager
        reqs = list(sch.running)
        n = len(reqs)
        t0 = time.perf_counter()
        # steps until the first request ends by length: known now, never overrun
        room = min(min(r.max_new_tokens - len(r.output), sch.max_model_len - r.num_tokens) for r in reqs)
        limit = room if max_steps is None else min(room, max_steps)
        launched = committed = 0
        tokens_dev = None
        ended: List[Request] = []
        stop = False
        while True:
            can_launch = (not stop and launched < limit and launched - committed < Sampler.SLOTS
                          and mgr.fits_all([r.id for r in reqs], 1))
            if can_launch:
                entries = []
                for r in reqs:
                    tok = r.output[-1] if launched == committed else 0          # 0: replaced on the device
                    entries.append(StepEntry(r.id, [tok], [0], mgr.append(r.id, 1)))
                logits = self.runner.step(entries, tokens_dev if launched > committed else None)
                params = [(r.temperature, r.top_k, r.top_p, uniform_draw(r.seed, len(r.output) + launched - committed))
                          for r in reqs]
                tokens_dev = self.sampler.launch(logits, params, launched % Sampler.SLOTS)
                launched += 1
                continue
            if committed == launched:
                break
            toks, lps = self.sampler.fetch(committed % Sampler.SLOTS)
            committed += 1
            for r, t, lp in zip(reqs, toks, lps):
                if r.finish_reason is not None:
                    continue                                  # ended a step ago: this token is one too many
                r.num_computed += 1
                r.push(t, lp)
                if r.finished or r.num_tokens >= sch.max_model_len:
                    r.finish_reason = r.reason() if r.finished else "length"
                    ended.append(r)
                    stop = True
            self._steps += 1
            self._dc_tok += n
        for r in ended:
            sch.finish(r)
        self._acc_decode += time.perf_counter() - t0
        return ended

    def run(self, max_steps: Optional[int] = None) -> List[Request]:
        """Runs model steps until no request is left or ``max_steps`` steps have run; returns the requests
        that ended.  Decode steps run ahead of the host where they can (see ``_decode_ahead``)."""
        ended: List[Request] = []
        left = max_steps
        while self.has_unfinished() and (left is None or left > 0):
            if self._can_run_ahead():
                before = self._steps
                ended += self._decode_ahead(left)
                if left is not None:
                    left -= self._steps - before
                if self._steps > before:
                    continue
            ended += self.step()                              # also where pages run short and someone gives way
            if left is not None:
                left -= 1
        return ended

    # ------------------------------------------------------------------ whole generations
    def generate(self, prompts: Sequence[Union[Request, Sequence[int]]], max_new_tokens: int = 32,
                 temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0,
                 stop_ids: Optional[List[List[int]]] = None, seed: Optional[int] = None,
                 eos_token_id: Optional[int] = None, keep: Optional[bool] = None,
                 ids: Optional[Sequence[Hashable]] = None) -> List[GenerationResult]:
        """Generates for every prompt (token ids, or ``Request`` records with their own options) and
        returns the results in the order given.  ``eos_token_id`` is a stop sequence of one token.  A
        request that cannot fit the pool raises ``KVCapacityError``.  ``ids`` names the requests (sessions);
        with ``keep`` a request's cache stays when it ends, and a later call whose prompt for the same id
        begins with that request's prompt and output runs only what is new."""
        stop_ids = list(stop_ids or [])
        if eos_token_id is not None:
            stop_ids.append([int(eos_token_id)])
        reqs: List[Request] = []
        for i, p in enumerate(prompts):
            if isinstance(p, Request):
                r = p
            else:
                r = Request(id=ids[i] if ids is not None else f"gen-{self._auto_id}", prompt_ids=list(p),
                            max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                            stop_ids=list(stop_ids or []), seed=None if seed is None else seed + i, keep=keep)
                self._auto_id += 1
            self.add_request(r)
            reqs.append(r)
        while self.has_unfinished():
            for r in self.run():
                if r.finish_reason == "error" and r in reqs:
                    raise r.error
        return [GenerationResult(r.id, list(r.output), list(r.output_logprobs), len(r.output), r.finish_reason)
                for r in reqs]

    # ------------------------------------------------------------------ counters (rollout/engine.py:84-125,308-315)
    @property
    def run_time(self) -> float:
        return time.perf_counter() - self._t_start

    @property
    def decode_tps(self):
        return self._dc_tok / self._acc_decode if self._acc_decode > 0 else None

    @property
    def prefill_tps(self):
        return self._pf_tok / self._acc_prefill if self._acc_prefill > 0 else None

    def stats(self) -> dict:
        m = self.runner.manager
        rt = self.run_time
        return {
            "run_time": rt, "steps": self._steps,
            "running": len(self.scheduler.running), "pending": len(self.scheduler.waiting),
            "decode_tps": self.decode_tps, "prefill_tps": self.prefill_tps,
            "decode_duty": self._acc_decode / rt if rt > 0 else 0.0,
            "prefill_duty": self._acc_prefill / rt if rt > 0 else 0.0,
            "preemptions": self._preemptions, "kept_sessions": len(self.scheduler.kept),
            # the pages of every group of layers (a model with full and window layers has two pools)
            "page_used": sum(m.pages_used()), "page_total": sum(g.num_pages for g in m.groups),
            "page_groups": [{"name": g.name, "used": u, "total": g.num_pages, "window": g.window}
                            for g, u in zip(m.groups, m.pages_used())],
        }


class AsyncEngine:
    """The reference's calling shape: ``start()``, ``await submit(request)``, ``release(id)``, ``stats()``.

    ``submit`` resolves when the request has finished and returns it; a request that cannot fit
    raises ``KVCapacityError`` from ``submit``.  Steps run in a worker thread, as the reference runs
    its model calls (rollout/engine.py:370,394).  ``release`` gives back what a finished request kept
    (``Request.keep`` or ``EngineConfig.keep_sessions``); without either a finished request holds nothing."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self._futures: Dict[Hashable, asyncio.Future] = {}
        self._wake = asyncio.Event()
        self._task: Optional[asyncio.Task] = None

    def start(self) -> None:
        self._task = asyncio.get_running_loop().create_task(self._run())

    async def stop(self) -> None:
        if self._task is not None:
            self._task.cancel()
            try:
                await self._task
            except asyncio.CancelledError:
                pass
            self._task = None

    async def submit(self, req: Request) -> Request:
        fut = asyncio.get_running_loop().create_future()
        try:
            self.engine.add_request(req)
        except Exception as e:          # too long for the pool: report to this caller only
            fut.set_exception(e)
            return await fut
        self._futures[req.id] = fut
        self._wake.set()
        return await fut

    def release(self, rid) -> None:
        self.engine.release(rid)

    def stats(self) -> dict:
        return self.engine.stats()

    async def _run(self) -> None:
        while True:
            self._wake.clear()
            if not self.engine.has_unfinished():
                await self._wake.wait()
                continue
            # a few steps at a time, so that decode steps can run ahead of the host and a new request still
            # waits for eight steps at most before the scheduler sees it
            ended = await asyncio.to_thread(self.engine.run, 8)
            for r in ended:
                fut = self._futures.pop(r.id, None)
                if fut is None or fut.done():
                    continue
                if r.finish_reason == "error":
                    fut.set_exception(r.error)
                else:
                    fut.set_result(r)
            await asyncio.sleep(0)
