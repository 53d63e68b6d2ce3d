"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees, and decides what happens when pages run out.  Host code only.

The reference (rollout/engine.py:199-409) admits a request only if the pages for its *whole*
uncached prompt fit beside what the running decodes need next, runs all prompt chunks of the
admitted group before any decode, lets decodes that find no page wait, and fails the first
waiter when none fits; it never preempts.  This scheduler differs where one step function
allows it:

* every step is a mix: first one token for every running request that is decoding, then, with
  what is left of the budget (``prefill_chunk`` tokens a step), portions of prompts in order of
  arrival, running requests before newly admitted ones;
* pages are taken portion by portion, not for the whole prompt at admission;
* when a decoding request finds no page, the youngest running request is preempted: its pages
  go back and it returns to the head of the queue with prompt + output as its new prompt
  (recompute), so the oldest requests always make progress and nothing deadlocks;
* a request that does not fit the empty pool on its own gets ``KVCapacityError``
  (at submit if the prompt alone is too long, else when it has grown that far);
* a request that ends may keep what it holds (``keep``), as every session of the reference does until
  ``release`` (rollout/engine.py:266-306): a later request with the same id whose prompt begins with
  the kept tokens starts behind them.  Kept sessions are a cache, not a promise: when pages or slots run
  short the one kept longest gives them back before any running request is preempted, and a follow-up
  whose prompt does not continue the kept tokens starts from nothing.
"""
from __future__ import annotations

from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Deque, Hashable, List, Optional

from ..cache.manager import CacheManager, KVCapacityError
from .request import Request


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    start: int                       # position of tokens[0]
    sample: bool                     # the portion reaches the end of what is known: sample the next token


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)

    @property
    def num_decode(self) -> int:
        return sum(1 for e in self.entries if e.request.output and len(e.tokens) == 1 and e.sample)


class Scheduler:
    def __init__(self, manager: CacheManager, prefill_chunk: int, max_model_len: int, keep_sessions: bool = False):
        self.manager = manager
        self.prefill_chunk = prefill_chunk
        self.max_model_len = max_model_len
        self.keep_sessions = keep_sessions
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []         # in order of admission: the last is the youngest
        self.kept: "OrderedDict[Hashable, List[int]]" = OrderedDict()    # ended requests that kept their cache: id -> cached tokens
        self._arrivals = 0

    # ------------------------------------------------------------------ requests
    def pool_tokens(self) -> int:
        return min(g.num_pages * g.page_size for g in self.manager.groups if g.window is None) \
            if any(g.window is None for g in self.manager.groups) else self.max_model_len

    def add(self, req: Request) -> None:
        if not req.prompt_ids:
            raise ValueError("a request needs at least one prompt token")
        if req.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if len(req.prompt_ids) > self.max_model_len - 1:
            raise KVCapacityError(f"prompt of {len(req.prompt_ids)} tokens exceeds the engine's sequence limit {self.max_model_len}")
        if len(req.prompt_ids) > self.pool_tokens():
            raise KVCapacityError('Request prefill exceeds the GPU KV page capacity')     # rollout/engine.py:219-221
        if any(r.id == req.id for r in self.running) or any(r.id == req.id for r in self.waiting):
            raise ValueError(f"request {req.id!r} is still running")
        req.arrival = self._arrivals
        self._arrivals += 1
        cached = self.kept.pop(req.id, None)
        if cached is not None:
            # a follow-up of a kept session starts behind the cached tokens if its prompt continues them
            if len(req.prompt_ids) > len(cached) and req.prompt_ids[:len(cached)] == cached:
                req.num_computed = len(cached)
            else:
                self.manager.free(req.id)
        self.waiting.append(req)

    def release(self, rid) -> bool:
        """Gives back what an ended request kept (rollout/engine.py:276-284); a request that still runs keeps
        nothing when it ends.  Returns whether anything was given back or marked."""
        if rid in self.kept:
            del self.kept[rid]
            self.manager.free(rid)
            return True
        for r in list(self.running) + list(self.waiting):
            if r.id == rid:
                r.keep = False
                return True
        return False

    def _evict_kept(self) -> bool:
        """The session that was kept longest gives back its pages and its slot; False if none is kept."""
        if not self.kept:
            return False
        rid, _ = self.kept.popitem(last=False)
        self.manager.free(rid)
        return True

    def finish(self, req: Request) -> None:
        """The request has ended: it leaves the running list and gives back what it holds, or keeps it."""
        self.running.remove(req)
        keep = self.keep_sessions if req.keep is None else req.keep
        # steps that ran ahead of the host may have cached a token or two past the request's end
        overrun = self.manager.length(req.id) > req.num_computed
        if keep and req.finish_reason != "error" and req.num_computed > 0 and (not overrun or self.manager.truncatable):
            if overrun:
                self.manager.truncate(req.id, req.num_computed)
            self.kept[req.id] = req.all_ids[:req.num_computed]
        else:
            self.manager.free(req.id)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one step
    def _max_fit(self, rid, want: int) -> int:
        """The most tokens (<= want) that the request can append with the pages that are free now."""
        if want <= 0:
            return 0
        if self.manager.fits(rid, want):
            return want
        lo, hi = 0, want                      # fits(lo) is true for lo = 0
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.manager.fits(rid, mid):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.manager.free(req.id)
        self.running.remove(req)
        req.num_computed = 0
        req.num_preemptions += 1
        self.waiting.appendleft(req)
        plan.preempted.append(req)

    def _fail(self, req: Request, plan: StepPlan, err: BaseException) -> None:
        if req.id in self.manager:
            self.manager.free(req.id)
        if req in self.running:
            self.running.remove(req)
        req.finish_reason, req.error = "error", err
        plan.failed.append(req)

    def _portion(self, req: Request, budget: int, plan: StepPlan, fits_budget: bool = False) -> int:
        """Plans the next portion of a request that still has uncomputed tokens; returns its size.
        ``fits_budget``: the caller has just seen that ``budget`` tokens fit the free pages."""
        total = req.num_tokens
        remaining = total - req.num_computed
        if not fits_budget:
            while not self.manager.fits(req.id, min(remaining, budget)) and self._evict_kept():
                pass
        n = min(remaining, budget) if fits_budget else self._max_fit(req.id, min(remaining, budget))
        if n <= 0:
            return 0
        start = self.manager.append(req.id, n)
        assert start == req.num_computed
        plan.entries.append(PlannedEntry(req, req.ids_slice(start, start + n), start, sample=(start + n == total)))
        return n

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        while True:
            budget = self.prefill_chunk
            # 1. one token for every decoding request, oldest first; the youngest give way
            for req in list(self.running):
                if req not in self.running or not req.output or req.num_computed != req.num_tokens - 1:
                    continue
                fits = self.manager.fits(req.id, 1)
                while not fits and self._evict_kept():
                    fits = self.manager.fits(req.id, 1)
                while not fits:
                    victim = self.running[-1]
                    if victim is req:
                        break
                    self._undo_entry(victim, plan)
                    self._preempt(victim, plan)
                    fits = self.manager.fits(req.id, 1)
                if not fits:
                    # alone and still no page: the request does not fit the pool
                    if len(self.running) == 1:
                        self._fail(req, plan, KVCapacityError('Active KV exhausted the GPU pool'))   # rollout/engine.py:336-338
                    else:
                        self._undo_entry(req, plan)
                        self._preempt(req, plan)
                    continue
                if budget <= 0:
                    continue
                budget -= self._portion(req, 1, plan, fits_budget=True)
            # 2. portions of prompts of running requests, then of newly admitted ones
            planned = {id(e.request) for e in plan.entries}
            for req in self.running:
                if budget <= 0:
                    break
                if id(req) in planned or req.num_computed >= req.num_tokens:
                    continue
                budget -= self._portion(req, budget, plan)
            while self.waiting and budget > 0:
                req = self.waiting[0]
                if req in plan.preempted:
                    break                     # it just gave way; it comes back in a later step
                resumed = req.id in self.manager          # a follow-up of a kept session: its slot and pages are there
                if not resumed:
                    if self.manager.free_slots == 0 and not self._evict_kept():
                        break
                    self.manager.add(req.id)
                got = self._portion(req, budget, plan)
                if got == 0:
                    self.manager.free(req.id)
                    req.num_computed = 0      # what was kept is gone: the whole prompt again, later
                    break
                self.waiting.popleft()
                self.running.append(req)
                budget -= got
            if plan.entries or not self.running:
                if not plan.entries and self.waiting and not self.running:
                    # the head of the queue finds no room in an empty pool: it can never run
                    req = self.waiting.popleft()
                    self._fail(req, plan, KVCapacityError('Request does not fit the GPU KV page capacity'))
                    if self.waiting:
                        continue
                return plan
            # nothing could be planned although requests are running: all of them wait for pages.
            victim = self.running[-1]
            if len(self.running) == 1:
                self._fail(victim, plan, KVCapacityError('Active KV exhausted the GPU pool'))
            else:
                self._preempt(victim, plan)

    def _undo_entry(self, req: Request, plan: StepPlan) -> None:
        """Takes a request's entry out of the plan (its pages go back when it is preempted)."""
        plan.entries = [e for e in plan.entries if e.request is not req]

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: StepPlan, sampled: dict) -> List[Request]:
        """Records the step: ``sampled`` maps request id -> (token, logprob) for entries with
        ``sample``.  Returns the requests that finished; their pages and slots are free again."""
        done = []
        for e in plan.entries:
            req = e.request
            req.num_computed = e.start + len(e.tokens)
            if e.sample:
                tok, lp = sampled[req.id]
                req.push(tok, lp)
                if req.finished or req.num_tokens >= self.max_model_len:
                    req.finish_reason = req.reason() if req.finished else "length"
                    self.finish(req)
                    done.append(req)
        return done
