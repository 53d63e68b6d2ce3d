"""One step's batch: the tokens it runs, packed, and the tables the kernels read.

A step is a list of entries (request, its next tokens, the places whose logits are wanted).
All entries form one packed sequence of T tokens: portions of prompts beside single decoded
tokens, cut anywhere.  The reference builds two kinds of tables for its two kinds of forward
(rollout/cache.py:282-328: ``qpos``, ``cu_q``, ragged page tables with per-page counts and start
positions); here one layout serves every mix, and because only a request's last page is partly
filled there is no per-page table: a key's page is ``block_table[segment][pos // page_size]``.

All integers travel in one pinned host buffer and one device buffer, one copy per step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # indices into ``tokens`` whose logits are wanted
    start: int = -1                   # position of tokens[0]; filled when the cache makes room


@dataclass
class HostBatch:
    """The step's tables as numpy int32 arrays."""
    num_tokens: int
    num_segments: int
    num_want: int
    tokens: np.ndarray        # [T]
    pos: np.ndarray           # [T] absolute position of each token
    tok_seg: np.ndarray       # [T] segment (entry) index of each token
    seg_slot: np.ndarray      # [n] the request's slot
    cu_q: np.ndarray          # [n+1] first token row of each segment
    seg_pos0: np.ndarray      # [n] position of the segment's first token
    seg_kv_len: np.ndarray    # [n] keys visible to the segment's last token
    want_rows: np.ndarray     # [n_want] token rows whose logits are wanted
    decode_segs: np.ndarray   # segments of one token
    num_multi: int = 0        # segments of several tokens
    # what the model's parts asked for (parts.base.Tiling): name -> [blocks, 2], (segment, first row within
    # it) of every block of rows of the segments of several tokens
    tiles: Dict[str, np.ndarray] = field(default_factory=dict)
    block_tables: List[np.ndarray] = field(default_factory=list)   # per group [n, blocks]
    rids: List[Hashable] = field(default_factory=list)


def build_host_batch(entries: Sequence[StepEntry], manager, vocab_size: Optional[int] = None,
                     max_positions: Optional[int] = None, tilings: Optional[Dict[str, object]] = None) -> HostBatch:
    """Packs entries whose cache room was already made (``entry.start`` set by ``manager.append``).
    ``tilings``: name -> parts.base.Tiling, the tables of row blocks that the model's parts read."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    n = len(entries)
    lens = [len(e.tokens) for e in entries]
    if min(lens) <= 0:
        raise ValueError("every entry of a step brings at least one token")
    rids = [e.rid for e in entries]
    if len(set(rids)) != n:
        raise ValueError("a request appears once in a step")
    T = sum(lens)
    tokens = np.empty(T, np.int32)
    pos = np.empty(T, np.int32)
    tok_seg = np.empty(T, np.int32)
    cu_q = np.zeros(n + 1, np.int32)
    seg_slot = np.empty(n, np.int32)
    seg_pos0 = np.empty(n, np.int32)
    seg_kv_len = np.empty(n, np.int32)
    want_rows: List[int] = []
    decode_segs: List[int] = []
    multi: List[int] = []
    row = 0
    for i, e in enumerate(entries):
        L = lens[i]
        if e.start < 0 or e.start + L != manager.length(e.rid):
            raise ValueError(f"entry of request {e.rid!r}: cache room was not made for these tokens")
        tokens[row:row + L] = np.asarray(e.tokens, dtype=np.int64)
        pos[row:row + L] = np.arange(e.start, e.start + L)
        tok_seg[row:row + L] = i
        cu_q[i + 1] = row + L
        seg_slot[i] = manager.slot(e.rid)
        seg_pos0[i] = e.start
        seg_kv_len[i] = e.start + L
        for w in e.want:
            if not (0 <= w < L):
                raise ValueError(f"want index {w} is outside the entry's {L} tokens")
            want_rows.append(row + w)
        (decode_segs if L == 1 else multi).append(i)
        row += L
    if vocab_size is not None and (tokens.min() < 0 or tokens.max() >= vocab_size):
        raise ValueError(f"token ids must lie in [0, {vocab_size})")
    if max_positions is not None and int(seg_kv_len.max()) > max_positions:
        raise ValueError(f"a request would reach {int(seg_kv_len.max())} tokens; the engine was set up for {max_positions}")
    tiles = {}
    for name, tiling in (tilings or {}).items():
        blocks = [(i, r0) for i in multi for r0 in range(0, lens[i], tiling.rows)]
        if tiling.heaviest_first:        # a block's work grows with the position of its rows
            blocks.sort(key=lambda sr: -(int(seg_pos0[sr[0]]) + sr[1]))
        tiles[name] = np.asarray(blocks, np.int32).reshape(-1, 2)
    tables = []
    for g, spec in enumerate(manager.groups):
        blocks = max((int(seg_kv_len[i]) + spec.page_size - 1) // spec.page_size for i in range(n))
        bt = np.full((n, blocks), -1, np.int32)
        for i, e in enumerate(entries):
            row_blocks = manager.block_table(e.rid, g)
            k = min(len(row_blocks), blocks)
            bt[i, :k] = row_blocks[:k]
        tables.append(bt)
    return HostBatch(
        num_tokens=T, num_segments=n, num_want=len(want_rows), tokens=tokens, pos=pos, tok_seg=tok_seg,
        seg_slot=seg_slot, cu_q=cu_q, seg_pos0=seg_pos0, seg_kv_len=seg_kv_len,
        want_rows=np.asarray(want_rows, np.int32), decode_segs=np.asarray(decode_segs, np.int32),
        num_multi=len(multi), tiles=tiles, block_tables=tables, rids=rids)


class StepBatch:
    """The tables on the device, as views of one int32 buffer."""

    _FIELDS = ("tokens", "pos", "tok_seg", "seg_slot", "cu_q", "seg_pos0", "seg_kv_len", "want_rows", "decode_segs")

    def __init__(self, host: HostBatch, device, staging: "BatchStaging"):
        self.host = host
        self.scratch = {}                    # work buffers and memoised choices of this step (LayerContext.buffer)
        self.num_tokens = host.num_tokens
        self.num_segments = host.num_segments
        self.num_want = host.num_want
        self.variant = {}                    # nothing is fixed beforehand: every part works its launches out from the host tables
        tile_names = list(host.tiles)
        arrays = ([getattr(host, f).reshape(-1) for f in self._FIELDS] + [host.tiles[n].reshape(-1) for n in tile_names]
                  + [bt.reshape(-1) for bt in host.block_tables])
        offsets, total = [], 0
        for a in arrays:
            offsets.append(total)
            total += (a.size + 3) // 4 * 4          # keep every table 16-byte aligned
        pinned, dev = staging.buffers(max(total, 4))
        hv = pinned.numpy()
        for a, off in zip(arrays, offsets):
            hv[off:off + a.size] = a
        dev[:total].copy_(pinned[:total], non_blocking=True)
        staging.mark()
        views = [dev[off:off + a.size] for a, off in zip(arrays, offsets)]
        for f, v in zip(self._FIELDS, views):
            setattr(self, f, v)
        k = len(self._FIELDS)
        self.tiles = {n: v.view(-1, 2) for n, v in zip(tile_names, views[k:k + len(tile_names)])}
        self.block_tables = [v.view(bt.shape) for v, bt in zip(views[k + len(tile_names):], host.block_tables)]


class BatchStaging:
    """Pinned host buffers and device buffers for the step tables.

    A step's host buffer must stay untouched until its copy has run, so buffers rotate: a buffer
    is reused only after the copy that read it was seen to finish."""

    def __init__(self, device, depth: int = 4):
        self.device = torch.device(device)
        self._slots = [None] * depth
        self._next = 0

    def buffers(self, n_ints: int):
        i = self._next
        self._next = (self._next + 1) % len(self._slots)
        slot = self._slots[i]
        if slot is not None:
            slot[2].synchronize()                   # the copy that last used this pair is done
        if slot is None or slot[0].numel() < n_ints:
            cap = max(4096, 1 << (n_ints - 1).bit_length())
            pinned = torch.empty(cap, dtype=torch.int32).pin_memory()
            dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            slot = [pinned, dev, None]
        ev = torch.cuda.Event()
        slot[2] = ev
        self._slots[i] = slot
        return slot[0], slot[1]

    def mark(self):
        """Records, on the current stream, the point after which the latest buffers are free again."""
        i = (self._next - 1) % len(self._slots)
        if self._slots[i] is not None:
            self._slots[i][2].record()


class _StaticHost:
    """What the kernels' dispatch looks at on the host, for a captured decode step of n tokens."""

    def __init__(self, n: int, tilings=None):
        self.num_tokens = self.num_segments = self.num_want = n
        self.decode_segs = np.arange(n, dtype=np.int32)
        self.num_multi = 0
        self.tiles = {name: np.zeros((0, 2), np.int32) for name in (tilings or {})}
        self.cu_q = np.arange(n + 1, dtype=np.int32)
        self.seg_slot = np.zeros(n, np.int32)
        self.seg_kv_len = np.ones(n, np.int32)


class StaticDecodeBatch:
    """Tables of a step of exactly ``n`` single decoded tokens at fixed device addresses, so that the
    step can be captured in a CUDA graph once and replayed with new contents.  The block tables
    have a fixed width (``max_blocks`` of each group); ``variant`` holds what the model's parts fixed
    beforehand because a captured launch cannot change it (``Part.graph_variant``).  A step of fewer than ``n`` tokens fills
    the first rows; the rows behind them are padding: one key, no page (nothing of the cache is read or
    written), and the state slot ``pad_slot`` that belongs to no request."""

    def __init__(self, n: int, max_blocks: Sequence[int], device, variant: Optional[dict] = None, pad_slot: int = 0,
                 tilings=None):
        self.n = n
        self.pad_slot = pad_slot
        self.num_tokens = self.num_segments = self.num_want = n
        self.variant = dict(variant or {})
        self.scratch = {}                    # work buffers of the captured step: they live as long as the graph
        self.host = _StaticHost(n, tilings)
        self._max_blocks = list(max_blocks)
        sizes = [n, n, n, n, n + 1, n, n, n, n] + [n * b for b in max_blocks]
        offs, total = [], 0
        for sz in sizes:
            offs.append(total)
            total += (sz + 3) // 4 * 4
        self._pinned = torch.zeros(total, dtype=torch.int32).pin_memory()
        self._dev = torch.zeros(total, dtype=torch.int32, device=device)
        hv = self._pinned.numpy()
        names = ("tokens", "pos", "tok_seg", "seg_slot", "cu_q", "seg_pos0", "seg_kv_len", "want_rows", "decode_segs")
        self._h = {}
        for name, off, sz in zip(names, offs, sizes):
            self._h[name] = hv[off:off + sz]
            setattr(self, name, self._dev[off:off + sz])
        self._h_bt, self.block_tables = [], []
        for b, off in zip(max_blocks, offs[len(names):]):
            self._h_bt.append(hv[off:off + n * b].reshape(n, b))
            self.block_tables.append(self._dev[off:off + n * b].view(n, b))
        self.tiles = {name: torch.zeros((0, 2), dtype=torch.int32, device=device) for name in (tilings or {})}
        self._h["tok_seg"][:] = np.arange(n)
        self._h["cu_q"][:] = np.arange(n + 1)
        self._h["want_rows"][:] = np.arange(n)
        self._h["decode_segs"][:] = np.arange(n)
        self._h["seg_kv_len"][:] = 1
        for bt in self._h_bt:
            bt[:] = -1                       # before the first fill: no page is read or written
        self._event = torch.cuda.Event()
        self.upload()

    def fill(self, host: HostBatch) -> None:
        """Takes the contents of a packed decode step of up to n tokens; the rows behind them are padding."""
        m = host.num_tokens
        assert m <= self.n and host.num_segments == m
        self._event.synchronize()            # the copy that last read the pinned buffer is done
        for name in ("tokens", "pos", "seg_slot", "seg_pos0", "seg_kv_len"):
            self._h[name][:m] = getattr(host, name)
        if m < self.n:
            for name, value in (("tokens", 0), ("pos", 0), ("seg_slot", self.pad_slot), ("seg_pos0", 0), ("seg_kv_len", 1)):
                self._h[name][m:] = value
        for dst, src in zip(self._h_bt, host.block_tables):
            if src.shape[1] > dst.shape[1]:
                raise ValueError("a request is longer than the captured block table")
            dst[:m, :src.shape[1]] = src     # what lies behind a row's pages is never read: its length bounds the keys
            if m < self.n:
                dst[m:] = -1
        self.host.seg_kv_len = self._h["seg_kv_len"]
        self.upload()

    def upload(self) -> None:
        self._dev.copy_(self._pinned, non_blocking=True)
        self._event.record()
