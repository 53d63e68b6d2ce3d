"""Throughput measurements of the engine: decode tokens/s at a batch size after prompts of a given
length, and prefill tokens/s, timed on the device with CUDA events.

After the reference's own definitions: decode tok/s = batch * steps / time over timed steps that
follow warm-up steps (rollout/utils/bench_sym.py:24-52), prefill tok/s = tokens / time for a whole
prompt including its one row of logits (rollout/utils/bench_prefill.py:22-43); token ids are
uniform over the vocabulary (rollout/utils/bench_sym.py:26).
"""
from __future__ import annotations

from typing import Dict, List

import torch


def _random_ids(vocab: int, n: int, gen: torch.Generator) -> List[int]:
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


def fill_requests(runner, batch: int, ctx: int, seed: int = 1, chunk: int = 4096, prefix: str = "bench") -> List[str]:
    """``batch`` requests with ``ctx`` tokens each in the cache (run through the model, nothing wanted)."""
    gen = torch.Generator().manual_seed(seed)
    rids = []
    for i in range(batch):
        rid = f"{prefix}-{i}"
        runner.add_request(rid)
        ids = _random_ids(runner.vocab_size, ctx, gen)
        for a in range(0, ctx, chunk):
            runner.step([runner.reserve(rid, ids[a:a + chunk])])
        rids.append(rid)
    torch.cuda.synchronize()
    return rids


def decode_throughput(runner, batch: int, ctx: int, steps: int, warmup: int, seed: int = 1) -> Dict[str, float]:
    """Decode steps of ``batch`` requests that each hold ``ctx`` tokens: every step appends one token
    per request and computes its logits.  Device time by CUDA events around exactly ``steps`` steps."""
    rids = fill_requests(runner, batch, ctx, seed)
    gen = torch.Generator().manual_seed(seed + 1)
    toks = [_random_ids(runner.vocab_size, batch, gen) for _ in range(steps + warmup)]

    def one(k):
        entries = [runner.reserve(rid, [toks[k][i]], [0]) for i, rid in enumerate(rids)]
        return runner.step(entries)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(warmup, warmup + steps):
        one(k)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    for rid in rids:
        runner.free_request(rid)
    return {"tokens_per_s": batch * 1000.0 / ms, "ms_per_step": ms, "kv_tokens": batch * (ctx + warmup + steps // 2)}


def prefill_throughput(runner, tokens: int, iters: int, warmup: int, seed: int = 2) -> Dict[str, float]:
    """One prompt of ``tokens`` tokens in one step, with the logits of its last position."""
    gen = torch.Generator().manual_seed(seed)
    times = []
    for k in range(warmup + iters):
        ids = _random_ids(runner.vocab_size, tokens, gen)
        rid = f"prefill-{k}"
        runner.add_request(rid)
        entry = runner.reserve(rid, ids, [tokens - 1])
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([entry])
        end.record()
        torch.cuda.synchronize()
        if k >= warmup:
            times.append(start.elapsed_time(end))
        runner.free_request(rid)
    ms = sum(times) / len(times)
    return {"tokens_per_s": tokens * 1000.0 / ms, "ms": ms, "tokens": tokens}


def decode_step_bytes(cfg, batch: int, kv_tokens_total: int, dtype_bytes: int = 2) -> int:
    """Bytes a decode step has to read: every weight it uses once (the embedding rows it gathers
    are negligible and left out; a tied head is counted once, as the head), plus the cached keys and
    values of the live requests."""
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = (q + 2 * kv) * H + H * q + 2 * I * H + H * I + 2 * H + 2 * cfg.head_dim
    weights = (L * per_layer + H + cfg.vocab_size * H) * dtype_bytes
    cache = kv_tokens_total * L * 2 * kv * dtype_bytes
    return weights + cache


def prefill_flops(cfg, tokens: int, logit_rows: int = 1) -> float:
    """Floating-point operations of one whole-prompt step: matrix products of every layer, causal
    attention (half the square), and the head on ``logit_rows`` rows."""
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    linear = 2.0 * tokens * ((q + 2 * kv) * H + H * q + 2 * I * H + H * I)
    attn = 4.0 * tokens * tokens * q / 2.0
    return L * (linear + attn) + 2.0 * logit_rows * cfg.vocab_size * H
