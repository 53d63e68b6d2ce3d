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


# Kernel names of a decode step by kind, after the reference's table (rollout/utils/prof_graph.py:27-43): its
# kinds, the names of this engine's kernels (and of the library's matrix products).
PROFILE_BUCKETS = [
    ("decode_attn", ["attn_decode", "attn_combine"]),
    ("prefill_attn", ["attn_prefill", "attention_simt", "tc5_merge"]),
    ("gemm/matmul", ["gemm", "nvjet", "cutlass", "cublas", "matmul"]),
    ("rmsnorm", ["rmsnorm", "norm_rows"]),
    ("rope", ["rope"]),
    ("elementwise", ["swiglu", "embedding", "elementwise", "copy", "fill"]),
    ("softmax/sample", ["sample", "argmax"]),
]


def profile_bucket(kernel_name: str) -> str:
    low = kernel_name.lower()
    for label, keys in PROFILE_BUCKETS:
        if any(k in low for k in keys):
            return label
    return "other"


def profile_decode(runner, batch: int, ctx: int, steps: int, warmup: int, seed: int = 1) -> Dict[str, object]:
    """Where the device time of decode steps goes, by kind of kernel: the table that the reference prints with
    ``torch.profiler`` over graph-replayed decode steps (rollout/utils/prof_graph.py:76-107).  CUDA activity only;
    times are each kernel's own device time summed, so kernels that overlap count twice and the sum may exceed
    the step's wall time."""
    from collections import defaultdict
    from torch.profiler import ProfilerActivity, profile
    rids = fill_requests(runner, batch, ctx, seed, prefix="prof")
    gen = torch.Generator().manual_seed(seed + 1)
    toks = [_random_ids(runner.vocab_size, batch, gen) for _ in range(steps + warmup)]

    def one(k):
        return runner.step([runner.reserve(rid, [toks[k][i]], [0]) for i, rid in enumerate(rids)])

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA], record_shapes=False) as prof:
        for k in range(warmup, warmup + steps):
            one(k)
        torch.cuda.synchronize()
    for rid in rids:
        runner.free_request(rid)
    bucket, count, per_kernel = defaultdict(float), defaultdict(int), defaultdict(float)
    for e in prof.key_averages():
        us = getattr(e, "self_device_time_total", 0) or getattr(e, "self_cuda_time_total", 0)
        if us <= 0:
            continue
        b = profile_bucket(e.key)
        bucket[b] += us
        count[b] += e.count
        per_kernel[e.key] += us
    total = sum(bucket.values()) or 1.0
    return {"batch": batch, "ctx": ctx, "steps": steps, "gpu_ms_per_step": total / 1e3 / steps,
            "buckets": [{"bucket": b, "ms_per_step": us / 1e3 / steps, "share": us / total, "kernels_per_step": count[b] / steps}
                        for b, us in sorted(bucket.items(), key=lambda kv: -kv[1])],
            "top_kernels": [{"kernel": k[:80], "ms_per_step": us / 1e3 / steps, "share": us / total}
                            for k, us in sorted(per_kernel.items(), key=lambda kv: -kv[1])[:12]]}


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


# ------------------------------------------------------------------------------- single kernels

def _paged_case(batch: int, ctx: int, q_len: int, heads: int, kv_heads: int, head_dim: int, page: int, device):
    """Random bfloat16 pools and the tables of ``batch`` requests that hold ``ctx`` keys each and
    bring ``q_len`` new tokens (already in the cache)."""
    blocks = (ctx + page - 1) // page
    n_pages = batch * blocks
    g = torch.Generator(device=device).manual_seed(0)
    k_pool = torch.randn((n_pages, kv_heads, page, head_dim), generator=g, device=device, dtype=torch.float32).bfloat16()
    v_pool = torch.randn((n_pages, kv_heads, page, head_dim), generator=g, device=device, dtype=torch.float32).bfloat16()
    perm = torch.randperm(n_pages, generator=g, device=device).to(torch.int32).view(batch, blocks)
    T = batch * q_len
    qkv = torch.randn((T, (heads + 2 * kv_heads) * head_dim), generator=g, device=device, dtype=torch.float32).bfloat16()
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=device)
    cu_q = i32([i * q_len for i in range(batch + 1)])
    seg_pos0 = i32([ctx - q_len] * batch)
    seg_kv_len = i32([ctx] * batch)
    return qkv, k_pool, v_pool, perm.contiguous(), cu_q, seg_pos0, seg_kv_len


def _time_kernels(fns, iters: int, warmup: int) -> float:
    """Mean device milliseconds of one launch: every pass runs all of ``fns`` back to back between two
    CUDA events, so launch overhead is hidden behind the queue as in a real step.  The callers make
    ``fns`` read different buffers whose total size exceeds L2, so every launch reads from HBM."""
    for _ in range(warmup):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()            # one pass as a graph: no host time between the launches
    with torch.cuda.graph(graph):
        for fn in fns:
            fn()
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / (iters * len(fns))


def _copies_beyond_l2(nbytes: int, l2_bytes: int = 126 << 20) -> int:
    return max(2, min(64, (2 * l2_bytes + nbytes - 1) // max(1, nbytes)))


def kernel_attention_decode(batch=64, ctx=2048, heads=32, kv_heads=8, head_dim=128, page=16, splits=0,
                            iters=10, warmup=3) -> Dict[str, float]:
    """The split-KV decode attention kernel alone: device time and the bandwidth of the keys and values it reads."""
    from .ext import ops
    dev = torch.device("cuda:0")
    nbytes = 2 * batch * ctx * kv_heads * head_dim * 2
    group = heads // kv_heads
    n = splits or ops.decode_splits(batch * kv_heads * ((group + 15) // 16), ctx)
    segs = torch.arange(batch, dtype=torch.int32, device=dev)
    fns = []
    for _ in range(_copies_beyond_l2(nbytes)):
        qkv, k_pool, v_pool, bt, cu_q, _, seg_kv_len = _paged_case(batch, ctx, 1, heads, kv_heads, head_dim, page, dev)
        out = torch.empty((batch, heads * head_dim), dtype=torch.bfloat16, device=dev)
        fns.append(lambda a=(qkv, k_pool, v_pool, cu_q, seg_kv_len, bt, out): ops.attention_decode_mma(
            a[0], a[1], a[2], segs, a[3], a[4], a[5], page, a[6], heads, kv_heads, head_dim, head_dim ** -0.5, 0, n))
    ms = _time_kernels(fns, iters, warmup)
    return {"kernel": "attention_decode", "batch": batch, "ctx": ctx, "splits": n, "ms": ms,
            "GBps": nbytes / ms / 1e6}


def kernel_attention_prefill(batch=1, ctx=2048, q_len=2048, heads=32, kv_heads=8, head_dim=128, page=16,
                             iters=10, warmup=3, impl=0, splits=0) -> Dict[str, float]:
    """The prefill attention kernel alone: device time and causal TFLOP/s.
    ``impl`` 0: the tcgen05 kernel (head sizes 64 and 128); 1: the mma.sync kernel.
    ``splits``: ways the tcgen05 kernel splits the keys (0: the engine's choice for this many CTAs)."""
    from .ext import ops
    dev = torch.device("cuda:0")
    qkv, k_pool, v_pool, bt, cu_q, seg_pos0, _ = _paged_case(batch, ctx, q_len, heads, kv_heads, head_dim, page, dev)
    out = torch.empty((batch * q_len, heads * head_dim), dtype=torch.bfloat16, device=dev)
    rows = 64 if impl else ops.TC5_TILE_ROWS
    tiles = torch.tensor([(i, r) for i in range(batch) for r in range(0, q_len, rows)], dtype=torch.int32, device=dev)
    kernel = ops.attention_prefill_mma if impl else ops.attention_prefill_tc5
    splits = splits or ops.prefill_splits(int(tiles.shape[0]) * heads, ctx)
    more = {} if impl else {"num_splits": splits, "held": {}}
    fn = lambda: kernel(qkv, k_pool, v_pool, tiles, cu_q, seg_pos0, bt, page, out, heads,
                        kv_heads, head_dim, head_dim ** -0.5, 0, **more)
    ms = _time_kernels([fn], iters, warmup)
    flops = 4.0 * batch * heads * head_dim * (q_len * (ctx - q_len) + q_len * q_len / 2.0)
    return {"kernel": "attention_prefill_mma" if impl else "attention_prefill_tc5", "batch": batch, "ctx": ctx, "q_len": q_len, "splits": 1 if impl else splits,
            "ctas": int(tiles.shape[0]) * heads, "ms": ms, "TFLOPs": flops / ms / 1e9}


def kernel_gemm(M=8, N=4096, K=4096, iters=10, warmup=3, out_f32=0, impl=0) -> Dict[str, float]:
    """A bfloat16 matrix product alone: device time, weight bandwidth and TFLOP/s.
    ``impl`` 0: ``ops.linear`` (the engine's choice); 1: the tcgen05 kernel; 2: cuBLAS (``torch.mm``);
    3: the tcgen05 weight-streaming kernel; 4: the mma.sync weight-streaming kernel; 5: the tcgen05 kernel on
    256 x 256 tiles by pairs of CTAs."""
    from .ext import ops
    dev = torch.device("cuda:0")
    fns = []
    for _ in range(_copies_beyond_l2(N * K * 2)):
        x = torch.randn((M, K), device=dev).bfloat16()
        w = torch.randn((N, K), device=dev).bfloat16()
        out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
        if impl == 1:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(*a))
        elif impl == 2:
            fns.append(lambda a=(x, w, out): torch.mm(a[0], a[1].t(), out=a[2]))
        elif impl == 3:
            fns.append(lambda a=(x, w, out): ops.gemm_stream(*a))
        elif impl == 4:
            fns.append(lambda a=(x, w, out): ops.gemm_skinny(*a))
        elif impl == 5:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(*a, pair=True))
        else:
            fns.append(lambda a=(x, w, out): ops.linear(*a))
    ms = _time_kernels(fns, iters, warmup)
    return {"kernel": ("linear", "gemm_tc5", "cublas", "gemm_stream", "gemm_skinny", "gemm_tc5_pair")[impl], "M": M, "N": N, "K": K, "ms": ms, "GBps": N * K * 2 / ms / 1e6,
            "TFLOPs": 2.0 * M * N * K / ms / 1e9}


def kernel_elementwise(rows=2048, hidden=4096, intermediate=12288, iters=10, warmup=3) -> Dict[str, object]:
    """The residual add + RMSNorm kernel and the SwiGLU kernel alone, over buffers larger than L2: device time and
    the bandwidth of what each must read and write (norm: stream in and out in float32, delta in, normed rows out;
    SwiGLU: [rows, 2 I] in, [rows, I] out)."""
    from .ext import ops
    dev = torch.device("cuda:0")
    w = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    norm_bytes = rows * hidden * (4 + 4 + 2 + 2)
    fns = []
    for _ in range(_copies_beyond_l2(norm_bytes)):
        stream = torch.randn(rows, hidden, device=dev)
        delta = torch.randn(rows, hidden, device=dev).bfloat16()
        out = torch.empty(rows, hidden, device=dev, dtype=torch.bfloat16)
        fns.append(lambda a=(stream, delta, out): ops.add_rmsnorm(a[0], a[1], w, 1e-6, a[2]))
    ms_norm = _time_kernels(fns, iters, warmup)
    act_bytes = rows * intermediate * 3 * 2
    fns = []
    for _ in range(_copies_beyond_l2(act_bytes)):
        gu = torch.randn(rows, 2 * intermediate, device=dev).bfloat16()
        out = torch.empty(rows, intermediate, device=dev, dtype=torch.bfloat16)
        fns.append(lambda a=(gu, out): ops.swiglu(a[0], a[1], 8))
    ms_act = _time_kernels(fns, iters, warmup)
    return {"rows": rows, "add_rmsnorm": {"ms": ms_norm, "GBps": norm_bytes / ms_norm / 1e6},
            "swiglu": {"ms": ms_act, "GBps": act_bytes / ms_act / 1e6}}


def kernel_gated(M=2048, I=12288, K=4096, iters=10, warmup=3, impl=0) -> Dict[str, float]:
    """The gated feed-forward product out = silu(x Wg^T) * (x Wu^T) alone.  ``impl`` 0: the engine's
    choice (``ops.gated_linear``); 1: the tcgen05 kernel with the SwiGLU epilogue; 2: cuBLAS + the SwiGLU kernel;
    3: the tcgen05 kernel by pairs of CTAs with the SwiGLU epilogue."""
    from .ext import ops
    dev = torch.device("cuda:0")
    fns = []
    for _ in range(_copies_beyond_l2(2 * I * K * 2)):
        x = torch.randn((M, K), device=dev).bfloat16()
        w = torch.randn((2 * I, K), device=dev).bfloat16()
        out = torch.empty((M, I), dtype=torch.bfloat16, device=dev)
        gu = torch.empty((M, 2 * I), dtype=torch.bfloat16, device=dev)
        if impl == 1:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(a[0], a[1], a[2], gated=True))
        elif impl == 3:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(a[0], a[1], a[2], gated=True, pair=True))
        elif impl == 2:
            def two(a=(x, w, out, gu)):
                torch.mm(a[0], a[1].t(), out=a[3])
                ops.swiglu(a[3], a[2], 8)
            fns.append(two)
        else:
            fns.append(lambda a=(x, w, out): ops.gated_linear(a[0], a[1], a[2], 8))
    ms = _time_kernels(fns, iters, warmup)
    return {"kernel": ("gated_linear", "gemm_tc5_gated", "cublas+swiglu", "gemm_tc5_pair_gated")[impl], "M": M, "I": I, "K": K, "ms": ms,
            "TFLOPs": 4.0 * M * I * K / ms / 1e9}


# ------------------------------------------------------------------------------- named workloads through the engine

WORKLOADS = {
    # 64 requests with prompt lengths uniform in [16, 4096], prompts in portions of 512 tokens beside decodes
    "0.6b-mixed": dict(
        model=dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                   num_attention_heads=16, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0,
                   rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960),
        seed=5, requests=64, prompt=(16, 4096), new=128, chunk=512, max_reside=64, ctx=8192),
    # 16 requests with 2,048-token prompts, then 256 decoded tokens each
    "32b": dict(
        model=dict(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                   num_attention_heads=64, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0,
                   rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960),
        seed=6, requests=16, prompt=(2048, 2048), new=256, chunk=8192, max_reside=16, ctx=8192),
}


def run_workload(name: str, layers: int = 0, new: int = 0) -> Dict[str, object]:
    """One of the named workloads through ``Engine.generate`` (scheduler, portions, decode, sampling off: greedy):
    wall time, tokens per second of the whole job and of its decode steps.  ``layers`` / ``new``: fewer layers or
    fewer new tokens than the workload names, where time needs it (both are reported)."""
    import time
    from .config.model_config import Qwen3Config
    from .engine.config import EngineConfig
    from .engine.engine import Engine
    from .engine.request import Request
    from .engine.runner import ModelRunner
    w = WORKLOADS[name]
    raw = dict(w["model"])
    full_layers = raw["num_hidden_layers"]
    if layers:
        raw["num_hidden_layers"] = layers
    cfg = Qwen3Config.from_dict(raw)
    n_new = new or w["new"]
    gen = torch.Generator().manual_seed(w["seed"])
    lo, hi = w["prompt"]
    lens = [int(torch.randint(lo, hi + 1, (1,), generator=gen)) for _ in range(w["requests"])]
    pool = sum((n + n_new + 63) // 64 * 64 for n in lens) + 1024
    ecfg = EngineConfig(max_token=pool, max_reside=w["max_reside"], page_size=16, prefill_chunk=w["chunk"], dtype="bfloat16",
                        max_model_len=w["ctx"], use_cuda_graph=True, capture_at_start=True, seed=w["seed"])
    runner = ModelRunner.from_random(cfg, ecfg, seed=w["seed"])
    engine = Engine(runner)
    reqs = [Request(f"w{i}", _random_ids(cfg.vocab_size, n, gen), max_new_tokens=n_new, temperature=0.0) for i, n in enumerate(lens)]
    # start-up, untimed: the engine has captured its decode graphs (as the reference's build_graph does);
    # one short request goes through prefill and a few decode steps
    engine.generate([_random_ids(cfg.vocab_size, 64, gen)], max_new_tokens=4, temperature=0.0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = engine.generate(reqs)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = engine.stats()
    return {"workload": name, "layers": cfg.num_hidden_layers, "full_layers": full_layers, "requests": len(reqs),
            "prompt_tokens": sum(lens), "new_tokens": sum(r.num_tokens for r in out), "seconds": round(dt, 3),
            "tokens_per_s": round((sum(lens) + sum(r.num_tokens for r in out)) / dt, 1),
            "generated_per_s": round(sum(r.num_tokens for r in out) / dt, 1),
            "steps": st["steps"], "preemptions": st["preemptions"], "decode_tps": st.get("decode_tps"),
            "prefill_tps": st.get("prefill_tps"), "decode_graphs": len(runner._graphs)}
