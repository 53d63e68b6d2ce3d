"""The reference arm of bench.py: wenhaoli-xmu/ReTurn's own rollout engine, unmodified, on the same
metric, model shape and GPU as the engine of this repository.

What runs is the reference's code from a plain copy of its tree (``baseline/_ref``, not tracked):
``rollout.monkey_patch.qwen3.QwenModel(container, max_token, max_reside)``, ``build_graph()``, then
``Model.prefill`` and ``Model.decode`` driven by duck-typed requests, exactly as its own scripts do
(rollout/utils/bench_sym.py:24-52, rollout/utils/bench_prefill.py:22-43,
rollout/utils/check_correctness.py:10-39).  Its Triton kernels are compiled by Triton for the GPU
they run on; its matrix products are ``F.linear`` (cuBLAS).  Nothing of ``return_b200`` is imported
here and none of its libraries is loaded.

The reference keeps a Hugging Face model object as the container of its weights and replaces every
forward (rollout/monkey_patch/qwen3.py:88-106).  The container here is a plain ``nn.Module`` tree
with the attribute names the reference touches and random bfloat16 weights made on the device
(N(0, 0.02) matrices, 1 + N(0, 0.1) norm weights): no forward of it ever runs, so the timed code is
the reference's alone.  ``scaling`` and ``inv_freq`` follow the reference's own fallbacks
(rollout/attention.py:195, rollout/utils/test_decode.py:14-17).  Stock settings stay: page 64,
prefill chunk 8,192, CUDA graphs for every batch size up to ``max_reside``.

``--kernels`` times the reference's four Triton kernels alone at the shapes of this model
(``flash_prefill`` rollout/attention.py:159-198, ``flash_decode`` :549-591, ``rms_norm``
rollout/fused.py:48-56, ``silu_and_mul`` :103-127) and prints one JSON line per kernel.
"""
from __future__ import annotations

import json
import os
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))


def find_reference():
    """The reference's tree: the copy that travels with this repository."""
    root = os.path.join(HERE, "_ref")
    if os.path.isfile(os.path.join(root, "rollout", "monkey_patch", "qwen3.py")):
        return root
    return None


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


# ------------------------------------------------------------------------------- the weight container

def make_container(shape: dict, device, seed: int):
    import torch
    from torch import nn

    c = types.SimpleNamespace(**shape)

    class Qwen3RMSNorm(nn.Module):            # the class name is what the reference's patch looks for
        def __init__(self, n):
            super().__init__()
            self.weight = nn.Parameter(torch.empty(n))
            self.variance_epsilon = c.rms_norm_eps

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            H, D = c.hidden_size, c.head_dim
            self.head_dim, self.scaling, self.sliding_window = D, D ** -0.5, None
            self.q_proj = nn.Linear(H, c.num_attention_heads * D, bias=False)
            self.k_proj = nn.Linear(H, c.num_key_value_heads * D, bias=False)
            self.v_proj = nn.Linear(H, c.num_key_value_heads * D, bias=False)
            self.o_proj = nn.Linear(c.num_attention_heads * D, H, bias=False)
            self.q_norm, self.k_norm = Qwen3RMSNorm(D), Qwen3RMSNorm(D)

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
            self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
            self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=False)

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn, self.mlp = Attn(), MLP()
            self.input_layernorm = Qwen3RMSNorm(c.hidden_size)
            self.post_attention_layernorm = Qwen3RMSNorm(c.hidden_size)

    class Rotary(nn.Module):
        def __init__(self):
            super().__init__()
            half = c.head_dim // 2
            self.inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, half, dtype=torch.float32) / half))
            self.attention_scaling = 1.0

    class Inner(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size)
            self.layers = nn.ModuleList([Layer() for _ in range(c.num_hidden_layers)])
            self.norm = Qwen3RMSNorm(c.hidden_size)
            self.rotary_emb = Rotary()

    class Container(nn.Module):
        def __init__(self):
            super().__init__()
            self.config = c
            self.model = Inner()
            self.lm_head = nn.Linear(c.hidden_size, c.vocab_size, bias=False)

    # parameters are born on the device in bfloat16 and never pass through the host
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            import torch.nn.init as init
            skip = lambda t, *a, **k: t             # the default initialisers would run over 8 G elements twice
            saved = init.kaiming_uniform_, init.normal_
            init.kaiming_uniform_ = init.normal_ = skip
            try:
                box = Container()
            finally:
                init.kaiming_uniform_, init.normal_ = saved
    finally:
        torch.set_default_dtype(old)
    g = torch.Generator(device=device).manual_seed(seed)
    with torch.no_grad():
        for name, p in box.named_parameters():
            if p.dim() == 1:
                p.normal_(0.0, 0.1, generator=g).add_(1.0)
            else:
                p.normal_(0.0, 0.02, generator=g)
    if c.tie_word_embeddings:
        box.lm_head.weight = box.model.embed_tokens.weight
    return box.eval()


class FakeReq:                                # after rollout/utils/check_correctness.py:10-19
    temperature, top_p, top_k = 0.0, 1.0, 0
    subs, swap = (), ()
    ephem_at = swap_at = None
    max_new_tokens = 1 << 30

    def __init__(self, rid, ids):
        self.id, self.prompt_ids, self.split_ids, self.output = rid, list(ids), [], []

    @property
    def last_token(self):
        return self.output[-1]


# ------------------------------------------------------------------------------- the engine's metric

def _decode(torch, model, vocab, batch, ctx, steps, warmup, dev, seed):
    """After rollout/utils/bench_sym.py:24-52: prompts of ``ctx`` random tokens, warm-up decode steps, then
    exactly ``steps`` timed steps.  Device time by CUDA events, wall time beside it; every step brings its
    tokens from the host and returns the sampled tokens to the host (``Model.decode`` does both)."""
    g = torch.Generator().manual_seed(seed)
    kv = model.get_kv_cache()
    reqs = [FakeReq(("bench", batch, i), torch.randint(0, vocab, (ctx,), generator=g).tolist()) for i in range(batch)]
    for r in reqs:
        kv.alloc(r.id)
    for r, t in zip(reqs, model.prefill(reqs)):
        r.output.append(t)
    for _ in range(warmup):
        for r, t in zip(reqs, model.decode(reqs)):
            r.output.append(t)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        for r, t in zip(reqs, model.decode(reqs)):
            r.output.append(t)
    e1.record()
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    ms = e0.elapsed_time(e1) / steps
    for r in reqs:
        kv.free(r.id)
    return {"ms_per_step": ms, "tokens_per_s": batch * 1000.0 / ms, "e2e_tokens_per_s": batch * steps / wall}


def _prefill(torch, model, vocab, tokens, iters, warmup, dev, seed):
    """After rollout/utils/bench_prefill.py:22-43: one prompt, one call of ``Model.prefill``."""
    g = torch.Generator().manual_seed(seed)
    kv = model.get_kv_cache()
    times = []
    for k in range(warmup + iters):
        r = FakeReq(("pf", k), torch.randint(0, vocab, (tokens,), generator=g).tolist())
        kv.alloc(r.id)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        model.prefill([r])
        e1.record()
        torch.cuda.synchronize(dev)
        if k >= warmup:
            times.append(e0.elapsed_time(e1))
        kv.free(r.id)
    ms = sum(times) / len(times)
    return {"ms": ms, "tokens_per_s": tokens * 1000.0 / ms}


def run(args, shape: dict, prompt_len: int, full_layers: int, peaks, clock_sampler_cls) -> int:
    """Prints the bench line of the reference arm (or its ``unavailable`` line) and returns the exit code."""
    ref = find_reference()
    if ref is None:
        return unavailable("no copy of the reference under baseline/_ref (cp -r of its tree); nothing to run")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device is visible")
        import triton                                         # noqa: F401  (the reference's kernels are Triton)
    except Exception as e:                                    # noqa: BLE001
        return unavailable(f"import failed: {type(e).__name__}: {e}")
    sys.path.insert(0, ref)
    try:
        import rollout.constant as rconst
        import rollout.monkey_patch.qwen3 as rq3
    except Exception as e:                                    # noqa: BLE001
        return unavailable(f"the reference's rollout package does not import here: {type(e).__name__}: {e}")

    dev = "cuda:0"
    torch.cuda.set_device(0)
    W, K = max(3, args.warmup), max(1, args.steps)
    big = 64
    shape = dict(shape, num_hidden_layers=args.layers)
    if getattr(args, "kernels", False):
        return kernels(torch, rq3, shape, dev)
    page = rconst.PAGE_SIZE
    max_token = big * (prompt_len + 2 * W + 2 * K + 8 + 2 * page)        # rollout/utils/bench_sym.py:69
    t0 = time.time()
    try:
        box = make_container(shape, dev, seed=4)
        model = rq3.QwenModel(box, max_token=max_token, max_reside=big, device=dev)
        model.build_graph()
        torch.cuda.synchronize()
    except Exception as e:                                    # noqa: BLE001
        return unavailable(f"the reference failed to start on this GPU: {type(e).__name__}: {e}")
    build_s = time.time() - t0
    vocab = shape["vocab_size"]
    hbm_gbs, bf16_tflops, peak_src = peaks
    clocks = clock_sampler_cls()
    clocks.start()
    try:
        pf = _prefill(torch, model, vocab, prompt_len, iters=5, warmup=3, dev=dev, seed=2)
        main_r = _decode(torch, model, vocab, args.batch, prompt_len, K, W, dev, seed=1)
        pts = {}
        for b in (1, 64):
            r = _decode(torch, model, vocab, b, prompt_len, max(8, K // 2), W, dev, seed=1)
            pts[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
            pts[f"decode_b{b}_ms"] = round(r["ms_per_step"], 3)
    except Exception as e:                                    # noqa: BLE001
        clocks.stop()
        return unavailable(f"the reference failed while running: {type(e).__name__}: {e}")
    clk = clocks.stop()
    ms = main_r["ms_per_step"]
    H, I, L = shape["hidden_size"], shape["intermediate_size"], shape["num_hidden_layers"]
    q, kvd = shape["num_attention_heads"] * shape["head_dim"], shape["num_key_value_heads"] * shape["head_dim"]
    per_layer = (q + 2 * kvd) * H + H * q + 2 * I * H + H * I + 2 * H + 2 * shape["head_dim"]
    weights = (L * per_layer + H + vocab * H) * 2
    cache = args.batch * (prompt_len + W + K // 2) * L * 2 * kvd * 2
    achieved = (weights + cache) / (ms * 1e-3) / 1e9
    linear = 2.0 * prompt_len * ((q + 2 * kvd) * H + H * q + 2 * I * H + H * I)
    flops = L * (linear + 4.0 * prompt_len * prompt_len * q / 2.0) + 2.0 * vocab * H
    n = args.batch
    out = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": round(main_r["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights (seed 4), uniform random token ids",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "full_layers": full_layers, "hidden": H,
                   "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": I, "vocab": vocab, "global_batch": n,
                   "seq_len": prompt_len, "page_size": page, "prefill_chunk": 8192, "parallelism": "1gpu",
                   "cuda_graph": True, "l2": "inputs larger than L2 (16 GB of weights per step)",
                   "peaks": peak_src, "path": "rollout QwenModel.build_graph + Model.prefill / Model.decode"},
        "clocks": clk,
        # Model.decode per step: write positions (int64), query positions (int32), last-page counts (uint8) and the
        # tokens (int64) go in; the sampled tokens (int64) and their log-probs (float32) come out
        "e2e": {"value": round(main_r["e2e_tokens_per_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 21 * n, "d2h_bytes_per_step": 12 * n, "steps": K},
        "gpu_launches": 0,
        "prefill": {"value": round(pf["tokens_per_s"], 1), "tokens": prompt_len, "ms": round(pf["ms"], 3),
                    "frac": round(flops / (pf["ms"] * 1e-3) / (bf16_tflops * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": pts,
        "build_s": round(build_s, 1),
    }
    print(json.dumps(out))
    return 0


# ------------------------------------------------------------------------------- the reference's kernels alone

def _time_graph(torch, fns, iters=10, warmup=3):
    """Mean device milliseconds of one launch: all of ``fns`` back to back in one CUDA graph, replayed."""
    for _ in range(warmup):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
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


def _copies(nbytes, l2=126 << 20):
    return max(2, min(64, (2 * l2 + nbytes - 1) // max(1, nbytes)))


def kernels(torch, rq3, shape, dev) -> int:
    """The reference's Triton kernels alone on random data, each over rotating buffers larger than L2."""
    from rollout.attention import _pick_num_splits, flash_decode, flash_prefill
    from rollout.cache import KVCache
    from rollout.fused import rms_norm, silu_and_mul
    Hq, Hkv, D = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    H, I = shape["hidden_size"], shape["intermediate_size"]
    half = D // 2
    inv = 1.0 / (shape["rope_theta"] ** (torch.arange(0, half, dtype=torch.float32, device=dev) / half))
    fr = torch.outer(torch.arange(40960, dtype=torch.float32, device=dev), inv)
    cos, sin = fr.cos().bfloat16().contiguous(), fr.sin().bfloat16().contiguous()
    scale = D ** -0.5
    rnd = lambda *s: torch.randn(*s, device=dev, dtype=torch.float32).bfloat16()

    def cache_with(batch, ctx):
        c = KVCache(1, batch * (ctx + 128), Hkv, D, max_reside=batch, device=dev)
        c.k_pool[0].copy_(rnd(*c.k_pool[0].shape))
        c.v_pool[0].copy_(rnd(*c.v_pool[0].shape))
        c.plan_reset()
        for sid in range(batch):
            c.alloc(sid)
            c.plan_append(sid, ctx, new_para=True)
        c.flush_wpos()
        return c

    for batch, ctx in ((1, 2048), (8, 2048), (64, 2048), (8, 32768)):
        nbytes = 2 * batch * ctx * Hkv * D * 2
        fns = []
        ns = _pick_num_splits(batch, Hkv, dev)
        for _ in range(_copies(nbytes)):
            c = cache_with(batch, ctx)
            c.build_tables(list(range(batch)), prefill=False)
            q = rnd(batch, Hq, D)
            fns.append(lambda c=c, q=q: flash_decode(q, c.page_table, c.mask_table, c.cu_pages, c.qpos, c.page_pos,
                                                     c.k_pool[0], c.v_pool[0], cos, sin, Hkv, ns, scale))
        ms = _time_graph(torch, fns)
        print(json.dumps({"impl": "reference", "kernel": "flash_decode", "batch": batch, "ctx": ctx, "splits": ns,
                          "ms": ms, "GBps": nbytes / ms / 1e6}), flush=True)
        del fns

    for ctx in (2048, 8192):
        c = cache_with(1, ctx)
        c.set_req_q({0: ctx})
        n, _, _ = c.build_tables([0], prefill=True)
        q = rnd(ctx, Hq, D)
        fn = lambda: flash_prefill(q, c.page_table, c.mask_table, c.cu_pages, c.cu_q, c.qpos, c.page_pos,
                                   c.k_pool[0], c.v_pool[0], cos, sin, Hkv, n, scale)
        ms = _time_graph(torch, [fn])
        flops = 4.0 * Hq * D * ctx * ctx / 2.0
        print(json.dumps({"impl": "reference", "kernel": "flash_prefill", "ctx": ctx, "q_len": ctx, "ms": ms,
                          "TFLOPs": flops / ms / 1e9}), flush=True)

    for rows in (8, 64, 2048):
        w = rnd(H)
        nbytes = rows * H * 2 * 2
        xs = [rnd(rows, H) for _ in range(_copies(nbytes))]
        ms = _time_graph(torch, [lambda x=x: rms_norm(x, w, 1e-6, offset=0.0) for x in xs])
        print(json.dumps({"impl": "reference", "kernel": "rms_norm", "rows": rows, "width": H, "ms": ms,
                          "GBps": nbytes / ms / 1e6}), flush=True)
        nbytes = rows * I * 3 * 2
        gus = [rnd(rows, 2 * I) for _ in range(_copies(nbytes))]
        ms = _time_graph(torch, [lambda gu=gu: silu_and_mul(gu) for gu in gus])
        print(json.dumps({"impl": "reference", "kernel": "silu_and_mul", "rows": rows, "width": I, "ms": ms,
                          "GBps": nbytes / ms / 1e6}), flush=True)
    return 0
