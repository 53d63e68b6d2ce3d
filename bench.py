"""Benchmark of the engine on one B200: decode tokens/s of a Qwen3-8B-shaped model with random
weights at batch 8 after 2,048-token prompts (the headline), the same at batch 1 and 64, prefill
tokens/s of a 2,048-token prompt, the decode step's HBM roofline, and the same decode metric end to
end through ``Engine.step`` with host tokens in and out.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  For --gpus > 1 it prints one line that says so and exits with 2: the engine
runs on one GPU.  Device times come from CUDA events around exactly K steps after W warm-up steps;
the step's inputs (16 GB of weights) are far larger than L2, so no flush is needed between steps.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the layer sizes of Qwen3-8B, the benchmark's named configuration
MODEL = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
             num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0,
             rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)
FULL_LAYERS = 36
PROMPT_LEN = 2048
CTX_LIMIT = 8192
PAGE = 16
FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS = 6650.0, 1590.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return float(p["hbm_gbs"]), float(p.get("bf16_tflops", FALLBACK_BF16_TFLOPS)), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=None)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(mhz)}


def run_reference(args):
    """The reference's own engine on the same metric (baseline/reference_arm.py); nothing of return_b200 is imported."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm
    return reference_arm.run(args, MODEL, PROMPT_LEN, FULL_LAYERS, peaks(), ClockSampler)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers where memory or time needs it")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="a reduced run for profiling: only the decode steps, or only the prefill")
    ap.add_argument("--kernels", action="store_true",
                    help="with --impl reference: time the reference's Triton kernels alone, one JSON line each")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(json.dumps({"error": f"return_b200 is a one-GPU engine; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    W = max(3, args.warmup)
    K = max(1, args.steps)

    import torch
    from return_b200 import benchmark
    from return_b200.config.model_config import Qwen3Config
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.engine import Engine
    from return_b200.engine.request import Request
    from return_b200.engine.runner import ModelRunner
    from return_b200.ext import ops

    cfg = Qwen3Config.from_dict(dict(MODEL, num_hidden_layers=args.layers))
    big = 64
    pool = big * ((PROMPT_LEN + W + K + 64 + 63) // 64 * 64)
    ecfg = EngineConfig(max_token=pool, max_reside=big, page_size=PAGE, prefill_chunk=8192, dtype="bfloat16",
                        max_model_len=CTX_LIMIT, use_cuda_graph=True, seed=4)
    t0 = time.time()
    runner = ModelRunner.from_random(cfg, ecfg, seed=4)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    hbm_gbs, bf16_tflops, peak_src = peaks()

    if args.only != "all":
        if args.only == "decode":
            r = benchmark.decode_throughput(runner, args.batch, PROMPT_LEN, K, W)
        else:
            r = benchmark.prefill_throughput(runner, PROMPT_LEN, iters=K, warmup=W)
        print(json.dumps({"only": args.only, "layers": args.layers, "batch": args.batch, **r}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    launches0 = ops.launch_count
    # the prefill is a burst of a few steps and is set against the burst peak: it runs first
    pf = benchmark.prefill_throughput(runner, PROMPT_LEN, iters=5, warmup=3)
    launches0 = ops.launch_count
    main_r = benchmark.decode_throughput(runner, args.batch, PROMPT_LEN, K, W)
    per_replay = runner.launches_per_replay.get(args.batch, 0)
    launches = per_replay * K if per_replay else ops.launch_count - launches0
    pts = {}
    for b in (1, 64):
        r = benchmark.decode_throughput(runner, b, PROMPT_LEN, max(8, K // 2), W)
        pts[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
        pts[f"decode_b{b}_ms"] = round(r["ms_per_step"], 3)

    # end to end: the same decode metric through Engine.step, host tokens in and out every step
    engine = Engine(runner)
    reqs = [Request(f"e2e-{i}", torch.randint(0, cfg.vocab_size, (PROMPT_LEN,), generator=torch.Generator().manual_seed(100 + i)).tolist(),
                    max_new_tokens=2 * W + K + 16, temperature=0.0) for i in range(args.batch)]
    for r in reqs:
        engine.add_request(r)
    while any(len(r.output) < 1 for r in reqs):        # prompts, in portions under the token budget
        engine.step()
    engine.run(max_steps=W)                              # warm-up decode steps (captures the graph)
    torch.cuda.synchronize()
    before = sum(len(r.output) for r in reqs)
    t1 = time.perf_counter()
    engine.run(max_steps=K)                              # every step: tables in from pinned memory, tokens out to the host
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t1
    e2e_tokens = sum(len(r.output) for r in reqs) - before
    n_steps = K
    clk = clocks.stop()

    ms = main_r["ms_per_step"]
    step_bytes = benchmark.decode_step_bytes(cfg, args.batch, main_r["kv_tokens"])
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = benchmark.prefill_flops(cfg, PROMPT_LEN)
    blocks = (PROMPT_LEN + W + K + PAGE - 1) // PAGE
    h2d = 4 * (5 * args.batch + args.batch + 1 + 3 * args.batch + args.batch * blocks) + 16 * args.batch
    out = {
        "metric": "decode_tokens_per_s", "value": round(main_r["tokens_per_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights (seed 4), uniform random token ids",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "full_layers": FULL_LAYERS, "hidden": 4096,
                   "heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288, "vocab": 151936,
                   "global_batch": args.batch, "seq_len": PROMPT_LEN, "ctx_limit": CTX_LIMIT, "page_size": PAGE,
                   "parallelism": "1gpu", "cuda_graph": True, "l2": "inputs larger than L2 (16 GB of weights per step)",
                   "peaks": peak_src},
        "clocks": clk,
        "e2e": {"value": round(e2e_tokens / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 8 * args.batch, "steps": n_steps},
        "gpu_launches": int(launches),
        "prefill": {"value": round(pf["tokens_per_s"], 1), "tokens": PROMPT_LEN, "ms": round(pf["ms"], 3),
                    "frac": round(flops / (pf["ms"] * 1e-3) / (bf16_tflops * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": pts,
        "build_s": round(build_s, 1),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
