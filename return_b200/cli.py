"""Command line: ``python -m return_b200 <command>``.

Option names follow the reference where it has them: ``--model``, ``--max-reside``, ``--max-token``
(rollout/server.py:87-98); ``--batch``, ``--ctx``, ``--prompt-len``, ``--steps``, ``--warmup``,
``--new`` (rollout/utils/bench_sym.py:55-63, rollout/utils/check_correctness.py:43-50); the
sampling options are the fields of its ``Request`` (rollout/engine.py:17-21).

  generate        tokens for prompts given as ids (``--prompt-ids``) or drawn at random (``--prompt-len``)
  random-weights  write a model folder (config.json, model.safetensors) from a config.json and a seed
  bench           decode tokens/s per batch size and prefill tokens/s
  kernel-bench    one kernel alone on random data
  workload        a named workload (Qwen3-0.6B mixed batch, Qwen3-32B batch 16) through the engine, random weights
  replay          trace replay (what ``bin/trace_run`` does), from a file of JSON lines
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _engine_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--max-reside", type=int, default=64, help="most requests that hold cache at a time")
    p.add_argument("--max-token", type=int, default=65536, help="capacity of the KV pool in token slots")
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--chunk", type=int, default=8192, help="most tokens one step runs (prefill chunk)")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--graph", action=argparse.BooleanOptionalAction, default=True,
                   help="replay CUDA graphs for steps that only decode")
    p.add_argument("--capture-at-start", action="store_true",
                   help="capture every decode graph before the first request instead of on first use")
    p.add_argument("--seed", type=int, default=0)


def _make_engine(args):
    from .engine.config import EngineConfig
    from .engine.engine import Engine
    cfg = EngineConfig(max_token=args.max_token, max_reside=args.max_reside, page_size=args.page_size,
                       prefill_chunk=args.chunk, dtype=args.dtype, use_cuda_graph=args.graph, capture_at_start=args.capture_at_start, seed=args.seed,
                       device=args.device)
    return Engine(args.model, cfg)


def _ids(text: str):
    return [int(x) for x in text.replace(",", " ").split()]


def cmd_generate(args) -> int:
    import torch
    engine = _make_engine(args)
    prompts = [_ids(p) for p in (args.prompt_ids or [])]
    if args.prompt_len:
        g = torch.Generator().manual_seed(args.seed)
        vocab = engine.runner.vocab_size
        prompts += [torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist() for _ in range(args.batch)]
    if not prompts:
        print("give --prompt-ids or --prompt-len", file=sys.stderr)
        return 2
    stops = [_ids(s) for s in (args.stop_ids or [])]
    results = engine.generate(prompts, max_new_tokens=args.new, temperature=args.temperature, top_p=args.top_p,
                              top_k=args.top_k, stop_ids=stops, seed=args.seed, eos_token_id=args.eos_token_id)
    for r in results:
        print(json.dumps(r.as_dict()))
    print(json.dumps({"stats": engine.stats()}), file=sys.stderr)
    return 0


def cmd_random_weights(args) -> int:
    import torch
    from .config import registry
    from .weights import loader
    with open(args.config) as f:
        raw = json.load(f)
    arch = registry.resolve(raw)
    cfg = arch.config_cls.from_dict(raw)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    loader.write_random_model(args.out, cfg, args.seed, dtype)
    print(args.out)
    return 0


def cmd_bench(args) -> int:
    from . import benchmark
    engine = _make_engine(args)
    for b in [int(x) for x in args.batch.split(",")]:
        r = benchmark.decode_throughput(engine.runner, b, args.ctx, args.steps, args.warmup)
        print(json.dumps({"batch": b, "ctx": args.ctx, **r}))
        if args.profile:
            p = benchmark.profile_decode(engine.runner, b, args.ctx, args.steps, args.warmup)
            print(f"bs={b} ctx={args.ctx}  GPU busy {p['gpu_ms_per_step']:.3f} ms/step")
            print(f"{'bucket':<18}{'ms/step':>10}{'%GPU':>8}{'kern/step':>11}")
            for row in p["buckets"]:
                print(f"{row['bucket']:<18}{row['ms_per_step']:>10.3f}{row['share'] * 100:>7.1f}%{row['kernels_per_step']:>11.1f}")
            print("--- top kernels (own device time) ---")
            for row in p["top_kernels"]:
                print(f"{row['ms_per_step']:>8.3f} ms {row['share'] * 100:>5.1f}%  {row['kernel']}")
    r = benchmark.prefill_throughput(engine.runner, args.prompt_len, max(1, args.steps // 4), max(1, args.warmup // 2))
    print(json.dumps({"prefill_tokens": args.prompt_len, **r}))
    return 0


def cmd_workload(args) -> int:
    from . import benchmark
    print(json.dumps(benchmark.run_workload(args.name, args.layers, args.new)))
    return 0


def cmd_kernel_bench(args) -> int:
    from . import benchmark
    fn = {"attention_decode": benchmark.kernel_attention_decode, "attention_prefill": benchmark.kernel_attention_prefill,
          "gemm": benchmark.kernel_gemm, "gated": benchmark.kernel_gated, "elementwise": benchmark.kernel_elementwise}[args.kernel]
    kw = {}
    for item in args.set or []:
        k, v = item.split("=")
        kw[k] = int(v)
    print(json.dumps(fn(**kw)))
    return 0


def cmd_replay(args) -> int:
    import torch
    from .engine.replay import TraceReplayer
    rp = TraceReplayer(args.model, args.dtype, args.max_tokens, page_size=args.page_size, use_cuda_graph=args.graph)
    os.makedirs(args.out, exist_ok=True)
    with open(args.trace) as f:
        for line in f:
            if not line.strip():
                continue
            rec = json.loads(line)
            logits = rp.run_step(rec)
            if logits is not None:
                logits.to("cpu", torch.float32).numpy().astype("<f4").tofile(os.path.join(args.out, f"{rec['step']}.f32"))
            print(f"done {rec['step']}", flush=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m return_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens")
    _engine_args(g)
    g.add_argument("--prompt-ids", action="append", help='token ids of one prompt, e.g. "5,17,3" (repeatable)')
    g.add_argument("--prompt-len", type=int, default=0, help="length of random prompts")
    g.add_argument("--batch", type=int, default=1, help="number of random prompts")
    g.add_argument("--new", "--max-new-tokens", dest="new", type=int, default=32)
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--stop-ids", action="append", help="a stop sequence of token ids (repeatable)")
    g.add_argument("--eos-token-id", type=int, default=None, help="a stop sequence of one token")
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("random-weights", help="write a random model folder")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r.set_defaults(fn=cmd_random_weights)

    b = sub.add_parser("bench", help="decode and prefill throughput")
    _engine_args(b)
    b.add_argument("--batch", default="1,8,64")
    b.add_argument("--ctx", type=int, default=2048)
    b.add_argument("--prompt-len", type=int, default=2048)
    b.add_argument("--steps", type=int, default=50)
    b.add_argument("--warmup", type=int, default=10)
    b.add_argument("--profile", action="store_true",
                   help="after each batch size, the share of device time by kind of kernel (GEMM, decode attention, norm, ...)")
    b.set_defaults(fn=cmd_bench)

    wl = sub.add_parser("workload", help="a named workload through the engine, random weights of that shape")
    wl.add_argument("name", choices=["0.6b-mixed", "32b"])
    wl.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has, where time needs it")
    wl.add_argument("--new", type=int, default=0, help="fewer new tokens per request than the workload names")
    wl.set_defaults(fn=cmd_workload)

    k = sub.add_parser("kernel-bench", help="time one kernel alone on random data (for profiles)")
    k.add_argument("kernel", choices=["attention_decode", "attention_prefill", "gemm", "gated", "elementwise"])
    k.add_argument("--set", action="append", help="an integer argument of the kernel case, e.g. batch=64 ctx=2048 M=8")
    k.set_defaults(fn=cmd_kernel_bench)

    t = sub.add_parser("replay", help="trace replay from a file")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    t.add_argument("--trace", required=True)
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--page-size", type=int, default=16)
    t.add_argument("--graph", action="store_true", help="steps of single tokens replay captured CUDA graphs")
    t.set_defaults(fn=cmd_replay)

    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
