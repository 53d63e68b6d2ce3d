"""Shared pieces of the tests: tiny configurations, model folders in temporary places, the plain
implementation's logits, and trace builders."""
from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

from plain import qwen3_plain as plain  # noqa: E402
from return_b200.config.model_config import Qwen3Config  # noqa: E402
from return_b200.weights import loader  # noqa: E402

# Tiny A and tiny B differ in every size and option; tiny C adds sliding-window layers beside full ones.
TINY_A = dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128)
TINY_B = dict(vocab_size=384, hidden_size=96, intermediate_size=224, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=3, head_dim=32, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256)
TINY_C = dict(vocab_size=200, hidden_size=80, intermediate_size=144, num_hidden_layers=4,
              num_attention_heads=5, num_key_value_heads=1, head_dim=48, rope_theta=50000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=512,
              sliding_window=24, use_sliding_window=True,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"])
CASES = {"A": (TINY_A, 0, 16), "B": (TINY_B, 2, 8), "C": (TINY_C, 7, 16)}   # config, weight seed, page size


def tiny_config(name: str) -> Qwen3Config:
    return Qwen3Config.from_dict(dict(CASES[name][0]))


def make_model_dir(tmp_path, name: str, dtype=torch.float32, **overrides) -> str:
    raw, seed, _ = CASES[name]
    cfg = Qwen3Config.from_dict({**raw, **overrides})
    d = os.path.join(str(tmp_path), f"tiny_{name}")
    loader.write_random_model(d, cfg, seed, dtype)
    return d


def random_ids(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(model_dir: str, ids, dtype=torch.float32, schedule=None) -> torch.Tensor:
    c = plain.read_config(model_dir)
    w = plain.read_weights(model_dir, dtype)
    return plain.forward_logits(c, w, ids, schedule)


# ------------------------------------------------------------------------------- traces

def whole(requests):
    """Each request alone and whole in one step, all logits wanted; freed afterwards."""
    steps = []
    for rid, ids in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}],
                      "end": [rid]})
    return steps


def tail_decoded(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[i]], "want": [0]}],
                          "end": [rid] if i == len(ids) - 1 else []})
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes):
    """Each request in portions of changing size (cycled), down to two tokens."""
    steps = []
    for rid, ids in requests.items():
        i, k = 0, 0
        while i < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - i)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[i:i + n], "want": list(range(n))}],
                          "end": [rid] if i + n == len(ids) else []})
            i += n
            k += 1
    return steps


def mixed(requests, max_live=4, portion=13, decode_tail=6, seed=0):
    """Up to ``max_live`` live requests: portions of some beside single tokens of others.  A request
    is fed in portions until ``decode_tail`` tokens remain, then one token a step; when it ends, the
    next waiting request starts, so pages are handed out again."""
    waiting = list(requests.items())
    live = {}
    steps = []
    g = torch.Generator().manual_seed(seed)
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = [ids, 0]
        entries, ended = [], []
        for rid in list(live):
            ids, done = live[rid]
            left = len(ids) - done
            if left > decode_tail:
                # sometimes skip a live request for a step: it goes on later
                if len(live) > 1 and torch.rand((), generator=g).item() < 0.15:
                    continue
                n = min(max(2, int(torch.randint(2, portion + 1, (), generator=g))), left - decode_tail)
            else:
                n = 1
            entries.append({"id": rid, "tokens": ids[done:done + n], "want": list(range(n))})
            live[rid][1] = done + n
            if done + n == len(ids):
                ended.append(rid)
                del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def collect(steps, step_logits):
    """{request: [T, V] logits by position} from the logits of each step (None where nothing wanted)."""
    rows, pos = {}, {}
    for st, lg in zip(steps, step_logits):
        r = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e.get("want", []):
                rows.setdefault(e["id"], {})[base + w] = lg[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
    return {rid: torch.stack([d[i] for i in sorted(d)]) for rid, d in rows.items()}


def pool_tokens(steps, round_to=64):
    """The most tokens that live requests hold at any time, each rounded up to ``round_to``."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak
