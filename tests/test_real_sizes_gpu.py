"""The engine at the layer sizes of Qwen3-8B against the plain implementation, in both precisions.

Every other model-level test is tiny (hidden size up to 96).  Here the layers have their real sizes
(hidden 4096, 32 heads of 128 in 8 groups, feed-forward 12288, theta 1e6, untied head), with two layers
and a vocabulary of 2,048 so that the plain implementation runs on the CPU in seconds.  One mixed
trace: a prompt long enough that the tcgen05 attention kernel runs several 256-row blocks and splits
the keys of a later portion, portions of some requests beside single decoded tokens of others, and so
few pages that they are handed out again.  In spirit rollout/utils/check_chunk_prefill.py:139-179
(the same scenario under different chunkings), with a plain oracle instead of the engine itself.
"""
import os

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

REAL = dict(vocab_size=2048, hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
            num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0,
            rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)


@pytest.fixture(scope="module")
def real_model(tmp_path_factory):
    from return_b200.config.model_config import Qwen3Config
    from return_b200.weights import loader
    d = os.path.join(str(tmp_path_factory.mktemp("real")), "m")
    # stored in bfloat16: both precisions of the engine and the plain implementation then read the same numbers
    loader.write_random_model(d, Qwen3Config.from_dict(REAL), 4, torch.bfloat16)
    return d


def _trace():
    """Four requests, three live at a time.  r0 (700 tokens): 520 in one step (three row blocks of the
    tcgen05 kernel), then a portion of 140 behind them (few CTAs: the keys are split), then tokens one by one
    beside the others' portions."""
    lens = {"r0": 700, "r1": 150, "r2": 90, "r3": 260}
    reqs = {rid: helpers.random_ids(REAL["vocab_size"], n, 500 + i) for i, (rid, n) in enumerate(lens.items())}
    want_tail = lambda n, k=3: list(range(max(0, n - k), n))            # the last places of a portion
    st = []
    add = lambda entries, end=(): st.append({"step": len(st), "entries": entries, "end": list(end)})
    seg = lambda rid, a, b: {"id": rid, "tokens": reqs[rid][a:b], "want": want_tail(b - a)}
    add([seg("r0", 0, 520)])
    add([seg("r0", 520, 660), seg("r1", 0, 100)])
    add([seg("r0", 660, 661), seg("r1", 100, 149), seg("r2", 0, 60)])
    add([seg("r0", 661, 662), seg("r1", 149, 150), seg("r2", 60, 62)], end=["r1"])
    add([seg("r0", 662, 663), seg("r2", 62, 63), seg("r3", 0, 200)])            # r3 takes r1's pages
    a = 200
    for k in range(27):                           # r0, r2 decode; r3 in portions of two, then token by token too
        n = 2 if k < 14 else 1                    # (from k = 14 on the steps hold single tokens only: the captured path)
        add([seg("r0", 663 + k, 664 + k), seg("r2", 63 + k, 64 + k), seg("r3", a, a + n)],
            end=["r2"] if k == 26 else [])
        a += n
    add([seg("r0", 690, 700), seg("r3", a, 260)], end=["r0", "r3"])
    return reqs, st


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graph", [False, True])
def test_mixed_trace_at_real_layer_sizes(real_model, dtype, graph):
    from return_b200.engine.replay import TraceReplayer
    reqs, steps = _trace()
    assert all(sum(len(e["tokens"]) for s in steps for e in s["entries"] if e["id"] == rid) == len(ids)
               for rid, ids in reqs.items())
    pool = helpers.pool_tokens(steps)
    assert pool < sum((len(v) + 63) // 64 * 64 for v in reqs.values())          # pages must be used again
    rp = TraceReplayer(real_model, dtype, pool, page_size=16, max_reside=3, poison=True, use_cuda_graph=graph)
    refs = {rid: helpers.plain_logits(real_model, ids) for rid, ids in reqs.items()}
    scale = float(torch.cat(list(refs.values())).std())
    # float32: the contract.  bfloat16: a twelfth of the logits' standard deviation, as for the tiny models
    tol = 1e-4 if dtype == "float32" else scale / 12
    pos, worst = {}, 0.0
    for st in steps:
        lg = rp.run_step(st).float().cpu()
        rp.runner.manager.check()
        r = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                err = float((lg[r] - refs[e["id"]][base + w]).abs().max())
                assert err <= tol, f"{dtype} step {st['step']} {e['id']} position {base + w}: error {err:.3g} (tolerance {tol:.3g})"
                worst = max(worst, err)
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
    assert rp.runner.manager.pages_used() == [0]
    print(f"real sizes {dtype} graph={graph}: worst error {worst:.3g}, logits' deviation {scale:.3g}")


def test_long_portions_take_the_pair_kernel(real_model):
    """Portions of 768 rows and more run the gated feed-forward product on the tcgen05 kernel by pairs of CTAs
    (ops.PAIR_MIN_ROWS): a prompt of 1,100 tokens in one step, then 840 tokens of a second request beside a
    decoded token of the first, against the plain implementation in bfloat16."""
    from return_b200.engine.replay import TraceReplayer
    from return_b200.ext import ops
    assert ops.PAIR_MIN_ROWS <= 840
    lens = {"p0": 1102, "p1": 850}
    reqs = {rid: helpers.random_ids(REAL["vocab_size"], n, 700 + i) for i, (rid, n) in enumerate(lens.items())}
    tail = lambda n, k=4: list(range(max(0, n - k), n))
    steps = [
        {"step": 0, "entries": [{"id": "p0", "tokens": reqs["p0"][:1100], "want": tail(1100) + [3, 500, 767, 768]}], "end": []},
        {"step": 1, "entries": [{"id": "p0", "tokens": reqs["p0"][1100:1101], "want": [0]},
                                {"id": "p1", "tokens": reqs["p1"][:840], "want": tail(840) + [0, 255, 256]}], "end": []},
        {"step": 2, "entries": [{"id": "p0", "tokens": reqs["p0"][1101:1102], "want": [0]},
                                {"id": "p1", "tokens": reqs["p1"][840:850], "want": tail(10)}], "end": ["p0", "p1"]},
    ]
    calls = []
    real = ops.gemm_tc5

    def spy(*a, **kw):
        calls.append((a[0].shape[0], kw.get("pair", False), kw.get("gated", False)))
        return real(*a, **kw)

    rp = TraceReplayer(real_model, "bfloat16", helpers.pool_tokens(steps), page_size=16, max_reside=2, poison=True)
    refs = {rid: helpers.plain_logits(real_model, ids) for rid, ids in reqs.items()}
    tol = float(torch.cat(list(refs.values())).std()) / 12
    ops.gemm_tc5 = spy
    try:
        pos = {}
        for st in steps:
            lg = rp.run_step(st).float().cpu()
            r = 0
            for e in st["entries"]:
                base = pos.get(e["id"], 0)
                for w in e["want"]:
                    err = float((lg[r] - refs[e["id"]][base + w]).abs().max())
                    assert err <= tol, f"step {st['step']} {e['id']} position {base + w}: error {err:.3g} (tolerance {tol:.3g})"
                    r += 1
                pos[e["id"]] = base + len(e["tokens"])
    finally:
        ops.gemm_tc5 = real
    # two layers in each of the two long steps, none in the short one
    assert sorted(calls) == [(841, True, True)] * 2 + [(1100, True, True)] * 2, calls
