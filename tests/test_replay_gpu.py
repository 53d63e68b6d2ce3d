"""The engine against the plain implementation, through trace replay, however the work is cut."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

# float32: the engine's contract.  bfloat16: the tiny models' logits have a standard deviation of about 0.18
# and the engine's error stays near 5e-3; a tenth of a deviation would already be a fault (a key tile dropped
# in one head moves them further: test_a_dropped_key_tile_breaks_the_bfloat16_tolerance).
TOL = {"float32": 1e-4, "bfloat16": 1.5e-2}


def _requests(name, lens, seed):
    vocab = helpers.CASES[name][0]["vocab_size"]
    return {f"r{i}": helpers.random_ids(vocab, n, seed + i) for i, n in enumerate(lens)}


def _replay(model_dir, dtype, steps, page, pool=None, poison=True, max_reside=8, graph=False, before_step=None):
    from return_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(model_dir, dtype, pool or helpers.pool_tokens(steps), page_size=page,
                       max_reside=max_reside, poison=poison, use_cuda_graph=graph)
    out = []
    for st in steps:
        undo = before_step(rp, st) if before_step is not None else None
        lg = rp.run_step(st)
        if undo is not None:
            undo()
        out.append(None if lg is None else lg.float().cpu())
        rp.runner.manager.check()
    assert rp.runner.manager.pages_used() == [0] * len(rp.runner.manager.groups)
    if graph:
        _replay.graphs = dict(rp.runner._graphs)
    return helpers.collect(steps, out)


def _compare(model_dir, requests, got, dtype, tol=None):
    worst = 0.0
    tol = TOL[dtype] if tol is None else tol
    for rid, ids in requests.items():
        ref = helpers.plain_logits(model_dir, ids)
        assert got[rid].shape == ref.shape
        err = (got[rid] - ref).abs().max(dim=1).values
        assert torch.isfinite(got[rid]).all(), f"{rid}: non-finite logits"
        bad = (err > tol).nonzero()
        assert bad.numel() == 0, f"{dtype} {rid}: first wrong position {int(bad[0])} of {len(ids)}, error {float(err.max()):.3g}"
        worst = max(worst, float(err.max()))
    return worst


LENS = {"A": (5, 17, 33, 100), "B": (1, 9, 40, 71), "C": (3, 50, 90, 130)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_whole_requests(tmp_path, case, dtype):
    d = helpers.make_model_dir(tmp_path, case)
    reqs = _requests(case, LENS[case], 10)
    got = _replay(d, dtype, helpers.whole(reqs), helpers.CASES[case][2])
    _compare(d, reqs, got, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(tmp_path, case, dtype):
    d = helpers.make_model_dir(tmp_path, case)
    reqs = _requests(case, LENS[case][1:], 20)
    got = _replay(d, dtype, helpers.tail_decoded(reqs, 32), helpers.CASES[case][2])
    _compare(d, reqs, got, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_portions_of_changing_size(tmp_path, case, dtype):
    d = helpers.make_model_dir(tmp_path, case)
    reqs = _requests(case, LENS[case][1:], 30)
    got = _replay(d, dtype, helpers.portions(reqs, [13, 2, 7, 3, 29, 2, 16]), helpers.CASES[case][2])
    _compare(d, reqs, got, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_mixed_batches_with_page_reuse(tmp_path, case, dtype):
    d = helpers.make_model_dir(tmp_path, case)
    reqs = _requests(case, (40, 71, 9, 1, 55, 33, 90, 17), 40)
    steps = helpers.mixed(reqs, max_live=4, portion=13, decode_tail=6, seed=3)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"] if len(s["entries"]) > 1)
    got = _replay(d, dtype, steps, helpers.CASES[case][2], max_reside=4)
    _compare(d, reqs, got, dtype)


def _decoding_together(requests, tails):
    """Every request's prompt but its last ``tails[rid]`` tokens in a step of its own; then all of them decode
    together, one token each a step, and end one by one as they run out."""
    steps, live = [], {}
    for rid, ids in requests.items():
        head = len(ids) - tails[rid]
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head], "want": [head - 1]}], "end": []})
        live[rid] = head
    while live:
        entries, ended = [], []
        for rid in list(live):
            ids = requests[rid]
            entries.append({"id": rid, "tokens": [ids[live[rid]]], "want": [0]})
            live[rid] += 1
            if live[rid] == len(ids):
                ended.append(rid)
                del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def _compare_wanted(model_dir, requests, steps, got_steps, dtype):
    """Like ``_compare`` for traces that want only some places."""
    pos, worst = {}, 0.0
    refs = {rid: helpers.plain_logits(model_dir, ids) for rid, ids in requests.items()}
    for st, lg in zip(steps, got_steps):
        r = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                err = float((lg[r] - refs[e["id"]][base + w]).abs().max())
                assert err <= TOL[dtype], f"{dtype} step {st['step']} {e['id']} position {base + w}: error {err:.3g}"
                worst = max(worst, err)
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_meet_the_oracle(tmp_path, dtype):
    """Steps of single tokens through captured CUDA graphs (the path generation takes by default): tables at
    fixed addresses, key splits fixed per graph, and, with eleven live requests, the graph of twelve with a
    padding row.  Their logits, not only their tokens, are compared with the plain implementation."""
    from return_b200.engine.replay import TraceReplayer
    d = helpers.make_model_dir(tmp_path, "B")
    reqs = _requests("B", (40, 71, 9, 33), 20)
    got = _replay(d, dtype, helpers.tail_decoded(reqs, 32), 8, graph=True)
    _compare(d, reqs, got, dtype)
    assert {n for n, _ in _replay.graphs} == {1}
    reqs = _requests("B", (40, 71, 9, 1, 55, 33, 90, 17), 40)
    got = _replay(d, dtype, helpers.mixed(reqs, max_live=4, portion=13, decode_tail=6, seed=3), 8, max_reside=4, graph=True)
    _compare(d, reqs, got, dtype)
    assert _replay.graphs, "no step of the mixed trace was a step of single tokens"
    # eleven requests that decode together and end one by one: 11 -> the graph of 12, then 8, 7, ...
    reqs = _requests("B", tuple(12 + 5 * i for i in range(11)), 90)
    steps = _decoding_together(reqs, {rid: 3 + k for k, rid in enumerate(reqs)})
    rp = TraceReplayer(d, dtype, helpers.pool_tokens(steps), page_size=8, max_reside=12, poison=True, use_cuda_graph=True)
    out = []
    for st in steps:
        lg = rp.run_step(st)
        out.append(None if lg is None else lg.float().cpu())
        rp.runner.manager.check()
    _compare_wanted(d, reqs, steps, out, dtype)
    assert 12 in {n for n, _ in rp.runner._graphs}


def test_a_dropped_key_tile_breaks_the_bfloat16_tolerance(tmp_path):
    """The tolerance can fail: for one step the first block of one request's block table is pointed at the
    request's second page (memory it holds and has written), so sixteen keys are lost and sixteen counted
    twice.  The comparison with the plain implementation must then fail; without the damage it passes."""
    d = helpers.make_model_dir(tmp_path, "A")
    reqs = _requests("A", (100,), 33)
    steps = helpers.tail_decoded(reqs, 32)
    _compare(d, reqs, _replay(d, "bfloat16", steps, 16), "bfloat16")

    def damage(rp, st):
        if st["step"] != 20:
            return None
        blocks = rp.runner.manager._req["r0"].blocks[0]
        first = blocks[0]
        blocks[0] = blocks[1]

        def undo():
            blocks[0] = first
        return undo

    got = _replay(d, "bfloat16", steps, 16, before_step=damage)
    ref = helpers.plain_logits(d, reqs["r0"])
    err = (got["r0"] - ref).abs().max(dim=1).values
    hit = 100 - 32 + 20 - 1                            # the position whose step was damaged
    assert float(err[hit]) > TOL["bfloat16"], float(err[hit])
    assert float(torch.cat([err[:hit], err[hit + 1:]]).max()) <= TOL["bfloat16"]


def test_cutting_does_not_change_float32_logits_at_all(tmp_path):
    """The 32-bit kernels fix the order of every sum, so any cutting gives the same bits."""
    d = helpers.make_model_dir(tmp_path, "B")
    reqs = _requests("B", (71, 40), 50)
    a = _replay(d, "float32", helpers.whole(reqs), 8)
    b = _replay(d, "float32", helpers.portions(reqs, [5, 2, 11]), 8)
    c = _replay(d, "float32", helpers.mixed(reqs, max_live=2, portion=9, seed=1), 8)
    for rid in reqs:
        assert torch.equal(a[rid], b[rid]) and torch.equal(a[rid], c[rid])


def test_long_decoding(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A")
    reqs = _requests("A", (300,), 60)
    steps = helpers.tail_decoded(reqs, 290)
    for dtype in ("float32", "bfloat16"):
        got = _replay(d, dtype, steps, 16)
        _compare(d, reqs, got, dtype)


def test_short_portions_of_a_long_prompt_split_their_keys(tmp_path, monkeypatch):
    """Head size 64 puts prompt portions on the tcgen05 attention kernel; a portion of 300 tokens behind more
    than a thousand cached ones gives so few CTAs that the keys of every block are split over several and
    merged.  The split must have happened, and the logits are those of the whole prompt."""
    from return_b200.ext import ops
    d = helpers.make_model_dir(tmp_path, "A", head_dim=64, max_position_embeddings=2048)
    reqs = _requests("A", (1500, 700), 80)
    steps = helpers.portions(reqs, (300, 260, 2, 130))
    used, kernel = set(), ops.attention_prefill_tc5

    def spy(*a, **k):
        used.add(a[14] if len(a) > 14 else k.get("num_splits", 1))
        return kernel(*a, **k)

    monkeypatch.setattr(ops, "attention_prefill_tc5", spy)
    got = _replay(d, "bfloat16", steps, 16)
    _compare(d, reqs, got, "bfloat16")
    assert 1 in used and max(used) > 1, used


def test_first_tokens_of_a_sequence(tmp_path):
    for case in "AB":
        d = helpers.make_model_dir(tmp_path / case, case)
        reqs = _requests(case, (1, 2, 3), 70)
        for dtype in ("float32", "bfloat16"):
            for steps in (helpers.whole(reqs), helpers.tail_decoded(reqs, 32)):
                got = _replay(d, dtype, steps, helpers.CASES[case][2])
                _compare(d, reqs, got, dtype)


def test_trace_run_program(tmp_path):
    """bin/trace_run as a user calls it: JSON lines in, <step>.f32 files and 'done <step>' lines out."""
    d = helpers.make_model_dir(tmp_path, "A")
    reqs = _requests("A", (33, 20), 80)
    steps = helpers.mixed(reqs, max_live=2, portion=7, decode_tail=4, seed=2)
    out = os.path.join(str(tmp_path), "out")
    proc = subprocess.run(
        [sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
         "--out", out, "--max-tokens", str(helpers.pool_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    logits = []
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        path = os.path.join(out, f"{s['step']}.f32")
        if n == 0:
            assert not os.path.exists(path)
            logits.append(None)
        else:
            logits.append(torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n, 256).copy()))
    _compare(d, reqs, helpers.collect(steps, logits), "float32")
