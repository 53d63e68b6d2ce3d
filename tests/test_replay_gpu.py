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

TOL = {"float32": 1e-4, "bfloat16": 6e-2}


def _requests(name, lens, seed):
    vocab = helpers.CASES[name][0]["vocab_size"]
    return {f"r{i}": helpers.random_ids(vocab, n, seed + i) for i, n in enumerate(lens)}


def _replay(model_dir, dtype, steps, page, pool=None, poison=True, max_reside=8):
    from return_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(model_dir, dtype, pool or helpers.pool_tokens(steps), page_size=page,
                       max_reside=max_reside, poison=poison)
    out = []
    for st in steps:
        lg = rp.run_step(st)
        out.append(None if lg is None else lg.float().cpu())
        rp.runner.manager.check()
    assert rp.runner.manager.pages_used() == [0] * len(rp.runner.manager.groups)
    return helpers.collect(steps, out)


def _compare(model_dir, requests, got, dtype):
    worst = 0.0
    for rid, ids in requests.items():
        ref = helpers.plain_logits(model_dir, ids)
        assert got[rid].shape == ref.shape
        err = (got[rid] - ref).abs().max(dim=1).values
        assert torch.isfinite(got[rid]).all(), f"{rid}: non-finite logits"
        bad = (err > TOL[dtype]).nonzero()
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
