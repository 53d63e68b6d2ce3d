"""The plain implementation against the reference's own code (golden files) and against itself."""
import json
import os

import pytest
import torch

import helpers
from helpers import plain

GOLDEN = os.path.join(helpers.HERE, "golden")


@pytest.mark.parametrize("case", ["ref_case_a", "ref_case_b"])
def test_plain_matches_reference_golden(case):
    """tests/golden/make_golden.py ran the reference's forwards, kernels and cache on these weights."""
    d = os.path.join(GOLDEN, case)
    with open(os.path.join(d, "golden.json")) as f:
        gold = json.load(f)
    c, w = plain.read_config(d), plain.read_weights(d)
    worst = 0.0
    for i, prompt in enumerate(gold["prompts"]):
        ids = prompt + gold["outputs"][i]
        logits = plain.forward_logits(c, w, ids)
        for rec in gold["records"]:
            if rec["request"] != i:
                continue
            ref = torch.tensor(rec["logits"])
            worst = max(worst, (logits[rec["position"]] - ref).abs().max().item())
        # the reference generated greedily: its tokens are the plain argmax too
        for k, tok in enumerate(gold["outputs"][i]):
            assert plain.greedy(logits[len(prompt) - 1 + k]) == tok
    assert worst < 5e-6, worst


def test_plain_is_causal_and_prefix_stable(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B")
    ids = helpers.random_ids(384, 40, 5)
    full = helpers.plain_logits(d, ids)
    part = helpers.plain_logits(d, ids[:17])
    assert torch.allclose(full[:17], part, atol=2e-6)


def test_plain_float64_agrees(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A")
    ids = helpers.random_ids(256, 33, 1)
    a = helpers.plain_logits(d, ids)
    b = helpers.plain_logits(d, ids, dtype=torch.float64)
    assert (a.double() - b).abs().max() < 1e-5


def test_plain_window_hides_far_keys(tmp_path):
    """With every layer sliding, a token further back than the window cannot change the logits."""
    d = helpers.make_model_dir(tmp_path, "C", layer_types=["sliding_attention"] * 4)
    ids = helpers.random_ids(200, 60, 2)
    other = list(ids)
    other[3] = (other[3] + 1) % 200
    a, b = helpers.plain_logits(d, ids), helpers.plain_logits(d, other)
    # 4 layers of window 24 reach back 4 * 23 positions at most
    assert torch.equal(a[3 + 4 * 23 + 1:], b[3 + 4 * 23 + 1:]) if len(ids) > 3 + 4 * 23 + 1 else True
    d2 = helpers.make_model_dir(tmp_path / "w", "C", num_hidden_layers=1, layer_types=["sliding_attention"])
    a, b = helpers.plain_logits(d2, ids), helpers.plain_logits(d2, other)
    assert torch.equal(a[3 + 24:], b[3 + 24:])
    assert not torch.equal(a[3:3 + 24], b[3:3 + 24])


def test_plain_schedule_shared_cache(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A")
    ids = helpers.random_ids(256, 12, 3)
    base = helpers.plain_logits(d, ids)
    twice = helpers.plain_logits(d, ids, schedule=[(0, None), (1, None), (0, None)])
    shared = helpers.plain_logits(d, ids, schedule=[(0, None), (1, 0)])
    assert not torch.allclose(base, twice) and not torch.allclose(base, shared)


def test_filtered_probs_semantics():
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0])
    p = plain.filtered_probs(logits, 1.0, 0, 1.0)
    assert torch.allclose(p, logits.double().softmax(-1))
    p = plain.filtered_probs(logits, 1.0, 2, 1.0)
    assert (p > 0).tolist() == [True, True, False, False, False] and abs(p.sum() - 1) < 1e-12
    # top_p: the token that crosses top_p stays
    sm = logits.double().softmax(-1)
    p = plain.filtered_probs(logits, 1.0, 0, float(sm[0]) + 1e-3)
    assert (p > 0).tolist() == [True, True, False, False, False]
    p = plain.filtered_probs(logits, 1.0, 0, 1e-6)
    assert (p > 0).tolist() == [True, False, False, False, False]
    assert plain.greedy(logits) == 0 and abs(plain.logprob(logits, 1) - float(torch.log_softmax(logits, -1)[1])) < 1e-6
