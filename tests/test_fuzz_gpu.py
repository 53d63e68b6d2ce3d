"""Random tiny configurations and random traces against the plain implementation: sizes that no
fixed case has (head sizes 16 to 128 in steps of 16, odd head counts and groups, windows, page sizes,
tied and untied heads), cut into mixed batches with few pages."""
import os
import random

import pytest
import torch

import helpers
from helpers import plain

pytestmark = pytest.mark.gpu


def _random_config(rng: random.Random):
    head_dim = rng.choice([16, 32, 48, 64, 80, 128])
    kv = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 3, 5])
    layers = rng.choice([1, 2, 3])
    hidden = 8 * rng.randint(3, 12)
    raw = dict(vocab_size=rng.randint(40, 300), hidden_size=hidden, intermediate_size=8 * rng.randint(2, 20) + rng.choice([0, 4]),
               num_hidden_layers=layers, num_attention_heads=kv * group, num_key_value_heads=kv, head_dim=head_dim,
               rope_theta=rng.choice([10000.0, 500000.0]), rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-4]),
               tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=512)
    if rng.random() < 0.4:
        raw.update(sliding_window=rng.randint(5, 40), use_sliding_window=True,
                   layer_types=[rng.choice(["sliding_attention", "full_attention"]) for _ in range(layers)])
    return raw


@pytest.mark.parametrize("seed", list(range(10)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration_and_trace(tmp_path, seed, dtype):
    from return_b200.config.model_config import Qwen3Config
    from return_b200.engine.replay import TraceReplayer
    from return_b200.weights import loader
    rng = random.Random(1000 + seed)
    raw = _random_config(rng)
    cfg = Qwen3Config.from_dict(raw)
    d = loader.write_random_model(os.path.join(str(tmp_path), "m"), cfg, seed, torch.float32)
    lens = [rng.randint(1, 90) for _ in range(rng.randint(2, 5))]
    reqs = {f"q{i}": helpers.random_ids(raw["vocab_size"], n, 77 * seed + i) for i, n in enumerate(lens)}
    steps = helpers.mixed(reqs, max_live=rng.randint(1, 4), portion=rng.randint(2, 40), decode_tail=rng.randint(0, 12), seed=seed)
    page = rng.choice([4, 8, 16, 32])
    rp = TraceReplayer(d, dtype, helpers.pool_tokens(steps), page_size=page, max_reside=4)
    rp.runner.storage.poison()
    got = helpers.collect(steps, [None if (lg := rp.run_step(s)) is None else lg.cpu() for s in steps])
    for rid, ids in reqs.items():
        want = helpers.plain_logits(d, ids)
        # bfloat16: a twelfth of the logits' standard deviation (the widths differ, so the logits' scale does)
        tol = 2e-4 if dtype == "float32" else float(want.std()) / 12
        err = (got[rid] - want).abs().max().item()
        assert err < tol, (raw, rid, len(ids), page, err, tol)
    assert rp.runner.manager.pages_used() == [0] * len(rp.runner.manager.groups)
