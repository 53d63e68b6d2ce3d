"""Configuration and registry (no GPU)."""
import json

import pytest

import helpers
from return_b200.config import registry
from return_b200.config.model_config import ConfigError, Qwen3Config
from return_b200.engine.config import EngineConfig
import return_b200.parts as parts
from return_b200.models import qwen3


def test_reads_every_size_from_config_json(tmp_path):
    for name in "ABC":
        raw = helpers.CASES[name][0]
        cfg = Qwen3Config.from_dict(dict(raw))
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
            assert getattr(cfg, k) == raw[k]
        again = Qwen3Config.from_dict(cfg.to_dict())
        assert again == cfg


def test_head_dim_fallback_and_nested_rope_theta():
    raw = dict(helpers.TINY_A)
    del raw["head_dim"], raw["rope_theta"]
    raw["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.head_dim == 64 // 4 and cfg.rope_theta == 12345.0


def test_windows_from_layer_types_and_max_window_layers():
    cfg = helpers.tiny_config("C")
    assert cfg.layer_windows == (24, None, 24, None)
    raw = dict(helpers.TINY_B, sliding_window=32, use_sliding_window=True, max_window_layers=1)
    assert Qwen3Config.from_dict(raw).layer_windows == (None, 32, 32)
    raw = dict(helpers.TINY_B, sliding_window=32, use_sliding_window=False)
    assert Qwen3Config.from_dict(raw).layer_windows == (None, None, None)


@pytest.mark.parametrize("change, words", [
    (dict(num_key_value_heads=3), "multiple"),
    (dict(hidden_act="gelu"), "silu"),
    (dict(attention_bias=True), "bias"),
    (dict(head_dim=15), "even"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope scaling"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(layer_types=["linear_attention", "full_attention"]), "not implemented"),
])
def test_rejects_what_it_does_not_run(change, words):
    with pytest.raises(ConfigError, match=words):
        Qwen3Config.from_dict(dict(helpers.TINY_A, **change))


def test_missing_key_is_named():
    raw = dict(helpers.TINY_A)
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        Qwen3Config.from_dict(raw)


def test_registry_resolves_by_architecture_then_model_type(tmp_path):
    assert registry.resolve({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert registry.resolve({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(ValueError, match="Qwen3ForCausalLM"):
        registry.resolve({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    d = helpers.make_model_dir(tmp_path, "B")
    arch, cfg = registry.read_config(d)
    assert arch.name == "Qwen3ForCausalLM" and cfg.hidden_size == 96


def test_decoder_spec_is_chosen_layer_by_layer():
    cfg = helpers.tiny_config("C")
    spec = qwen3.decoder_spec(cfg, 128)
    assert [b.mixer.window for b in spec.layers] == [24, None, 24, None]
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and all(e.cache_of is None for e in spec.schedule)
    m = spec.layers[0].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.qk_norm.eps, m.position.theta) == (5, 1, 48, 3e-6, 50000.0)
    assert abs(m.scale - 48 ** -0.5) < 1e-12
    spec.validate()


def test_schedule_validation():
    cfg = helpers.tiny_config("A")
    spec = qwen3.decoder_spec(cfg, 64)
    import dataclasses
    bad = dataclasses.replace(spec, schedule=(parts.ScheduleEntry(0), parts.ScheduleEntry(1, cache_of=1)))
    with pytest.raises(ValueError):
        bad.validate()
    bad = dataclasses.replace(spec, schedule=(parts.ScheduleEntry(0), parts.ScheduleEntry(5)))
    with pytest.raises(ValueError):
        bad.validate()


def test_engine_config_checks():
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(max_token=8, page_size=16)
    assert EngineConfig(max_token=1024, page_size=16).num_pages == 64


def test_layers_share_one_pair_of_rotary_tables():
    """Every layer's attention builds its own position encoding from the same specification; the
    tables exist once per device, not once per layer."""
    import torch
    from return_b200.parts import rope
    from return_b200.parts.base import BuildEnv
    from return_b200.parts.spec import RopeSpec
    env = BuildEnv(torch.float32, torch.device("cpu"))
    spec = RopeSpec(rotary_dim=16, theta=10000.0, max_positions=64)
    a, b = rope.RotaryEncoding(spec, env), rope.RotaryEncoding(spec, env)
    ca, sa, _ = a.rotary_tables()
    cb, sb, _ = b.rotary_tables()
    assert ca.data_ptr() == cb.data_ptr() and sa.data_ptr() == sb.data_ptr()
    other = rope.RotaryEncoding(RopeSpec(rotary_dim=16, theta=500000.0, max_positions=64), env).rotary_tables()
    assert other[0].data_ptr() != ca.data_ptr()
