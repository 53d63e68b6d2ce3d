"""Weights: safetensors by name, dtype rule, one clear error, random-weights folders (no GPU)."""
import json
import os

import pytest
import torch

import helpers
from return_b200.config import registry
from return_b200.models.decoder import DecoderModel
from return_b200.parts.base import BuildEnv
from return_b200.weights import loader
from return_b200.weights.loader import WeightError
from return_b200.weights.safetensors_io import ModelFiles, SafetensorsError, write_safetensors


def _load(model_dir, act=torch.float32):
    arch, cfg = registry.read_config(model_dir)
    model = DecoderModel(arch.decoder_spec(cfg, 32), BuildEnv(act, torch.device("cpu")))
    expected = {n: s for n, (s, _) in loader.checkpoint_shapes(arch, cfg).items()}
    return cfg, model, loader.load_parameters(model.params(), arch.weight_sources(cfg), expected, model_dir,
                                              act, "cpu", arch.ignorable_tensors(cfg))


def test_random_model_folder_roundtrip(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B")
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    from safetensors.torch import load_file           # an independent reader
    theirs = load_file(os.path.join(d, "model.safetensors"))
    ours = ModelFiles(d)
    assert sorted(theirs) == sorted(ours.names())
    for n, t in theirs.items():
        assert torch.equal(t, ours.tensor(n)) and t.dtype == torch.float32
    assert "lm_head.weight" in theirs and theirs["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert abs(float(theirs["model.layers.0.mlp.up_proj.weight"].std()) - 0.02) < 2e-3
    assert abs(float(theirs["model.norm.weight"].mean()) - 1.0) < 0.05
    # same seed, same values; a tensor's value depends on its name and the seed only
    d2 = helpers.make_model_dir(tmp_path / "again", "B")
    assert torch.equal(ModelFiles(d2).tensor("model.norm.weight"), ours.tensor("model.norm.weight"))


def test_tied_model_has_no_head_tensor(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A")
    assert "lm_head.weight" not in ModelFiles(d).names()
    cfg, model, params = _load(d)
    model.bind(params)
    assert model.lm_head is model.embed


def test_fused_parameters_are_concatenations(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B")
    cfg, model, params = _load(d)
    f = ModelFiles(d)
    p = "model.layers.1."
    qkv = torch.cat([f.tensor(p + f"self_attn.{x}_proj.weight") for x in "qkv"])
    assert torch.equal(params["layers.1.mixer.qkv"], qkv)
    # gate and up rows are woven in blocks of 8: [g0..g7, u0..u7, g8..g15, u8..u15, ...]
    g, u = f.tensor(p + "mlp.gate_proj.weight"), f.tensor(p + "mlp.up_proj.weight")
    gu = torch.stack([g.view(-1, 8, 96), u.view(-1, 8, 96)], dim=1).reshape(-1, 96)
    assert torch.equal(params["layers.1.feed_forward.gate_up"], gu)
    assert torch.equal(gu[:8], g[:8]) and torch.equal(gu[8:16], u[:8]) and torch.equal(gu[16:24], g[8:16])


def test_dtype_rule(tmp_path):
    # bf16 file, bf16 run: everything bf16
    d = helpers.make_model_dir(tmp_path / "bf", "A", dtype=torch.bfloat16)
    _, _, params = _load(d, torch.bfloat16)
    assert {t.dtype for t in params.values()} == {torch.bfloat16}
    # fp32 file, bf16 run: matrices become bf16, norm weights stored in 32-bit stay so
    d = helpers.make_model_dir(tmp_path / "f32", "A", dtype=torch.float32)
    _, _, params = _load(d, torch.bfloat16)
    assert params["layers.0.mixer.qkv"].dtype == torch.bfloat16
    assert params["layers.0.mixer_norm.weight"].dtype == torch.float32
    assert params["layers.0.mixer.q_norm.weight"].dtype == torch.float32
    # bf16 file, fp32 run: everything 32-bit
    d = helpers.make_model_dir(tmp_path / "bf2", "A", dtype=torch.bfloat16)
    _, _, params = _load(d, torch.float32)
    assert {t.dtype for t in params.values()} == {torch.float32}


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A")
    f = ModelFiles(d)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    del tensors["model.layers.0.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    tensors["model.layers.1.self_attn.q_norm.weight"] = torch.zeros(32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as e:
        _load(d)
    err = e.value
    assert err.missing == ["model.layers.0.mlp.down_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(err.wrong_shape) == 2
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "down_proj", "inv_freq", "k_proj", "[16, 64]", "[32, 64]"):
        assert word in msg


def test_untied_model_without_head_is_an_error_and_tied_head_copy_is_ignored(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B")
    f = ModelFiles(d)
    tensors = {n: f.tensor(n) for n in f.names() if n != "lm_head.weight"}
    f.close()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError, match="lm_head.weight"):
        _load(d)
    d = helpers.make_model_dir(tmp_path / "t", "A")
    f = ModelFiles(d)
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    _load(d)
    # a tied model whose file holds another head: loading it would silently drop that head
    tensors["lm_head.weight"] = tensors["lm_head.weight"].clone()
    tensors["lm_head.weight"][3, 5] += 0.5
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError, match="lm_head.weight differs from model.embed_tokens.weight"):
        _load(d)


def test_sharded_checkpoint_and_missing_shard(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A")
    f = ModelFiles(d)
    names = f.names()
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for shard, ns in shards.items():
        write_safetensors(os.path.join(d, shard), [(n, f.tensor(n)) for n in ns])
    f.close()
    os.remove(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {n: s for s, ns in shards.items() for n in ns}}, fh)
    _load(d)
    os.remove(os.path.join(d, "model-00002-of-00002.safetensors"))
    with pytest.raises(SafetensorsError, match="missing"):
        _load(d)


def test_integer_tables_become_int32(tmp_path):
    p = os.path.join(str(tmp_path), "x.safetensors")
    write_safetensors(p, [("table", torch.arange(6, dtype=torch.int64).view(2, 3)), ("w", torch.ones(2, dtype=torch.float32))])
    assert loader._target_dtype(torch.int64, "matrix", torch.bfloat16) == torch.int32
    assert loader._target_dtype(torch.float32, "vector", torch.bfloat16) == torch.float32
    assert loader._target_dtype(torch.float32, "matrix", torch.bfloat16) == torch.bfloat16
    assert loader._target_dtype(torch.bfloat16, "vector", torch.float32) == torch.float32


def test_broken_file_is_reported(tmp_path):
    d = str(tmp_path)
    with open(os.path.join(d, "model.safetensors"), "wb") as fh:
        fh.write(b"\xff" * 5)
    with pytest.raises(SafetensorsError):
        ModelFiles(d)
    with pytest.raises(SafetensorsError, match="neither"):
        ModelFiles(os.path.join(d, "nothing"))
