"""Typed model configurations read from an architecture's own config.json keys.

A configuration has two faces.  ``Qwen3Config`` is the typed, validated record of the
keys that a Qwen3 ``config.json`` holds (the reference reads ``model_type``,
``vocab_size``, ``num_key_value_heads``, ``head_dim`` / ``hidden_size`` /
``num_attention_heads`` itself, rollout/engine_actor.py:27 and
rollout/monkey_patch/qwen3.py:114-117, and the rest through the modules it patches).
``DecoderSpec`` (return_b200/parts/spec.py) is what a configuration turns into: the
list of layers, each with its mixer, feed-forward, norm and position encoding, and the
order in which they run.  No size lives anywhere but in these records.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Optional, Tuple


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine does not run."""


_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "num_key_value_heads", "rms_norm_eps")


@dataclass(frozen=True)
class Qwen3Config:
    """The Qwen3 dense decoder (``Qwen3ForCausalLM``), every size explicit."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    hidden_act: str = "silu"
    attention_bias: bool = False
    # per layer: the sliding window in tokens, or None for full attention
    layer_windows: Tuple[Optional[int], ...] = ()
    architectures: Tuple[str, ...] = ("Qwen3ForCausalLM",)
    model_type: str = "qwen3"
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise ConfigError(f"config.json lacks {missing}")
        n_layers = int(raw["num_hidden_layers"])
        heads = int(raw["num_attention_heads"])
        hidden = int(raw["hidden_size"])
        # head_dim falls back to hidden // heads (rollout/monkey_patch/qwen3.py:117)
        head_dim = int(raw["head_dim"]) if raw.get("head_dim") else hidden // heads
        if "rope_theta" in raw:
            theta = float(raw["rope_theta"])
        elif isinstance(raw.get("rope_parameters"), dict) and "rope_theta" in raw["rope_parameters"]:
            theta = float(raw["rope_parameters"]["rope_theta"])
        else:
            raise ConfigError("config.json lacks rope_theta (top level or under rope_parameters)")
        scaling = raw.get("rope_scaling") or {}
        nested = raw.get("rope_parameters") or {}
        rope_type = scaling.get("rope_type", scaling.get("type", nested.get("rope_type", "default")))
        if rope_type not in (None, "default"):
            raise ConfigError(f"rope scaling {rope_type!r} is not implemented (only the default rope)")
        windows = _layer_windows(raw, n_layers)
        arch = tuple(raw.get("architectures") or ("Qwen3ForCausalLM",))
        cfg = cls(
            vocab_size=int(raw["vocab_size"]), hidden_size=hidden,
            intermediate_size=int(raw["intermediate_size"]), num_hidden_layers=n_layers,
            num_attention_heads=heads, num_key_value_heads=int(raw["num_key_value_heads"]),
            head_dim=head_dim, rms_norm_eps=float(raw["rms_norm_eps"]), rope_theta=theta,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            hidden_act=str(raw.get("hidden_act", "silu")),
            attention_bias=bool(raw.get("attention_bias", False)),
            layer_windows=windows, architectures=arch,
            model_type=str(raw.get("model_type", "qwen3")),
            torch_dtype=str(raw.get("torch_dtype", raw.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        def positive(name):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim"):
            positive(name)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for the rotary encoding")
        if self.hidden_act != "silu":
            # the reference hard-wires SiLU (rollout/fused.py:103-127) and ignores the key
            raise ConfigError(f"hidden_act={self.hidden_act!r}: only 'silu' is implemented")
        if self.attention_bias:
            raise ConfigError("attention_bias=true is not implemented (the projections have no bias)")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        if len(self.layer_windows) != self.num_hidden_layers:
            raise ConfigError("layer_windows must name every layer")
        for w in self.layer_windows:
            if w is not None and w <= 0:
                raise ConfigError(f"sliding window must be positive, got {w}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {
            "architectures": list(self.architectures), "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "hidden_act": self.hidden_act, "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta, "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "attention_bias": self.attention_bias, "torch_dtype": self.torch_dtype,
        }
        windows = [w for w in self.layer_windows if w is not None]
        if windows:
            if len(set(windows)) != 1:
                raise ConfigError("config.json holds one sliding_window for all sliding layers")
            d["sliding_window"] = windows[0]
            d["use_sliding_window"] = True
            d["layer_types"] = ["sliding_attention" if w is not None else "full_attention"
                                for w in self.layer_windows]
        else:
            d["sliding_window"] = None
            d["use_sliding_window"] = False
        return d

    def replace(self, **kw) -> "Qwen3Config":
        cfg = dataclasses.replace(self, **kw)
        cfg.validate()
        return cfg


def _layer_windows(raw: dict, n_layers: int):
    """Which layers slide, from ``layer_types`` or ``use_sliding_window``/``max_window_layers``."""
    window = raw.get("sliding_window")
    types = raw.get("layer_types")
    if types is None:
        if raw.get("use_sliding_window") and window:
            first = int(raw.get("max_window_layers", n_layers))
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(n_layers)]
        else:
            types = ["full_attention"] * n_layers
    if len(types) != n_layers:
        raise ConfigError(f"layer_types names {len(types)} layers, num_hidden_layers is {n_layers}")
    out = []
    for t in types:
        if t == "full_attention":
            out.append(None)
        elif t == "sliding_attention":
            if not window:
                raise ConfigError("layer_types has sliding_attention but sliding_window is not set")
            out.append(int(window))
        else:
            raise ConfigError(f"layer type {t!r} is not implemented")
    return tuple(out)
