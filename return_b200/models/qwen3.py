"""The Qwen3 dense decoder as a ``DecoderSpec`` plus the map from checkpoint tensor names to the
parts' parameters.

Layer order and formulas: rollout/monkey_patch/qwen3.py:59-81.  Tensor names are those of a
Hugging Face ``Qwen3ForCausalLM`` checkpoint, which the reference loads
(rollout/engine_actor.py:14-21).  Fusions at load: q, k and v projections into one ``qkv``
matrix (rows q, then k, then v), gate and up projections into ``gate_up`` (the reference
concatenates them, rollout/monkey_patch/qwen3.py:99-105; here their rows are interleaved in blocks
of 8 when the intermediate size allows, see ``SwiGLUSpec``).
"""
from __future__ import annotations

from typing import Dict, Optional

from ..config.model_config import Qwen3Config
from ..parts.spec import (AttentionSpec, BlockSpec, DecoderSpec, NormSpec, RopeSpec, ScheduleEntry,
                          SwiGLUSpec)
from ..weights.loader import Source


def _gate_up_interleave(cfg: Qwen3Config) -> int:
    return 8 if cfg.intermediate_size % 8 == 0 else 0


def decoder_spec(cfg: Qwen3Config, max_positions: Optional[int] = None) -> DecoderSpec:
    D = cfg.head_dim
    rope = RopeSpec(rotary_dim=D, theta=cfg.rope_theta,
                    max_positions=max_positions or cfg.max_position_embeddings)
    head_norm = NormSpec(size=D, eps=cfg.rms_norm_eps)
    stream_norm = NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps)
    ffn = SwiGLUSpec(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                     interleave=_gate_up_interleave(cfg))
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = AttentionSpec(hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                              num_kv_heads=cfg.num_key_value_heads, head_dim=D,
                              scale=D ** -0.5,       # rollout/attention.py:195
                              window=cfg.layer_windows[i], qk_norm=head_norm, position=rope)
        layers.append(BlockSpec(mixer=mixer, feed_forward=ffn, mixer_norm=stream_norm,
                                feed_forward_norm=stream_norm))
    return DecoderSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=tuple(layers),
                       schedule=DecoderSpec.in_order(cfg.num_hidden_layers), final_norm=stream_norm,
                       tie_embeddings=cfg.tie_word_embeddings)


def weight_sources(cfg: Qwen3Config) -> Dict[str, Source]:
    """Model parameter -> the checkpoint tensors that fill it (concatenated along dim 0)."""
    m: Dict[str, Source] = {"embed": Source(("model.embed_tokens.weight",)),
                            "final_norm.weight": Source(("model.norm.weight",))}
    if not cfg.tie_word_embeddings:
        m["lm_head"] = Source(("lm_head.weight",))
    for i in range(cfg.num_hidden_layers):
        src, dst = f"model.layers.{i}.", f"layers.{i}."
        m[dst + "mixer.qkv"] = Source((src + "self_attn.q_proj.weight", src + "self_attn.k_proj.weight",
                                       src + "self_attn.v_proj.weight"))
        m[dst + "mixer.o"] = Source((src + "self_attn.o_proj.weight",))
        m[dst + "mixer.q_norm.weight"] = Source((src + "self_attn.q_norm.weight",))
        m[dst + "mixer.k_norm.weight"] = Source((src + "self_attn.k_norm.weight",))
        m[dst + "feed_forward.gate_up"] = Source((src + "mlp.gate_proj.weight", src + "mlp.up_proj.weight"),
                                                 interleave=_gate_up_interleave(cfg))
        m[dst + "feed_forward.down"] = Source((src + "mlp.down_proj.weight",))
        m[dst + "mixer_norm.weight"] = Source((src + "input_layernorm.weight",))
        m[dst + "feed_forward_norm.weight"] = Source((src + "post_attention_layernorm.weight",))
    return m


def ignorable_tensors(cfg: Qwen3Config):
    """Checkpoint tensors that may be present without being used, each with the tensor it must equal: a tied
    head saved beside the embedding."""
    return {"lm_head.weight": "model.embed_tokens.weight"} if cfg.tie_word_embeddings else {}


def split_rows(cfg: Qwen3Config, param: str):
    """Rows that each checkpoint tensor has inside a fused parameter."""
    if param.endswith("mixer.qkv"):
        q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
        return [q, kv, kv]
    return None
