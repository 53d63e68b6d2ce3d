"""Plain, slow, whole-sequence implementation of the Qwen3 dense decoder.

This file is the oracle of the test-suite.  It is written from the formulas of
wenhaoli-xmu/ReTurn's rollout engine (its replaced forwards, its Triton kernels
and its own test oracles); every function cites the file and lines it restates.
It has no cache, no batching and no kernels, runs on the CPU in float32 (or in
float64 when asked), and shares no code with the ``return_b200`` package: it
reads ``config.json`` as a plain dict and ``model.safetensors`` through the
``safetensors`` library.

The reference keeps its bfloat16 roundings inside its kernels (rope tables,
rotated q/k, softmax probabilities).  This oracle does not round anywhere: it is
the exact formula, and the engine's 32-bit path is compared with it tightly, its
bfloat16 path loosely.

Two things go beyond what the reference runs and rest on their definition here:
  * a sliding window (the reference asserts that there is none,
    rollout/monkey_patch/qwen3.py:130-132): a key at position j is visible to
    a query at position i iff ``i - window < j <= i``;
  * a layer schedule (a list of entries ``(layer, cache_of)``): an entry whose
    ``cache_of`` names an earlier entry attends over that entry's keys and
    values instead of computing its own.
``tests/golden/`` holds logits that the reference's own code produced on a tiny
random model; ``tests/test_plain.py`` compares this file with them.
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- config / weights

def read_config(model_dir):
    """config.json as a dict with the defaults the reference relies on.

    head_dim falls back to hidden_size // num_attention_heads
    (rollout/monkey_patch/qwen3.py:117); rope_theta may sit at top level or under
    ``rope_parameters``.
    """
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    if "rope_theta" not in c:
        c["rope_theta"] = c["rope_parameters"]["rope_theta"]
    c.setdefault("tie_word_embeddings", False)
    return c


def layer_windows(c):
    """Per layer: the sliding window, or None for full attention."""
    n = c["num_hidden_layers"]
    types = c.get("layer_types")
    w = c.get("sliding_window")
    if types is None:
        if c.get("use_sliding_window") and w:
            first = c.get("max_window_layers", n)
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(n)]
        else:
            types = ["full_attention"] * n
    return [w if t == "sliding_attention" else None for t in types]


def read_weights(model_dir, dtype=torch.float32):
    """All tensors of model.safetensors by their Hugging Face names, cast to ``dtype``.

    The tied head is an alias of the embedding (rollout/engine_actor.py:46).
    """
    from safetensors.torch import load_file
    w = {k: v.to(dtype) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return w


# --------------------------------------------------------------------------- parts

def embedding(w, ids):
    """x0 = E[ids], no scaling (rollout/monkey_patch/qwen3.py:73-75)."""
    return w["model.embed_tokens.weight"][torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w, eps inside the root, weight not offset.

    rollout/fused.py:13-17 with OFFSET=0 (rollout/monkey_patch/qwen3.py:15-17).
    """
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def linear(x, weight):
    """y = x W^T, weight is [out, in], no bias (rollout/monkey_patch/qwen3.py:29-31,56)."""
    return x @ weight.T


def rope_tables(positions, head_dim, theta, dtype=torch.float32):
    """cos, sin of pos * theta^(-i/(D/2)), i = 0..D/2-1.

    rollout/monkey_patch/qwen3.py:121-127 (outer(pos, inv_freq), attention scaling 1)
    with inv_freq as in rollout/utils/test_decode.py:14-17.
    """
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=dtype) / half))
    ang = torch.outer(torch.as_tensor(positions, dtype=dtype), inv_freq)
    return ang.cos(), ang.sin()


def rope_rotate(x, cos, sin):
    """Half-split rotation of x [T, heads, D] with cos/sin [T, D/2].

    o1 = x1 cos - x2 sin, o2 = x2 cos + x1 sin, the same angle index for both halves
    (rollout/attention.py:10-25; rollout/utils/test_decode.py:23-30).
    """
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def attention_scores_softmax_pv(q, k, v, q_pos, k_pos, scale, window=None):
    """Causal grouped-query attention of rotated q [Tq,Hq,D] over rotated k, v [Tk,Hkv,D].

    kv head of q head h is h // (Hq/Hkv); s = q.k * scale; a key is visible iff
    pos_k <= pos_q; softmax with natural exp; o = p v
    (rollout/attention.py:125-139; oracle rollout/utils/test_decode.py:41-50 and
    opd/test_parallel.py:14-42).  ``window`` adds the lower bound pos_k > pos_q - window.
    """
    group = q.shape[1] // k.shape[1]
    kk = k.repeat_interleave(group, dim=1)
    vv = v.repeat_interleave(group, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    q_pos = torch.as_tensor(q_pos)
    k_pos = torch.as_tensor(k_pos)
    hidden = k_pos[None, :] > q_pos[:, None]
    if window is not None:
        hidden = hidden | (k_pos[None, :] <= q_pos[:, None] - window)
    s = s.masked_fill(hidden[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", s.softmax(-1), vv)


def attention_project_qkv(c, w, prefix, x, positions):
    """q, k, v of one layer: projections, per-head q/k RMSNorm, then rotation.

    rollout/monkey_patch/qwen3.py:29-31 (norm over head_dim before RoPE, v has none),
    rotation as rope_rotate.  Returns rotated q [T,Hq,D], rotated k [T,Hkv,D], v [T,Hkv,D].
    """
    D, Hq, Hkv, eps = c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"], c["rms_norm_eps"]
    T = x.shape[0]
    q = rms_norm(linear(x, w[prefix + "self_attn.q_proj.weight"]).view(T, Hq, D), w[prefix + "self_attn.q_norm.weight"], eps)
    k = rms_norm(linear(x, w[prefix + "self_attn.k_proj.weight"]).view(T, Hkv, D), w[prefix + "self_attn.k_norm.weight"], eps)
    v = linear(x, w[prefix + "self_attn.v_proj.weight"]).view(T, Hkv, D)
    cos, sin = rope_tables(positions, D, c["rope_theta"], dtype=x.dtype)
    return rope_rotate(q, cos, sin), rope_rotate(k, cos, sin), v


def swiglu_mlp(w, prefix, x):
    """down( silu(gate(x)) * up(x) ) (rollout/monkey_patch/qwen3.py:20-22; rollout/fused.py:103-127)."""
    g = linear(x, w[prefix + "mlp.gate_proj.weight"])
    u = linear(x, w[prefix + "mlp.up_proj.weight"])
    return linear(g * torch.sigmoid(g) * u, w[prefix + "mlp.down_proj.weight"])


def decoder_layer(c, w, layer, x, positions, window=None, shared_kv=None):
    """One block: x += attn(norm(x)); x += mlp(norm(x)) (rollout/monkey_patch/qwen3.py:59-68).

    Returns the new stream and the (k, v) this layer attended over.
    """
    p = f"model.layers.{layer}."
    eps = c["rms_norm_eps"]
    a = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q, k, v = attention_project_qkv(c, w, p, a, positions)
    if shared_kv is not None:
        k, v = shared_kv
    scale = c["head_dim"] ** -0.5      # rollout/attention.py:195 (fallback 1/sqrt(D))
    o = attention_scores_softmax_pv(q, k, v, positions, positions, scale, window)
    x = x + linear(o.reshape(x.shape[0], -1), w[p + "self_attn.o_proj.weight"])
    b = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(w, p, b)
    return x, (k, v)


def lm_head(c, w, h):
    """logits = h Wlm^T; the tied head is the embedding (rollout/model.py:286-290; engine_actor.py:46)."""
    name = "model.embed_tokens.weight" if c["tie_word_embeddings"] else "lm_head.weight"
    return linear(h, w[name])


def forward_logits(c, w, ids, schedule=None):
    """Logits [T, V] at every position of one whole sequence (rollout/monkey_patch/qwen3.py:71-81).

    ``schedule``: list of (layer, cache_of) entries; default one entry per layer in order.
    """
    x = embedding(w, ids)
    positions = torch.arange(len(ids))
    windows = layer_windows(c)
    if schedule is None:
        schedule = [(i, None) for i in range(c["num_hidden_layers"])]
    kvs = []
    for layer, cache_of in schedule:
        shared = kvs[cache_of] if cache_of is not None else None
        x, kv = decoder_layer(c, w, layer, x, positions, windows[layer], shared)
        kvs.append(kv)
    x = rms_norm(x, w["model.norm.weight"], c["rms_norm_eps"])
    return lm_head(c, w, x)


# --------------------------------------------------------------------------- sampling

def filtered_probs(logits, temperature, top_k, top_p):
    """The distribution the reference samples from, for one row of raw logits.

    rollout/model.py:15-61: divide by temperature; keep the top_k largest (0 = all);
    sort descending, drop column j iff the mass of the columns before it exceeds top_p
    (the column that crosses top_p stays, the first always stays); renormalise.
    Returns probabilities over the vocabulary (zeros for dropped tokens).
    """
    x = logits.double() / temperature
    V = x.numel()
    k = top_k if top_k > 0 else V
    vals, idx = x.sort(descending=True, stable=True)
    vals = vals.clone()
    vals[k:] = float("-inf")
    cum = vals.softmax(-1).cumsum(-1)
    remove = torch.zeros(V, dtype=torch.bool)
    remove[1:] = cum[:-1] > top_p
    vals[remove] = float("-inf")
    probs = torch.zeros(V, dtype=torch.double)
    probs[idx] = vals.softmax(-1)
    return probs


def greedy(logits):
    """argmax of the raw logits (rollout/model.py:23-26)."""
    return int(torch.as_tensor(logits).argmax(-1))


def logprob(logits, token):
    """log_softmax of the raw float logits at the chosen token, no temperature (rollout/model.py:64-67)."""
    return float(torch.log_softmax(logits.double(), -1)[token])


def greedy_generate(c, w, prompt, max_new_tokens, stop_ids=()):
    """Greedy continuation by recomputing the whole sequence for every token.

    Stops at max_new_tokens or when the output ends with one of the stop sequences;
    the stop tokens stay in the output (rollout/engine.py:49-57).
    """
    ids, out = list(prompt), []
    while len(out) < max_new_tokens:
        t = greedy(forward_logits(c, w, ids)[-1])
        ids.append(t)
        out.append(t)
        if any(len(s) and out[-len(s):] == list(s) for s in stop_ids):
            break
    return out
