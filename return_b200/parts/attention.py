"""Causal grouped-query attention over the paged cache (rollout/monkey_patch/qwen3.py:25-56).

Projections q, k, v as one fused product (the reference runs three, :29-31; the fused weight is
their row-wise concatenation), per-head RMSNorm of q and k before the rotation (:29-30),
rotation and cache write in one kernel (for a step of single tokens: inside the attention kernel),
attention over the block table, output projection
(:55-56).  Sizes, window, norm and position encoding come from the specification.
"""
from __future__ import annotations

import torch

from ..ext import ops
from .base import MIXERS, NORMS, POSITION_ENCODINGS, KVCacheNeed, Mixer, ParamSpec, Tiling


@MIXERS.register("attention")
class PagedAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_kv_heads={spec.num_kv_heads}")
        if spec.head_dim % 16 or not (16 <= spec.head_dim <= 256):
            raise ValueError(f"head_dim={spec.head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        self.q_norm = NORMS.build(spec.qk_norm, env) if spec.qk_norm is not None else None
        self.k_norm = NORMS.build(spec.qk_norm, env) if spec.qk_norm is not None else None
        if spec.qk_norm is not None and (spec.qk_norm.kind != "rmsnorm" or spec.qk_norm.size != spec.head_dim):
            raise ValueError("the fused q/k norm is an RMSNorm over head_dim")
        self.position = POSITION_ENCODINGS.build(spec.position, env) if spec.position is not None else None
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim

    # ------------------------------------------------------------------ parameters and cache
    def params(self):
        s = self.spec
        p = {"qkv": ParamSpec((self.q_size + 2 * self.kv_size, s.hidden_size)),
             "o": ParamSpec((s.hidden_size, self.q_size))}
        if self.q_norm is not None:
            p["q_norm.weight"] = self.q_norm.params()["weight"]
            p["k_norm.weight"] = self.k_norm.params()["weight"]
        return p

    def bind(self, tensors):
        self.p_qkv = tensors["qkv"]
        self.p_o = tensors["o"]
        if self.q_norm is not None:
            self.q_norm.bind({"weight": tensors["q_norm.weight"]})
            self.k_norm.bind({"weight": tensors["k_norm.weight"]})

    def cache_need(self):
        return KVCacheNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def batch_tilings(self):
        """The row blocks of the tensor-core kernel for prompt portions that this head size runs on."""
        if self.env.act_dtype != torch.bfloat16:
            return {}
        if self.spec.head_dim in ops.TC5_ATTENTION_HEAD_DIMS:
            return {ops.TILES_TC5: Tiling(ops.TC5_TILE_ROWS, heaviest_first=True)}
        return {ops.TILES_MMA: Tiling(ops.MMA_TILE_ROWS)}

    def graph_variant(self, n_tokens, longest_context):
        """A captured step cannot change the grid of the split-KV decode kernel: the number of key splits
        is fixed per captured graph."""
        if self.env.act_dtype != torch.bfloat16:
            return {}
        s = self.spec
        return {ops.decode_splits_key(s.num_heads, s.num_kv_heads, s.window):
                ops.decode_splits_for(n_tokens, longest_context, s.num_heads, s.num_kv_heads, s.window)}

    # ------------------------------------------------------------------ one step
    def forward(self, x, ctx):
        T = x.shape[0]
        qkv = ctx.buffer("attention.qkv", (T, self.q_size + 2 * self.kv_size), x.dtype, x.device)
        ops.linear(x, self.p_qkv, qkv)
        o = self.core(qkv, ctx)
        y = ctx.buffer("attention.y", (T, self.spec.hidden_size), x.dtype, x.device)
        ops.linear(o, self.p_o, y)
        return y

    # A mixer that is "product, something in the middle, product" says so, and a block may then run the two
    # products in kernels of its own choosing (fused with the norms around them).
    def in_projection(self):
        """(weight [q + 2 kv, hidden], name of the buffer its output goes to)."""
        return self.p_qkv, "attention.qkv"

    def out_projection(self):
        return self.p_o

    def core(self, qkv, ctx):
        """From the projections [T, q + 2 kv] to the attention output [T, q]: per-head norm, position encoding,
        cache write, attention over the block table."""
        s, b, kv = self.spec, ctx.batch, ctx.kv
        T = qkv.shape[0]
        qw = self.q_norm.p_weight if self.q_norm is not None else None
        kw = self.k_norm.p_weight if self.k_norm is not None else None
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        offset = s.qk_norm.offset if s.qk_norm is not None else 0.0
        tables = self.position.rotary_tables() if self.position is not None else None
        o = ctx.buffer("attention.o", (T, self.q_size), qkv.dtype, qkv.device)
        if (tables is not None or self.position is None) and ops.decode_only(b, qkv.dtype, s.num_heads, s.num_kv_heads, s.window):
            # single decoded tokens only: norm, rotation, cache write and attention are one kernel
            cos, sin, rot = tables if tables is not None else (None, None, 0)
            ops.attention_decode_fused(qkv, qw, kw, eps, offset, cos, sin, rot, kv.k, kv.v, b, kv.block_table,
                                       kv.page_size, o, s.num_heads, s.num_kv_heads, s.head_dim, s.scale, s.window,
                                       write_kv=ctx.write_cache)
            return o
        if tables is not None or self.position is None:
            cos, sin, rot = tables if tables is not None else (None, None, 0)
            ops.qk_norm_rope_write(qkv, qw, kw, eps, cos, sin, rot, b.pos, b.tok_seg, kv.block_table,
                                   kv.page_size, kv.k, kv.v, s.num_heads, s.num_kv_heads, s.head_dim,
                                   write_kv=ctx.write_cache, offset=offset)
        else:
            # an encoding that is not a rotation of pairs: norm, then the encoding's own in-place
            # step on q and k, then the cache write
            ops.qk_norm_rope_write(qkv, qw, kw, eps, None, None, 0, b.pos, b.tok_seg, kv.block_table,
                                   kv.page_size, kv.k, kv.v, s.num_heads, s.num_kv_heads, s.head_dim,
                                   write_kv=False, offset=offset)
            self.position.apply(qkv, b, s.num_heads, s.num_kv_heads, s.head_dim)
            if ctx.write_cache:
                ops.qk_norm_rope_write(qkv, None, None, 0.0, None, None, 0, b.pos, b.tok_seg, kv.block_table,
                                       kv.page_size, kv.k, kv.v, s.num_heads, s.num_kv_heads, s.head_dim,
                                       write_kv=True)
        ops.paged_attention(qkv, kv.k, kv.v, b, kv.block_table, kv.page_size, o, s.num_heads,
                            s.num_kv_heads, s.head_dim, s.scale, s.window)
        return o
