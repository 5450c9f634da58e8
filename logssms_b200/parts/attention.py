"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed
from ..ops import kernels as K
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import MATRIX, ParamSpec, Part
from .rope import NoPositionEncoding


@MIXERS.register("attention")
class Attention(Part):
    """q/k/v projection -> key multiplier + rotation + store into the page cache (one kernel) ->
    causal attention over the cache -> output projection.

    Checkpoint tensors `q_proj / k_proj / v_proj .weight` are concatenated (rows q | k | v) at
    bind time, as the reference merges them at load (python/logssms/models/weight.py:27-31);
    the flow is python/logssms/layers/attention.py:115-167."""
    takes_normed_rows = True      # forward() passes its input straight into a product
    joins_residual = True         # forward() takes `join=`: its last product may add the residual in its epilogue
    kernels = ("rope", "attention_decode", "attention_decode_fused", "attention_prefill", "attention_prefill_tc", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        s = spec
        self.q_size, self.kv_size = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        self.scale = s.softmax_scale if s.softmax_scale is not None else s.head_dim ** -0.5
        if s.position is None:
            self.position = NoPositionEncoding()
        else:
            key = ("position", s.position)
            if shared is not None and key in shared:
                self.position = shared[key]
            else:
                self.position = POSITION_ENCODINGS.get(s.position.kind)(s.position)
                if shared is not None:
                    shared[key] = self.position
        self.qkv_weight = self.o_weight = None

    def param_specs(self):
        s = self.spec
        return {
            "q_proj.weight": ParamSpec((self.q_size, s.hidden_size), MATRIX),
            "k_proj.weight": ParamSpec((self.kv_size, s.hidden_size), MATRIX),
            "v_proj.weight": ParamSpec((self.kv_size, s.hidden_size), MATRIX),
            "o_proj.weight": ParamSpec((s.hidden_size, self.q_size), MATRIX),
        }

    def bind(self, t):
        self.qkv_weight = torch.cat([t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"]], 0).contiguous()
        self.o_weight = t["o_proj.weight"]

    def setup(self, rt) -> None:
        self.position.setup(rt)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(kv=KVNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True, join=None):
        s = self.spec
        T = x.shape[0]
        qkv = K.linear(x, self.qkv_weight)
        k_cache, v_cache, group = ctx.cache.kv(cache_layer)
        if ctx.max_len == 1:
            # a decode step: rotation, cache store, attention over the pages and the merge of key ranges in one launch
            splits = ctx.attention_splits or K.decode_step_splits(T, s.num_heads, s.num_kv_heads, ctx.max_context,
                                                                  head_dim=s.head_dim)
            o = K.attention_decode_step(qkv, s.num_heads, s.num_kv_heads, s.head_dim, ctx.positions,
                                        ctx.slot_mappings[group], self.position.table, k_cache, v_cache,
                                        ctx.block_tables[group], ctx.token_req, self.scale, s.key_scale, s.window or 0,
                                        writes_cache, splits=splits)
            o = o.view(T, self.q_size)
            if K.linear_join_ok(o, self.o_weight, None, join):
                # the output projection adds the other mixer's output and the residual in its epilogue
                return K.linear_join(o, self.o_weight, None, join)
            return K.linear(o, self.o_weight)
        q = K.rope_kv_store(qkv, s.num_heads, s.num_kv_heads, s.head_dim, ctx.positions, ctx.slot_mappings[group],
                            self.position.table, k_cache, v_cache, s.key_scale, writes_cache)
        tables = ctx.block_tables[group]
        window = s.window or 0
        o = None
        token_list, n_short = None, T
        if q.dtype == torch.bfloat16 and ctx.has_long_portions:
            # long portions on the tensor-core kernel; what is left (decoded tokens, short portions) token by token
            if K.attention_prefill_tc_ok(q, k_cache):
                tiles, n_tiles = ctx.long_portion_tiles(K.ATTENTION_TC_TILE)
                o = K.attention_prefill_tc(q, k_cache, v_cache, tables, ctx.cu_seqlens, ctx.start_pos, tiles, n_tiles,
                                           self.scale, window, splits=K.prefill_splits(n_tiles, s.num_heads, ctx.max_context))
            else:
                tiles, n_tiles = ctx.long_portion_tiles(K.ATTENTION_TILE)
                o = K.attention_prefill(q, k_cache, v_cache, tables, ctx.cu_seqlens, ctx.start_pos, tiles, n_tiles,
                                        self.scale, window)
            token_list, n_short = ctx.short_portion_tokens()
        if n_short > 0 and token_list is not None and K.attention_decode_listed_ok(q, k_cache):
            # decoded tokens and short portions beside prompt portions: the decode step's kernel, on the listed rows
            splits = ctx.attention_splits or K.decode_step_splits(n_short, s.num_heads, s.num_kv_heads, ctx.max_context,
                                                                  listed=True)
            o = K.attention_decode_listed(q, k_cache, v_cache, tables, ctx.token_req, ctx.positions, token_list, n_short,
                                          self.scale, window, splits=splits, out=o)
        elif n_short > 0:
            splits = ctx.attention_splits or K.attention_splits(n_short, s.num_heads, s.num_kv_heads, ctx.max_context)
            o = K.attention_decode(q, k_cache, v_cache, tables, ctx.token_req, ctx.positions, self.scale, window,
                                   splits=splits, token_list=token_list, out=o)
        return K.linear(o.view(T, self.q_size), self.o_weight)
