"""Grouped-query attention over a sliding window of tokens plus pooled blocks behind it, with rotated values."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed, PagedNeed, PagedTensor
from ..ops import kernels as K
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import MATRIX, ParamSpec, Part, normal_init
from .rope import NoPositionEncoding


def _position(spec, shared):
    if spec is None:
        return NoPositionEncoding()
    key = ("position", spec)
    if shared is not None and key in shared:
        return shared[key]
    part = POSITION_ENCODINGS.get(spec.kind)(spec)
    if shared is not None:
        shared[key] = part
    return part


@MIXERS.register("pooled_window_attention")
class PooledWindowAttention(Part):
    """q, k [heads | kv_heads, head_dim], v [kv_heads, value_dim] from the input; query head h reads key/value head
    h // (heads / kv_heads).  Query i sees the tokens j with 0 <= i - j < window and, as one key and value each (the
    means of the cached keys and values), every block of `pool` tokens that lies wholly behind the window; one softmax
    over both, scores times `softmax_scale`.  Queries and keys are rotated over neighbouring pairs of their first
    `position.rotary_dim` columns; values over all their columns by their own position (they are cached so), and a
    head's summed values are turned back by the query's position.

    Two paged needs: the tokens' keys and values in a group with a window (pages go back once the window and the
    block that is being filled have passed them), and the blocks' means in a group of one entry per `pool` tokens that
    is kept for the request's life.  The token that ends a block writes the block's means.  Prompt portions of a bfloat16
    engine run on the tensor cores (`K.pooled_attention_tile`); decoded tokens, short portions and float32 engines cut
    every token's keys into ranges that run side by side (`K.pooled_attention_split`), or, for sizes that form does not
    take, run a warp per (token, head) (`K.pooled_attention`).  Tensors: q, k, v, o."""
    kernels = ("attention_pooled", "rope", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        self.spec = spec
        self.position = _position(spec.position, shared)
        self.value_position = _position(spec.value_position, shared)
        self.in_w = self.o_w = None

    def param_specs(self):
        s = self.spec
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        return {
            "q": ParamSpec((s.num_heads * s.head_dim, s.hidden_size), MATRIX, fan),
            "k": ParamSpec((s.num_kv_heads * s.head_dim, s.hidden_size), MATRIX, fan),
            "v": ParamSpec((s.num_kv_heads * s.value_dim, s.hidden_size), MATRIX, fan),
            "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim), MATRIX, normal_init(2.0 * (s.num_heads * s.value_dim) ** -0.5)),
        }

    def bind(self, t):
        self.in_w = torch.cat([t["q"], t["k"], t["v"]], 0).contiguous()
        self.o_w = t["o"]

    def setup(self, rt) -> None:
        self.position.setup(rt)
        self.value_position.setup(rt)

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        # a block's means are made when its last token arrives, from the cached rows of all its tokens: they must still
        # be there, so the token group keeps what the window OR the block that is being filled still needs
        tokens = KVNeed(s.num_kv_heads, s.head_dim, max(s.window, s.pool), s.value_dim)
        blocks = PagedNeed((PagedTensor("k_pooled", (s.num_kv_heads, s.head_dim)),
                            PagedTensor("v_pooled", (s.num_kv_heads, s.value_dim))), None, s.pool)
        return CacheNeeds(kv=tokens, more_paged=(blocks,))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        k_cache, v_cache, gi = ctx.cache.kv(cache_layer)
        kp_cache, gp = ctx.cache.paged_tensor(cache_layer, "k_pooled")
        vp_cache, _ = ctx.cache.paged_tensor(cache_layer, "v_pooled")
        qkv = K.linear(x, self.in_w)
        q = K.pooled_prepare(qkv, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, ctx.positions, ctx.slot_mappings[gi],
                             self.position.table, self.value_position.table, k_cache, v_cache, writes_cache)
        if writes_cache:
            K.pooled_blocks(k_cache, v_cache, kp_cache, vp_cache, ctx.positions, ctx.token_req, ctx.block_tables[gi],
                            ctx.slot_mappings[gp], s.pool)
        tables = (ctx.block_tables[gi], ctx.block_tables[gp])
        # the most keys a token of this step sees (a captured step is replayed for other positions: `max_context` is
        # then the engine's limit)
        most_keys = min(s.window, ctx.max_context) + ctx.max_context // s.pool

        def few_rows(token_list=None, out=None, n=x.shape[0]):
            # decoded tokens and short portions: key ranges side by side where the sizes allow, else a warp per (token, head)
            args = (q, k_cache, v_cache, kp_cache, vp_cache, *tables, ctx.token_req, ctx.positions, self.value_position.table,
                    s.softmax_scale, s.window, s.pool)
            if K.pooled_attention_split_ok(q, v_cache):
                return K.pooled_attention_split(*args, K.pooled_splits(n, s.num_kv_heads, most_keys), token_list=token_list, out=out)
            return K.pooled_attention(*args, token_list=token_list, out=out)

        if ctx.has_long_portions and K.pooled_attention_tile_ok(q, v_cache):
            # long portions on the tensor cores: runs of neighbouring tokens share their keys through shared memory; decoded
            # tokens and short portions (other rows of the output) a warp per (token, head)
            tiles, n_tiles = ctx.long_portion_tiles(K.pooled_attention_tile_q())
            short, n_short = ctx.short_portion_tokens()
            o = torch.empty((x.shape[0], s.num_heads * s.value_dim), dtype=q.dtype, device=q.device)
            K.pooled_attention_tile(q, k_cache, v_cache, kp_cache, vp_cache, *tables, ctx.cu_seqlens, ctx.start_pos, ctx.positions,
                                    tiles, self.value_position.table, s.softmax_scale, s.window, s.pool, o,
                                    splits=K.pooled_tile_splits(n_tiles, s.num_heads))
            if n_short > 0:
                few_rows(short, o, n_short)
        else:
            o = few_rows()
        return K.linear(o, self.o_w)
