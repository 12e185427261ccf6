"""Gated linear attention: a matrix-valued state per head with a decay per key channel."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, StateNeed
from ..ops import kernels as K
from ..registry import MIXERS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init, ones_init


@MIXERS.register("gla")
class GatedLinearAttention(Part):
    """q, k [heads, key_dim], v, g [heads, value_dim] from the input h; z = a2 (a1 h) + a2.b gives the decay
    sigmoid(z)^(1/tau) per key channel.  Per head S <- diag(decay) S + k v^T, o = S^T q / sqrt(key_dim); o is
    RMS-normed per head (one weight [value_dim] for all heads), times silu(g), then the output projection.

    Per-request state: S [heads, key_dim, value_dim] in float32.  Prompt portions of a bfloat16 engine run in chunks of
    16 tokens on the tensor cores (`K.gla_chunked`), everything else token by token (`K.gla_scan`).  The five input projections are one product
    (rows q | k | v | g | a1, merged at bind time).  Decay, state and the head norm are 32-bit in every engine dtype.
    Tensors: q, k, v, g, o, norm, a1, a2, a2.b."""
    kernels = ("gla", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self._jitter = 0.1 if perturb_init else 0.0
        self.in_w = self.a2_w = self.a2_b = self.norm_w = self.o_w = None
        self.rank = spec.decay_rank

    def param_specs(self):
        s = self.spec
        qk, vg = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        rank = -1 if s.decay_rank is None else s.decay_rank
        # random weights: products of unit-size rows stay of unit size; decays from long to short memories
        fan = normal_init(s.hidden_size ** -0.5)
        return {
            "q": ParamSpec((qk, s.hidden_size), MATRIX, fan), "k": ParamSpec((qk, s.hidden_size), MATRIX, fan),
            "v": ParamSpec((vg, s.hidden_size), MATRIX, fan), "g": ParamSpec((vg, s.hidden_size), MATRIX, fan),
            "o": ParamSpec((s.hidden_size, vg), MATRIX, normal_init(2.0 * vg ** -0.5)),
            "norm": ParamSpec((s.value_dim,), VECTOR, ones_init(self._jitter)),
            "a1": ParamSpec((rank, s.hidden_size), MATRIX, fan),
            "a2": ParamSpec((qk, rank), MATRIX, normal_init(max(rank, 1) ** -0.5)),
            "a2.b": ParamSpec((qk,), VECTOR, normal_init(3.0)),
        }

    def bind(self, t):
        if t["a1"].shape[0] != t["a2"].shape[1]:
            raise ValueError(f"the decay's two projections disagree on their rank: {tuple(t['a1'].shape)} and {tuple(t['a2'].shape)}")
        self.rank = t["a1"].shape[0]
        self.in_w = torch.cat([t["q"], t["k"], t["v"], t["g"], t["a1"]], 0).contiguous()
        self.a2_w, self.o_w, self.norm_w = t["a2"].contiguous(), t["o"], t["norm"]
        self.a2_b = t["a2.b"].to(self.a2_w.dtype)       # (stored in the matrices' dtype: the cast back is exact)

    def setup(self, rt) -> None:
        pass

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(states=(StateNeed("gla", (s.num_heads, s.key_dim, s.value_dim), torch.float32),))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        qk, vg = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        proj = K.linear(x, self.in_w)                                     # q | k | v | g | low-rank decay input
        low = proj[:, 2 * qk + 2 * vg:]
        z = K.linear(low, self.a2_w, self.a2_b, out_f32=True)
        state = ctx.cache.states[cache_layer]["gla"]
        sizes = (s.num_heads, s.key_dim, s.value_dim, s.tau, s.key_dim ** -0.5)
        if ctx.has_long_portions and K.gla_chunked_ok(proj, s.key_dim):
            # long portions in chunks on the tensor cores; decoded tokens and short portions (other requests, other rows
            # of o) token by token
            chunks, n_chunks, per_request, n_long = ctx.long_portion_chunks(K.GLA_CHUNK)
            _, _, short_list, n_short = ctx.requests_by_portion()
            o = torch.empty((x.shape[0], vg), dtype=torch.float32, device=x.device)
            seg = {}
            if K.gla_segmented_pays(ctx.num_tokens, n_long, s.num_heads, s.value_dim):
                # few long portions (a lone prompt): their segments side by side instead of one CTA walking each
                segments, _, seg_requests, _ = ctx.long_portion_segments(K.GLA_CHUNK, K.GLA_SEGMENT)
                seg = {"segments": segments, "segment_requests": seg_requests}
            K.gla_chunked(proj, z, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, chunks, n_chunks, per_request, n_long,
                          *sizes, out=o, **seg)
            if n_short > 0:
                K.gla_scan(proj, z, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests, *sizes,
                           request_list=short_list, out=o)
        else:
            o = K.gla_scan(proj, z, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests, *sizes)
        y = K.gla_norm_gate(o, proj[:, 2 * qk + vg: 2 * qk + 2 * vg], self.norm_w, s.norm_eps, s.num_heads)
        return K.linear(y, self.o_w)
