"""minGRU: a gated recurrence per channel whose gates read the current token only."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, StateNeed
from ..ops import kernels as K
from ..registry import MIXERS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init


@MIXERS.register("mingru")
class MinGRU(Part):
    """z = sigmoid(W_z h + b_z), u = W_x h + b_x, candidate c = u + 1/2 where u >= 0 and sigmoid(u) where u < 0;
    per channel S <- (1 - z) S + z c; output W_o (S * silu(W_g h)).

    Per-request state: S [width] in float32, zero at a sequence's start.  The three input products are one (rows z | x | g,
    merged at bind time); biases, gates, candidate and state are 32-bit in every engine dtype.  Long prompt portions run
    in chunks side by side (`K.mingru_chunked`), everything else token by token (`K.mingru_scan`).
    Tensors: z, z.b, x, x.b, g, o."""
    kernels = ("mingru", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self.in_w = self.bias_z = self.bias_x = self.o_w = None

    def param_specs(self):
        s = self.spec
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        return {
            "z": ParamSpec((s.width, s.hidden_size), MATRIX, fan), "z.b": ParamSpec((s.width,), VECTOR, normal_init(1.0)),
            "x": ParamSpec((s.width, s.hidden_size), MATRIX, fan), "x.b": ParamSpec((s.width,), VECTOR, normal_init(0.5)),
            "g": ParamSpec((s.width, s.hidden_size), MATRIX, fan),
            "o": ParamSpec((s.hidden_size, s.width), MATRIX, normal_init(2.0 * s.width ** -0.5)),
        }

    def bind(self, t):
        self.in_w = torch.cat([t["z"], t["x"], t["g"]], 0).contiguous()
        self.bias_z, self.bias_x, self.o_w = t["z.b"], t["x.b"], t["o"]

    def setup(self, rt) -> None:
        pass

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(states=(StateNeed("mingru", (self.spec.width,), torch.float32),))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        W = self.spec.width
        proj = K.linear(x, self.in_w)                                     # z | candidate | gate products
        state = ctx.cache.states[cache_layer]["mingru"]
        args = (proj, self.bias_z, self.bias_x, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots)
        if ctx.has_long_portions:
            # long portions in chunks side by side; decoded tokens and short portions (other requests, other rows of the
            # output) token by token
            chunks, n_chunks, per_request, n_long = ctx.long_portion_chunks(K.mingru_chunk())
            _, _, short_list, n_short = ctx.requests_by_portion()
            out = torch.empty((x.shape[0], W), dtype=proj.dtype, device=x.device)
            K.mingru_chunked(*args, chunks, n_chunks, per_request, n_long, ctx.num_requests, W, out)
            if n_short > 0:
                K.mingru_scan(*args, ctx.num_requests, W, request_list=short_list, out=out)
        else:
            out = K.mingru_scan(*args, ctx.num_requests, W)
        return K.linear(out, self.o_w)
