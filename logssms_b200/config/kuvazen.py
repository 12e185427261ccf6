"""Typed configuration of the Kuvazen decoder: pre-norm layers on a 32-bit stream with a scale per channel on every
sublayer's output and a per-layer input from the token itself; each layer has one mixer (a minGRU recurrence, or
grouped-query attention over a sliding window plus pooled blocks with rotated values) and a dense or routed
feed-forward; a run of layers may be looped with the same weights.

config.json is nested: `vocab`, `width`, `norm.eps`, `token_side.dim`, `loop` (start, stop, times) and `layers`, a list
whose entries give `type` (the mixer), `mixer` (its sizes) and `mlp` (the feed-forward, or null).  Every size and
constant is read from there.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, require
from .specs import (ClampedGLUSpec, MinGRUSpec, MixerSlot, ModelSpec, NormSpec, PooledWindowAttentionSpec, RopeSpec,
                    RoutedMLPSpec, ScheduleEntry, StreamBlockSpec, TokenSideSpec)

ARCHITECTURE = "Kuvazen"
MIXER_TYPES = ("mingru", "attention")
MAX_POSITIONS = 1 << 20


def _sub(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json lacks the mapping {where}{key!r}")
    return value


def _positive(raw: Mapping[str, Any], key: str, where: str) -> int:
    value = require(raw, key, int)
    if value < 1:
        raise ConfigError(f"{where}{key} must be positive")
    return value


@dataclass(frozen=True)
class KuvazenConfig:
    raw: tuple                 # the config.json mapping, kept to write it back unchanged
    vocab_size: int
    hidden_size: int
    norm_eps: float
    side_dim: int              # 0: no side input
    loop: tuple[int, int, int]  # start, stop, times (times 1 or an empty range: every layer runs once)
    layers: tuple              # of (type, mixer mapping, mlp mapping or None), validated
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 8192
    architectures: tuple[str, ...] = (ARCHITECTURE,)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KuvazenConfig":
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks the list 'layers'")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = require(layer, "type", str)
            mixer = _sub(layer, "mixer", where)
            if kind == "mingru":
                _positive(mixer, "width", where + "mixer.")
            elif kind == "attention":
                heads, kv = _positive(mixer, "heads", where + "mixer."), _positive(mixer, "kv_heads", where + "mixer.")
                if heads % kv:
                    raise ConfigError(f"{where}mixer.heads must be a multiple of kv_heads")
                dim, vdim = _positive(mixer, "dim", where + "mixer."), _positive(mixer, "vdim", where + "mixer.")
                if vdim % 2:
                    raise ConfigError(f"{where}mixer.vdim must be even (values are rotated in pairs)")
                require(mixer, "scale", float)
                rot = _sub(mixer, "rot", where + "mixer.")
                dims = require(rot, "dims", int)
                if dims < 0 or dims % 2 or dims > dim:
                    raise ConfigError(f"{where}mixer.rot.dims must be even and within dim")
                if require(rot, "base", float) <= 0:
                    raise ConfigError(f"{where}mixer.rot.base must be positive")
                mask = _sub(mixer, "mask", where + "mixer.")
                _positive(mask, "size", where + "mixer.mask.")
                _positive(mask, "pool", where + "mixer.mask.")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this architecture; known: {MIXER_TYPES}")
            mlp = layer.get("mlp")
            if mlp is not None:
                ff_kind = require(mlp, "kind", str)
                if ff_kind == "dense":
                    _positive(mlp, "ff", where + "mlp.")
                    require(mlp, "limit", float)
                elif ff_kind == "moe":
                    _positive(_sub(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")
                    router = _sub(mlp, "router", where + "mlp.")
                    if not 1 <= require(router, "top", int) <= _positive(router, "experts", where + "mlp.router."):
                        raise ConfigError(f"{where}mlp.router.top must lie within 1 .. experts")
                else:
                    raise ConfigError(f"{where}mlp.kind {ff_kind!r} is neither 'dense' nor 'moe'")
            checked.append((kind, copy.deepcopy(dict(mixer)), None if mlp is None else copy.deepcopy(dict(mlp))))
        eps = require(_sub(raw, "norm", ""), "eps", float)
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        side = raw.get("token_side")
        side_dim = 0 if side is None else _positive(side, "dim", "token_side.")
        loop = raw.get("loop")
        if loop is None:
            bounds = (0, 0, 1)
        else:
            bounds = (require(loop, "start", int), require(loop, "stop", int), require(loop, "times", int))
            if not 0 <= bounds[0] <= bounds[1] <= len(checked) or bounds[2] < 1:
                raise ConfigError("loop must name a range of layers start <= stop and times >= 1")
        return cls(
            raw=tuple(sorted(copy.deepcopy(dict(raw)).items(), key=lambda kv: kv[0])),
            vocab_size=_positive(raw, "vocab", ""), hidden_size=_positive(raw, "width", ""), norm_eps=eps,
            side_dim=side_dim, loop=bounds, layers=tuple(checked), torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            max_position_embeddings=int(raw.get("max_position_embeddings", 8192)),
        )

    def __hash__(self):
        return hash((self.vocab_size, self.hidden_size, len(self.layers)))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ as parts
    def layer_runs(self) -> list[int]:
        """The layers in the order they run: the looped range `times` times in a row, between what lies before and after."""
        start, stop, times = self.loop
        n = len(self.layers)
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def model_spec(self) -> ModelSpec:
        H, eps = self.hidden_size, self.norm_eps
        norm = NormSpec(H, eps, kind="layernorm", param_name="")
        blocks = []
        for i, (kind, m, mlp) in enumerate(self.layers):
            if kind == "mingru":
                mixer = MinGRUSpec(hidden_size=H, width=int(m["width"]))
            else:
                dim, vdim = int(m["dim"]), int(m["vdim"])
                dims, base = int(m["rot"]["dims"]), float(m["rot"]["base"])
                mixer = PooledWindowAttentionSpec(
                    hidden_size=H, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=dim, value_dim=vdim,
                    softmax_scale=float(m["scale"]), window=int(m["mask"]["size"]), pool=int(m["mask"]["pool"]),
                    position=None if dims == 0 else RopeSpec(head_dim=dim, rotary_dim=dims, theta=base, max_position=MAX_POSITIONS),
                    value_position=RopeSpec(head_dim=vdim, rotary_dim=vdim, theta=base, max_position=MAX_POSITIONS))
            ff = None
            if mlp is not None and mlp["kind"] == "dense":
                ff = ClampedGLUSpec(H, int(mlp["ff"]), float(mlp["limit"]))
            elif mlp is not None:
                r = mlp["router"]
                ff = RoutedMLPSpec(hidden_size=H, expert_size=int(mlp["expert"]["ff"]), num_experts=int(r["experts"]),
                                   num_identity=0, top=int(r["top"]), num_groups=1, keep_groups=1, route_scale=1.0, limit=0.0,
                                   score="sigmoid", expert="silu", weigh="input", correction=False)
            side = None
            if self.side_dim:
                side = TokenSideSpec(hidden_size=H, dim=self.side_dim, offset=i * self.side_dim,
                                     table_width=len(self.layers) * self.side_dim, vocab_size=self.vocab_size, eps=eps)
            blocks.append(StreamBlockSpec(
                prefix=f"l{i}.", mixer=MixerSlot(mixer, "mix."), mixer_norm=norm, mixer_norm_name="norm1",
                feed_forward=ff, feed_forward_name="mlp.", feed_forward_norm=None if ff is None else norm,
                feed_forward_norm_name="norm2", layer_scale=True, side=side))
        schedule = tuple(ScheduleEntry(layer, run) for run, layer in enumerate(self.layer_runs()))
        return ModelSpec(
            vocab_size=self.vocab_size, hidden_size=H, embedding_name="", embedding_multiplier=1.0,
            lm_head_name="head", lm_head_multiplier=1.0, tie_word_embeddings=False,
            final_norm=norm, final_norm_name="final.norm", layers=tuple(blocks), schedule=schedule,
            embedding_kind="normed_embedding", lm_head_kind="lm_head_bare",
            embedding_options=(("norm", NormSpec(H, eps, kind="layernorm", param_name="embed.norm")),),
        )
