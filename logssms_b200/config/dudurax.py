"""Typed configuration of the Dudurax decoder: post-norm layers on a 32-bit stream, each with one mixer (gated
linear attention, or windowed attention over cached latents) and a dense or routed feed-forward, behind a token
embedding with a hashed pair embedding.

config.json is nested: `embedding`, `norm`, `postln_alpha`, `vocab`, `width`, and `layers`, a list whose entries
give `type` (the mixer), `mixer` (its sizes) and `mlp` (the feed-forward, or null).  Every size and constant is
read from there; the only size that config.json does not give is the rank of the decay's low-rank projection,
which the checkpoint's tensors give (`mixer.decay_rank` may state it, and the random-weights writer needs it).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, require
from .specs import (DenseMLPSpec, GLASpec, LatentAttentionSpec, MixerSlot, ModelSpec, NormSpec, PostNormBlockSpec,
                    RopeSpec, RoutedMLPSpec)

ARCHITECTURE = "Dudurax"
GLA_TYPES = ("gla", "gla_2")            # two names of the one gated-linear-attention mixer
MAX_POSITIONS = 1 << 20


def _sub(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json lacks the mapping {where}{key!r}")
    return value


@dataclass(frozen=True)
class DuduraxConfig:
    raw: tuple                 # the config.json mapping, kept to write it back unchanged
    vocab_size: int
    hidden_size: int
    norm_eps: float
    skip_scale: float
    embedding_scale: float
    pair_buckets: int
    pair_mul_prev: int
    pair_mul_cur: int
    layers: tuple              # of (type, mixer mapping, mlp mapping or None), validated
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 8192
    architectures: tuple[str, ...] = (ARCHITECTURE,)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DuduraxConfig":
        emb = _sub(raw, "embedding", "")
        pair = _sub(emb, "bigram", "embedding.")
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks the list 'layers'")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = require(layer, "type", str)
            mixer = _sub(layer, "mixer", where)
            if kind in GLA_TYPES:
                for key in ("heads", "dim", "vdim"):
                    if require(mixer, key, int) <= 0:
                        raise ConfigError(f"{where}mixer.{key} must be positive")
                if require(mixer, "tau", float) <= 0:
                    raise ConfigError(f"{where}mixer.tau must be positive")
            elif kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    if require(mixer, key, int) < (0 if key in ("dim", "rot_dim") else 1):
                        raise ConfigError(f"{where}mixer.{key} is out of range")
                require(mixer, "scale", float)
                rot = _sub(mixer, "rot", where + "mixer.")
                dims = require(rot, "dims", int)
                if dims % 2 or dims > mixer["rot_dim"]:
                    raise ConfigError(f"{where}mixer.rot.dims must be even and within rot_dim")
                require(rot, "base", float)
                if require(_sub(mixer, "mask", where + "mixer."), "size", int) < 1:
                    raise ConfigError(f"{where}mixer.mask.size must be positive")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this architecture; known: {GLA_TYPES + ('latent_attention',)}")
            mlp = layer.get("mlp")
            if mlp is not None:
                ff_kind = require(mlp, "kind", str)
                if ff_kind == "dense":
                    require(mlp, "ff", int)
                elif ff_kind == "moe":
                    expert, router = _sub(mlp, "expert", where + "mlp."), _sub(mlp, "router", where + "mlp.")
                    require(expert, "ff", int)
                    require(expert, "limit", float)
                    n = require(router, "experts", int) + int(router.get("identity", 0))
                    groups = router.get("groups") or {"count": 1, "keep": 1}
                    count, keep = require(groups, "count", int), require(groups, "keep", int)
                    if count < 1 or n % count or not 1 <= keep <= count:
                        raise ConfigError(f"{where}mlp.router.groups does not divide the {n} router outputs")
                    if not 1 <= require(router, "top", int) <= keep * (n // count):
                        raise ConfigError(f"{where}mlp.router.top exceeds the experts that may be chosen")
                    require(router, "scale", float)
                else:
                    raise ConfigError(f"{where}mlp.kind {ff_kind!r} is neither 'dense' nor 'moe'")
            checked.append((kind, copy.deepcopy(dict(mixer)), None if mlp is None else copy.deepcopy(dict(mlp))))
        eps = require(_sub(raw, "norm", ""), "eps", float)
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        buckets = require(pair, "buckets", int)
        if buckets < 1:
            raise ConfigError("embedding.bigram.buckets must be positive")
        return cls(
            raw=tuple(sorted(copy.deepcopy(dict(raw)).items(), key=lambda kv: kv[0])),
            vocab_size=require(raw, "vocab", int), hidden_size=require(raw, "width", int), norm_eps=eps,
            skip_scale=require(raw, "postln_alpha", float), embedding_scale=require(emb, "scale", float),
            pair_buckets=buckets, pair_mul_prev=require(pair, "mul_prev", int), pair_mul_cur=require(pair, "mul_cur", int),
            layers=tuple(checked), torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            max_position_embeddings=int(raw.get("max_position_embeddings", 8192)),
        )

    def __hash__(self):
        return hash((self.vocab_size, self.hidden_size, len(self.layers)))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ as parts
    def model_spec(self) -> ModelSpec:
        H, eps = self.hidden_size, self.norm_eps
        norm = NormSpec(H, eps, param_name="")
        blocks = []
        for i, (kind, m, mlp) in enumerate(self.layers):
            if kind in GLA_TYPES:
                mixer = GLASpec(hidden_size=H, num_heads=int(m["heads"]), key_dim=int(m["dim"]), value_dim=int(m["vdim"]),
                                tau=float(m["tau"]), norm_eps=eps,
                                decay_rank=None if m.get("decay_rank") is None else int(m["decay_rank"]))
            else:
                rot_dim = int(m["rot_dim"])
                rope = None
                if int(m["rot"]["dims"]) > 0:
                    rope = RopeSpec(head_dim=rot_dim, rotary_dim=int(m["rot"]["dims"]), theta=float(m["rot"]["base"]),
                                    max_position=MAX_POSITIONS)
                mixer = LatentAttentionSpec(hidden_size=H, num_heads=int(m["heads"]), nope_dim=int(m["dim"]), rot_dim=rot_dim,
                                            value_dim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), softmax_scale=float(m["scale"]),
                                            window=int(m["mask"]["size"]), position=rope, norm_eps=eps)
            ff = None
            if mlp is not None and mlp["kind"] == "dense":
                ff = DenseMLPSpec(H, int(mlp["ff"]))
            elif mlp is not None:
                r = mlp["router"]
                groups = r.get("groups") or {"count": 1, "keep": 1}
                ff = RoutedMLPSpec(hidden_size=H, expert_size=int(mlp["expert"]["ff"]), num_experts=int(r["experts"]),
                                   num_identity=int(r.get("identity", 0)), top=int(r["top"]), num_groups=int(groups["count"]),
                                   keep_groups=int(groups["keep"]), route_scale=float(r["scale"]), limit=float(mlp["expert"]["limit"]))
            blocks.append(PostNormBlockSpec(
                prefix=f"l{i}.", mixer=MixerSlot(mixer, "mix."), mixer_norm=norm, mixer_norm_name="norm1",
                feed_forward=ff, feed_forward_name="mlp.", feed_forward_norm=None if ff is None else norm,
                feed_forward_norm_name="norm2", skip_scale=self.skip_scale))
        return ModelSpec(
            vocab_size=self.vocab_size, hidden_size=H, embedding_name="", embedding_multiplier=self.embedding_scale,
            lm_head_name="head", lm_head_multiplier=1.0, tie_word_embeddings=False,
            final_norm=norm, final_norm_name="final.norm", layers=tuple(blocks),
            embedding_kind="pair_embedding", lm_head_kind="lm_head_bare",
            embedding_options=(("buckets", self.pair_buckets), ("mul_prev", self.pair_mul_prev), ("mul_cur", self.pair_mul_cur)),
        )
