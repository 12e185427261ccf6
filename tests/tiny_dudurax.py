"""Small Dudurax configurations (sizes unlike any real model's, several values of every option), a writer of random
model folders for them, and the plain implementation's logits."""
from __future__ import annotations

import json
import os

import torch

from logssms_b200.config import make_model_config
from logssms_b200.weights import write_random_model

from plain.dudurax_plain import PlainDudurax


def _latent(heads, dim, rot_dim, rot_dims, vdim, rank, window, base=1e4, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": window},
                      "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def _gla(kind, heads, dim, vdim, tau, rank):
    return {"type": kind, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}}


def _moe(ff, limit, experts, identity, count, keep, top, scale):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "groups": {"count": count, "keep": keep}, "top": top, "scale": scale}}


def _model(width, vocab, eps, alpha, scale, buckets, mul_prev, mul_cur, layers):
    return {"architecture": "Dudurax", "embedding": {"bigram": {"buckets": buckets, "mul_cur": mul_cur, "mul_prev": mul_prev}, "scale": scale},
            "layers": layers, "norm": {"eps": eps}, "postln_alpha": alpha, "vocab": vocab, "width": width}


# A: every kind of layer once; windows of 20 (inside a page) and 70 (across a page edge); a rotation of half the
# rotated part; a layer without a feed-forward; routers with and without identity experts and groups
DUDU_A = _model(64, 211, 1e-5, 2.0, 4.0, 97, 31, 7, [
    {**_latent(2, 16, 8, 8, 24, 40, 20), "mlp": {"kind": "dense", "ff": 96}},
    {**_gla("gla", 3, 16, 24, 4.0, 8), "mlp": _moe(48, 2.0, 4, 2, 3, 2, 2, 1.2)},
    {**_gla("gla_2", 1, 48, 40, 16.0, 4), "mlp": None},
    {**_latent(3, 8, 16, 8, 16, 24, 70, base=500.0, scale=0.3), "mlp": _moe(40, 0.5, 3, 0, 1, 1, 1, 1.0)},
])

# B: key channels of 128 (two threads share a state column), a window of one token and one longer than any request,
# a rotated key part larger than the unrotated one, more identity experts than real ones, another skip scale
DUDU_B = _model(96, 333, 1e-6, 1.0, 2.5, 50, 3, 1000003, [
    {**_gla("gla_2", 2, 128, 80, 1.0, 16), "mlp": _moe(24, 1.0, 2, 4, 2, 1, 3, 2.0)},
    {**_latent(4, 32, 32, 32, 8, 72, 1), "mlp": {"kind": "dense", "ff": 50}},
    {**_latent(1, 8, 64, 64, 48, 136, 400, base=1e6), "mlp": None},
    {**_gla("gla", 5, 8, 24, 64.0, 2), "mlp": {"kind": "dense", "ff": 200}},
])

# C: one layer of each mixer with sizes of 1 where the design allows them
DUDU_C = _model(48, 130, 1e-5, 3.0, 1.0, 1, 1, 1, [
    {**_gla("gla", 1, 4, 1, 2.0, 1), "mlp": _moe(8, 4.0, 1, 1, 2, 2, 2, 0.7)},
    {**_latent(1, 2, 2, 2, 1, 1, 3), "mlp": None},
])

# D: recurrent layers only (no paged cache at all); E: attention layers only (no state but the previous token), two
# of them with equal needs (one page group) and one with others
DUDU_D = _model(40, 90, 1e-5, 1.5, 3.0, 13, 5, 3, [
    {**_gla("gla", 2, 32, 16, 8.0, 4), "mlp": {"kind": "dense", "ff": 64}},
    {**_gla("gla_2", 2, 16, 32, 2.0, 4), "mlp": _moe(16, 1.5, 2, 1, 1, 1, 2, 1.0)},
])
DUDU_E = _model(48, 77, 1e-5, 2.5, 5.0, 31, 7, 11, [
    {**_latent(4, 8, 16, 16, 8, 32, 48), "mlp": None},
    {**_latent(4, 8, 16, 16, 8, 32, 48), "mlp": {"kind": "dense", "ff": 64}},
    {**_latent(2, 16, 16, 8, 24, 64, 9), "mlp": _moe(24, 3.0, 3, 1, 2, 1, 2, 1.5)},
])

def random_dudurax(seed: int) -> dict:
    """A configuration with every size and option drawn at random within what config.json allows."""
    import random
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.55:
            mixer = _gla(rng.choice(["gla", "gla_2"]), rng.randint(1, 4), rng.choice([8, 16, 24, 32, 48, 64, 80]),
                         rng.choice([8, 16, 24, 40, 64, 72]), rng.choice([1.0, 2.0, 4.0, 16.0, 64.0]), rng.randint(1, 8))
        else:
            rot = rng.choice([8, 16, 32])
            mixer = _latent(rng.choice([1, 2, 3, 4, 6, 16]), rng.choice([8, 16, 32]), rot, rng.choice([rot, rot // 2]),
                            rng.choice([8, 16, 24, 40]), rng.choice([16, 24, 32, 40, 64, 96]),
                            rng.choice([1, 3, 17, 64, 65, 100, 1000]), base=rng.choice([100.0, 1e4, 1e6]))
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = {"kind": "dense", "ff": 2 * rng.randint(8, 60)}
        else:
            experts, identity = rng.randint(1, 6), rng.randint(0, 3)
            n = experts + identity
            count = rng.choice([d for d in range(1, n + 1) if n % d == 0])
            keep = rng.randint(1, count)
            mlp = _moe(2 * rng.randint(4, 30), rng.choice([0.5, 1.0, 2.0, 7.0]), experts, identity, count, keep,
                       rng.randint(1, keep * (n // count)), rng.choice([1.0, 1.5, 2.5]))
        layers.append({**mixer, "mlp": mlp})
    return _model(2 * rng.randint(16, 48), rng.randint(60, 400), rng.choice([1e-5, 1e-6]), rng.choice([1.0, 2.0, 3.0]),
                  rng.choice([1.0, 4.0, 12.0]), rng.randint(1, 2000), rng.randint(1, 200), rng.randint(1, 200), layers)


DUDU = {"A": DUDU_A, "B": DUDU_B, "C": DUDU_C, "D": DUDU_D, "E": DUDU_E}
DUDU.update({f"R{seed}": random_dudurax(seed) for seed in range(1, 25)})


def make_dudurax_dir(path, raw: dict, seed: int = 0, dtype=torch.float32, sharp: float = 1.0, steady_router: bool = False) -> str:
    """Random weights for `raw` in `path`.  `sharp` scales the query projections of the attention layers so that the
    softmax picks single keys (a missing or surplus key then moves the logits far beyond any tolerance);
    `steady_router` spaces the routers' choice corrections so that no choice is a close call (a bfloat16 engine may
    otherwise choose another expert than a float64 oracle)."""
    from safetensors.torch import load_file, save_file
    out = write_random_model(make_model_config(raw), str(path), seed=seed, dtype=dtype, perturb=True)
    file = os.path.join(out, "model.safetensors")
    t = load_file(file)
    gen = torch.Generator().manual_seed(seed + 1)
    for name in list(t):
        if sharp != 1.0 and name.endswith(".mix.q") and name.replace(".mix.q", ".mix.dkv") in t:
            t[name] = (t[name].float() * sharp).to(t[name].dtype)
        if steady_router and name.endswith(".mlp.correction"):
            n = t[name].numel()
            t[name] = (1.5 * torch.randperm(n, generator=gen).float()).to(t[name].dtype)
    save_file(t, file)
    return out


def plain_model(model_dir: str) -> PlainDudurax:
    return PlainDudurax.from_folder(model_dir, torch.float64)


def plain_logits(model_dir: str, ids) -> torch.Tensor:
    m = plain_model(model_dir)
    return m.forward(list(ids), m.new_state()).float()


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square of the logits' difference (its mean over the vocabulary taken off) over the
    root mean square of the wanted logits."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), "engine produced non-finite logits"
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)


# (tiny random models are ill-conditioned at their first positions: a head norm over one or two nearly cancelling outer
# products multiplies float32 rounding a hundredfold; a wrong or missing term moves the logits by tenths)
TOL = {"float32": 3e-4, "bfloat16": 5e-2}
