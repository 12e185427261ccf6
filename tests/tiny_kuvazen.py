"""Small Kuvazen configurations (sizes unlike any real model's, several values of every option), a writer of random
model folders for them, and the plain implementation's logits."""
from __future__ import annotations

import os

import torch

from logssms_b200.config import make_model_config
from logssms_b200.weights import write_random_model

from plain.kuvazen_plain import PlainKuvazen


def _attn(heads, kv_heads, dim, vdim, rot_dims, window, pool, base=1e4, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window, "pool": pool},
                      "rot": {"base": base, "dims": rot_dims}, "scale": scale if scale is not None else dim ** -0.5}}


def _gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _model(width, vocab, eps, side, loop, layers):
    raw = {"architecture": "Kuvazen", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if side:
        raw["token_side"] = {"dim": side}
    if loop is not None:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


# A: both mixers and both feed-forwards; grouped queries (3 query heads per key head), a rotation of part of the head, a
# window inside a page (20) with blocks of 5 that divide neither the window nor a page of 64, and a window across page
# edges (70) with blocks of 16; two experts of three chosen; the last two layers run three times
KUVA_A = _model(64, 211, 1e-5, 6, (2, 4, 3), [
    {**_attn(6, 2, 16, 24, 8, 20, 5), "mlp": _dense(96, 1.0)},
    {**_gru(40), "mlp": _moe(24, 3, 2)},
    {**_attn(2, 2, 24, 8, 24, 70, 16, base=500.0, scale=0.3), "mlp": _moe(40, 5, 1)},
    {**_gru(88), "mlp": None},
])

# B: blocks longer than the window (a token is unseen for a while), a window of one token, blocks of one token (every
# token behind the window is seen through its "block"), a layer without a feed-forward, value heads wider than 128, no loop
KUVA_B = _model(96, 333, 1e-6, 3, None, [
    {**_attn(4, 1, 8, 136, 4, 7, 24, base=1e6), "mlp": None},
    {**_gru(24), "mlp": _dense(50, 3.0)},
    {**_attn(3, 3, 32, 16, 0, 1, 3), "mlp": _moe(16, 8, 3)},
    {**_attn(2, 1, 16, 12, 16, 40, 1), "mlp": _dense(64, 0.5)},
])

# C: sizes of 1 where the design allows them, no side input, the whole model looped twice
KUVA_C = _model(48, 130, 1e-5, 0, (0, 2, 2), [
    {**_gru(1), "mlp": _moe(8, 1, 1)},
    {**_attn(1, 1, 2, 2, 2, 3, 2), "mlp": None},
])

# D: recurrent layers only (no paged cache at all), a side input of one column; E: attention layers only, two of them
# with equal needs (one page group each for tokens and blocks) and one with others
KUVA_D = _model(40, 90, 1e-5, 1, (1, 2, 2), [
    {**_gru(72), "mlp": _dense(64, 2.0)},
    {**_gru(16), "mlp": _moe(16, 4, 2)},
])
KUVA_E = _model(48, 77, 1e-5, 4, (0, 1, 2), [
    {**_attn(4, 2, 8, 16, 8, 48, 8), "mlp": None},
    {**_attn(4, 2, 8, 16, 8, 48, 8), "mlp": _dense(64, 1.5)},
    {**_attn(2, 1, 16, 24, 8, 9, 4), "mlp": _moe(24, 6, 2)},
])


# F: nothing is a multiple of 8, or even of 2 where the design allows it: an odd width and vocabulary, a recurrent width,
# feed-forward sizes and a side input that are odd, head sizes of 12 and 20 (no 16-byte rows anywhere)
KUVA_F = _model(45, 101, 1e-5, 5, (1, 3, 2), [
    {**_attn(3, 1, 12, 20, 6, 11, 3), "mlp": _dense(31, 1.0)},
    {**_gru(33), "mlp": _moe(19, 3, 2)},
    {**_attn(2, 2, 6, 10, 6, 30, 7, base=777.0), "mlp": None},
])


def random_kuvazen(seed: int) -> dict:
    """A configuration with every size and option drawn at random within what config.json allows."""
    import random
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.45:
            mixer = _gru(rng.choice([8, 24, 40, 72, 130]))
        else:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 64])
            mixer = _attn(kv * rng.choice([1, 2, 4]), kv, dim, 2 * rng.randint(2, 40), rng.choice([0, dim // 2, dim]),
                          rng.choice([1, 3, 17, 64, 65, 100, 1000]), rng.choice([1, 2, 7, 16, 33, 64]), base=rng.choice([100.0, 1e4, 1e6]))
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = _dense(2 * rng.randint(8, 60), rng.choice([0.5, 1.0, 2.0, 7.0]))
        else:
            experts = rng.randint(1, 9)
            mlp = _moe(2 * rng.randint(4, 30), experts, rng.randint(1, min(experts, 3)))
        layers.append({**mixer, "mlp": mlp})
    a = rng.randint(0, len(layers))
    b = rng.randint(a, len(layers))
    return _model(2 * rng.randint(16, 48), rng.randint(60, 400), rng.choice([1e-5, 1e-6]), rng.choice([0, 1, 5, 12]),
                  rng.choice([None, (a, b, rng.randint(1, 3))]), layers)


KUVA = {"A": KUVA_A, "B": KUVA_B, "C": KUVA_C, "D": KUVA_D, "E": KUVA_E, "F": KUVA_F}
KUVA.update({f"R{seed}": random_kuvazen(seed) for seed in range(1, 13)})


def make_kuvazen_dir(path, raw: dict, seed: int = 0, dtype=torch.float32, sharp: float = 1.0) -> str:
    """Random weights for `raw` in `path`.  `sharp` scales the query projections of the attention layers so that the
    softmax picks single keys (a missing or surplus key or block then moves the logits far beyond any tolerance)."""
    from safetensors.torch import load_file, save_file
    out = write_random_model(make_model_config(raw), str(path), seed=seed, dtype=dtype, perturb=True)
    file = os.path.join(out, "model.safetensors")
    t = load_file(file)
    for name in list(t):
        if sharp != 1.0 and name.endswith(".mix.q"):
            t[name] = (t[name].float() * sharp).to(t[name].dtype)
    save_file(t, file)
    return out


def plain_model(model_dir: str) -> PlainKuvazen:
    return PlainKuvazen.from_folder(model_dir, torch.float64)


def plain_logits(model_dir: str, ids, dtype=torch.float64) -> torch.Tensor:
    m = PlainKuvazen.from_folder(model_dir, dtype)
    return m.forward(list(ids), m.new_state()).double()


def without_close_calls(raw: dict) -> dict:
    """The same configuration without the two places where rounding in a bfloat16 engine decides: every router chooses
    all its experts (their weights still differ token by token), and the side input has at least 16 columns.  No router
    of this design can be kept from close calls by its weights alone (its scores are a linear map of a zero-mean
    input), and the side input is a unit-size vector whose direction rests on a few products that may nearly cancel
    (with one column: on a sign).  The float32 runs keep the choice and the small sizes."""
    import copy
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    if raw.get("token_side"):
        raw["token_side"]["dim"] = max(16, raw["token_side"]["dim"])
    return raw


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square of the logits' difference (its mean over the vocabulary taken off) over the
    root mean square of the wanted logits."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), "engine produced non-finite logits"
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)


# float32: 1e-4, or three times what rounding alone does to the plain implementation run in float32 where that is more
# (tiny random models are ill-conditioned at a few positions: a norm over nearly cancelling values, a softmax of sharp
# scores); a wrong or missing term moves the logits by tenths
TOL = {"float32": 1e-4, "bfloat16": 5e-2}
