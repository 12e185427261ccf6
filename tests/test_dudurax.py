"""Dudurax on the CPU: configuration, registry, declared tensors, and the plain implementation against itself."""
import copy
import math

import pytest
import torch

from logssms_b200.config import ConfigError, make_model_config
from logssms_b200.config.dudurax import DuduraxConfig
from logssms_b200.models import build_model
from logssms_b200.weights.loader import WeightError, check_and_place
from logssms_b200.weights.random_init import random_tensors

from plain import dudurax_plain as P
from tiny_dudurax import DUDU, make_dudurax_dir, plain_model


def test_config_is_chosen_by_the_architecture_string_and_round_trips():
    cfg = make_model_config(DUDU["A"])
    assert isinstance(cfg, DuduraxConfig) and cfg.architectures == ("Dudurax",)
    assert make_model_config(cfg.to_dict()).to_dict() == cfg.to_dict() == DUDU["A"]
    spec = cfg.model_spec()
    assert [b.kind for b in spec.layers] == ["postnorm"] * 4
    assert [b.mixer.spec.kind for b in spec.layers] == ["latent_attention", "gla", "gla", "latent_attention"]
    assert [None if b.feed_forward is None else b.feed_forward.kind for b in spec.layers] == ["dense_mlp", "routed_mlp", None, "routed_mlp"]
    assert spec.layers[3].mixer.spec.window == 70 and spec.layers[3].mixer.spec.position.rotary_dim == 8
    assert spec.layers[1].feed_forward.num_identity == 2 and spec.layers[1].feed_forward.keep_groups == 2
    assert spec.layers[0].skip_scale == 2.0


@pytest.mark.parametrize("edit, message", [
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r.pop("postln_alpha"), "postln_alpha"),
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "neither"),
    (lambda r: r["norm"].update(eps=0.0), "eps"),
])
def test_config_refuses_what_it_cannot_run(edit, message):
    raw = copy.deepcopy(DUDU["A"])
    edit(raw)
    with pytest.raises(ConfigError, match=message):
        make_model_config(raw)


def test_declared_tensors_carry_the_design_names_and_the_decay_rank_may_come_from_the_checkpoint():
    model = build_model(make_model_config(DUDU["A"]))
    names = dict(model.named_param_specs())
    for n in ("embed", "bigram", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.dkv.norm", "l0.mix.uk", "l0.mlp.up",
              "l1.mix.a2.b", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e3.down", "l2.norm1", "l3.mlp.e2.gate"):
        assert n in names, n
    assert "l2.norm2" not in names and "l1.mlp.e4.gate" not in names
    assert names["bigram"].shape == (98, 64) and names["l1.mlp.router"].shape == (6, 64)
    # without `decay_rank` in config.json the rank is whatever the checkpoint has ...
    raw = copy.deepcopy(DUDU["A"])
    stored = random_tensors(model, 0, torch.float32)
    del raw["layers"][1]["mixer"]["decay_rank"]
    open_model = build_model(make_model_config(raw))
    assert dict(open_model.named_param_specs())["l1.mix.a1"].shape == (-1, 64)
    open_model.bind_tree(check_and_place(open_model, stored, torch.float32, "cpu"))
    assert open_model.layers[1].mixer.rank == 8
    # ... but every other size must fit
    stored["l1.mix.a1"] = torch.zeros(8, 63)
    with pytest.raises(WeightError, match="l1.mix.a1"):
        check_and_place(open_model, stored, torch.float32, "cpu")


def test_cache_needs_latents_in_pages_with_a_window_and_states_in_slots():
    needs = build_model(make_model_config(DUDU["A"])).cache_needs()
    assert [t.name for t in needs[0].kv.tensors] == ["c", "kr"] and needs[0].kv.window == 20
    assert [t.shape for t in needs[3].kv.tensors] == [(24,), (16,)] and needs[3].kv.window == 70
    assert needs[1].states[0].shape == (3, 16, 24) and needs[1].states[0].dtype == torch.float32
    assert needs[4].states[0].name == "previous_token" and needs[4].states[0].dtype == torch.int32


def test_plain_model_gives_the_same_logits_however_the_prompt_is_cut(tmp_path):
    md = make_dudurax_dir(tmp_path / "m", DUDU["A"], seed=2, sharp=4.0)
    m = plain_model(md)
    ids = torch.randint(0, 211, (100,), generator=torch.Generator().manual_seed(0)).tolist()
    whole = m.forward(ids, m.new_state())
    st, parts, p = m.new_state(), [], 0
    for n in [1, 2, 19, 1, 44, 2, 31]:
        parts.append(m.forward(ids[p:p + n], st))
        p += n
    assert p == 100 and torch.allclose(torch.cat(parts), whole, atol=1e-10)


def test_plain_router_groups_identity_and_negative_choice_scores():
    g = torch.Generator().manual_seed(1)
    h = torch.randn(200, 16, generator=g, dtype=torch.float64)
    W = torch.randn(6, 16, generator=g, dtype=torch.float64)
    corr = torch.tensor([-3.0, -3.0, -2.5, -2.5, -9.0, -9.0], dtype=torch.float64)       # every choice score is negative
    w = P.route(h, W, corr, top=2, groups=3, keep=2, scale=1.5)
    assert ((w > 0).sum(-1) == 2).all()
    assert (w[:, 4:] == 0).all()                              # the third group never makes it, although 0 > its scores
    s = torch.softmax(h @ W.T, -1)
    assert torch.allclose(w[w > 0], (1.5 * s)[w > 0])         # weights: the scores without the correction, not renormalised
    # an identity expert returns its input times the weight
    Wd = {"router": W, "correction": corr, **{f"e0.{n}": torch.randn(4, 16, generator=g, dtype=torch.float64) for n in ("gate", "up")},
          "e0.down": torch.randn(16, 4, generator=g, dtype=torch.float64)}
    only_identity = P.route(h, W, torch.tensor([-9.0, 0, 0, 0, 0, 0], dtype=torch.float64), top=5, groups=1, keep=1, scale=1.0)
    out = P.moe_ff(h, {**Wd, "correction": torch.tensor([-9.0, 0, 0, 0, 0, 0], dtype=torch.float64)}, experts=1, identity=5, top=5,
                   groups=1, keep=1, scale=1.0, limit=1.0)
    assert torch.allclose(out, h * only_identity[:, 1:].sum(-1, keepdim=True))


def test_plain_expert_clamps_and_gla_decay():
    h = torch.tensor([[10.0, -10.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    y = P.expert(h, eye, eye, eye, limit=2.0)
    g, u = torch.tensor([2.0, -10.0]), torch.tensor([2.0, -2.0])
    assert torch.allclose(y[0], (g * torch.sigmoid(1.702 * g) * (u + 1)).double())
    # one head, one key channel: S_t = a S_{t-1} + k v, o = q S / sqrt(1)
    W = {"q": torch.ones(1, 1), "k": torch.ones(1, 1), "v": torch.ones(1, 1), "g": torch.ones(1, 1), "o": torch.ones(1, 1),
         "norm": torch.ones(1), "a1": torch.zeros(1, 1), "a2": torch.zeros(1, 1), "a2.b": torch.tensor([0.0])}
    W = {k: v.double() for k, v in W.items()}
    st = {}
    P.gla(torch.ones(3, 1, dtype=torch.float64), W, st, heads=1, dim=1, vdim=1, tau=2.0, eps=0.0)
    a = math.sqrt(0.5)
    assert abs(float(st["S"]) - (a * a + a + 1)) < 1e-12
