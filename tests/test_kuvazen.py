"""Kuvazen on the CPU: configuration, registry, declared tensors, the looped schedule, page groups of block summaries,
and the plain implementation against itself."""
import copy
import random

import pytest
import torch

from logssms_b200.cache import CacheManager, CacheNeeds, KVNeed, OutOfPages, PagedNeed, PagedTensor
from logssms_b200.config import ConfigError, make_model_config
from logssms_b200.config.kuvazen import KuvazenConfig
from logssms_b200.models import build_model

from plain import kuvazen_plain as P
from tiny_kuvazen import KUVA, make_kuvazen_dir, plain_model


def test_config_is_chosen_by_the_architecture_string_and_round_trips():
    cfg = make_model_config(KUVA["A"])
    assert isinstance(cfg, KuvazenConfig) and cfg.architectures == ("Kuvazen",)
    assert make_model_config(cfg.to_dict()).to_dict() == cfg.to_dict() == KUVA["A"]
    spec = cfg.model_spec()
    assert [b.kind for b in spec.layers] == ["prenorm_stream"] * 4
    assert [b.mixer.spec.kind for b in spec.layers] == ["pooled_window_attention", "mingru", "pooled_window_attention", "mingru"]
    assert [None if b.feed_forward is None else b.feed_forward.kind for b in spec.layers] == ["clamped_glu", "routed_mlp", "routed_mlp", None]
    a = spec.layers[0].mixer.spec
    assert (a.num_heads, a.num_kv_heads, a.window, a.pool, a.position.rotary_dim, a.value_position.rotary_dim) == (6, 2, 20, 5, 8, 24)
    r = spec.layers[1].feed_forward
    assert (r.score, r.expert, r.weigh, r.correction, r.top) == ("sigmoid", "silu", "input", False, 2)
    assert [s.side.offset for s in spec.layers] == [0, 6, 12, 18] and spec.layers[0].side.table_width == 24
    # the looped range three times in a row, every run with a cache layer of its own
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (3, 3), (2, 4), (3, 5), (2, 6), (3, 7)]
    assert [e.layer for e in make_model_config(KUVA["B"]).model_spec().schedule] == [0, 1, 2, 3]
    assert [e.layer for e in make_model_config(KUVA["C"]).model_spec().schedule] == [0, 1, 0, 1]


@pytest.mark.parametrize("edit, message", [
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=4), "top"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"].update(heads=5), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["mask"].pop("pool"), "pool"),
    (lambda r: r["layers"][0]["mixer"].update(vdim=9), "vdim"),
    (lambda r: r["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "neither"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["norm"].update(eps=0.0), "eps"),
])
def test_config_refuses_what_it_cannot_run(edit, message):
    raw = copy.deepcopy(KUVA["A"])
    edit(raw)
    with pytest.raises(ConfigError, match=message):
        make_model_config(raw)


def test_declared_tensors_carry_the_design_names():
    model = build_model(make_model_config(KUVA["A"]))
    names = {n: tuple(s.shape) for n, s in model.named_param_specs()}
    assert names["embed"] == (211, 64) and names["embed.norm"] == (64,) and names["side.embed"] == (211, 24)
    assert names["head"] == (211, 64) and names["final.norm"] == (64,)
    assert names["l0.mix.q"] == (96, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.v"] == (48, 64) and names["l0.mix.o"] == (64, 144)
    assert names["l1.mix.z.b"] == (40,) and names["l1.mix.x"] == (40, 64) and names["l1.mix.o"] == (64, 40)
    assert names["l1.mlp.router"] == (3, 64) and names["l1.mlp.e2.down"] == (64, 24) and "l1.mlp.correction" not in names
    assert names["l0.mlp.gate"] == (96, 64) and names["l0.ls2"] == (64,) and names["l2.side.gate"] == (6, 64) and names["l2.side.proj"] == (64, 6)
    assert "l3.ls1" in names and "l3.ls2" not in names and "l3.norm2" not in names        # no feed-forward: nothing of it is stored
    bare = {n for n, _ in build_model(make_model_config(KUVA["C"])).named_param_specs()}
    assert not any("side" in n for n in bare)                                                # no side input: no table, no tensors


def test_cache_needs_of_the_attention_layer_are_a_window_of_tokens_and_a_group_of_blocks():
    model = build_model(make_model_config(KUVA["B"]))
    needs = model.cache_needs()
    assert needs[0].kv.window == 24 and needs[0].more_paged[0].every == 24        # blocks longer than the window: the block being filled is kept
    assert needs[2].kv.window == 3 and needs[2].more_paged[0].every == 3
    assert needs[3].kv.window == 40 and needs[3].more_paged[0].every == 1
    assert needs[1].kv is None and needs[1].states[0].shape == (24,)


# --------------------------------------------------------------------------- page groups of one entry per block of tokens
def manager(pages=12, page=16, every=4, window=20, max_requests=3, **kw):
    tokens = KVNeed(2, 8, window, 6)
    blocks = PagedNeed((PagedTensor("k_pooled", (2, 8)), PagedTensor("v_pooled", (2, 6))), None, every)
    needs = [CacheNeeds(kv=tokens, more_paged=(blocks,)), CacheNeeds(kv=tokens, more_paged=(blocks,))]
    return CacheManager(needs, page_size=page, num_pages=pages, max_requests=max_requests, max_seq_len=1024,
                        dtype=torch.float32, device="cpu", **kw)


def test_a_group_of_block_summaries_has_one_entry_per_block_and_keeps_its_pages():
    m = manager()
    assert len(m.groups) == 2 and m.group_of_layer == {0: 0, 1: 0}
    t, gi = m.paged_tensor(1, "k_pooled")
    assert gi == 1 and t.shape[1:] == (16, 2, 8) and m.groups[1].need.every == 4
    assert m.groups[1].pool.count == 12 // 4 + 3                   # a quarter of the token pages and one per request
    assert m.groups[1].pages_for(64) == 1 and m.groups[1].pages_for(65) == 2 and m.groups[1].pages_for(1) == 1
    rc = m.admit()
    m.extend(rc, 100)
    assert m.groups[0].num_pages_of[rc.row] == 7 and m.groups[1].num_pages_of[rc.row] == 2
    m.extend(rc, 101)                                              # one more token: the window group gives pages back
    assert m.groups[0].first_page[rc.row] == (100 - 20 + 1) // 16 == 5
    assert m.groups[1].first_page[rc.row] == 0                     # ... the blocks stay for the request's life
    m.check_integrity()
    m.release(rc)
    m.check_integrity()
    assert m.groups[1].pool.num_free == m.groups[1].pool.count


def test_block_pages_run_dry_before_anything_grows_and_are_used_again():
    m = manager(pages=12, every=2, max_requests=2)                  # 12 token pages; 6 + 2 block pages of 16 blocks = 32 tokens each
    a, b = m.admit(), m.admit()
    m.extend(a, 60)
    m.extend(b, 60)
    with pytest.raises(OutOfPages):
        m.check_room([(a, 170), (b, 70)])                          # a would need 6 block pages, b 3: one more than there are
    assert m.live[a.row].length == 60
    m.release(a)
    c = m.admit()
    m.extend(c, 60)
    m.check_integrity()
    rng = random.Random(0)
    live = {b.row: b, c.row: c}
    for _ in range(200):                                           # random growth and release: nothing lost, nothing held twice
        rc = rng.choice(list(live.values()))
        try:
            m.check_room([(rc, rc.length + rng.randint(1, 9))])
            m.extend(rc, rc.length + rng.randint(1, 9))
        except OutOfPages:
            m.release(rc)
            del live[rc.row]
            new = m.admit()
            live[new.row] = new
        m.check_integrity()


def test_two_paged_needs_of_a_layer_must_not_share_a_tensor_name():
    tokens = KVNeed(2, 8)
    with pytest.raises(ValueError, match="clash"):
        CacheManager([CacheNeeds(kv=tokens, more_paged=(PagedNeed((PagedTensor("k", (2, 8)),), None, 4),))], page_size=16,
                     num_pages=4, max_requests=2, max_seq_len=64, dtype=torch.float32, device="cpu")
    with pytest.raises(ValueError, match="window"):
        PagedNeed((PagedTensor("x", (1,)),), 8, 4)


# --------------------------------------------------------------------------- the plain implementation against itself
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_model_gives_the_same_logits_in_pieces(tmp_path, name):
    model = plain_model(make_kuvazen_dir(tmp_path / "m", KUVA[name], seed=2, sharp=3.0))
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, KUVA[name]["vocab"], (90,), generator=g).tolist()
    whole = model.forward(ids, model.new_state())
    state, parts = model.new_state(), []
    for lo, hi in ((0, 1), (1, 30), (30, 32), (32, 89), (89, 90)):
        parts.append(model.forward(ids[lo:hi], state))
    assert float((torch.cat(parts) - whole).abs().max()) < 1e-9


def test_plain_attention_sees_the_window_and_only_the_blocks_wholly_behind_it():
    """One head, no rotation, keys that are unit vectors by position: the softmax weights name what is seen."""
    n, W_, P_ = 40, 6, 4
    h = torch.eye(n, dtype=torch.float64)
    Wm = {"q": torch.zeros(n, n, dtype=torch.float64),
          "k": torch.eye(n, dtype=torch.float64), "v": torch.eye(n, dtype=torch.float64), "o": torch.eye(n, dtype=torch.float64)}
    # zero queries: every visible key weighs the same, so the output is the mean of the visible values
    out = P.pooled_window_attention(h, Wm, {}, heads=1, kv_heads=1, dim=n, vdim=n, scale=1.0, window=W_, pool=P_, base=1e4, rot_dims=0)
    back = torch.stack([P.turn_pairs(out[i], i, 1e4, n) for i in range(n)])      # undo the turning back: values were turned by j
    for i in (3, 9, 10, 25):
        first, blocks = max(0, i - W_ + 1), max(0, (i - W_ + 1) // P_)
        seen = torch.zeros(n, dtype=torch.float64)
        for j in range(first, i + 1):
            seen += P.turn_pairs(torch.eye(n, dtype=torch.float64)[j], j, 1e4, n)
        for b in range(blocks):
            seen += torch.stack([P.turn_pairs(torch.eye(n, dtype=torch.float64)[j], j, 1e4, n) for j in range(b * P_, (b + 1) * P_)]).mean(0)
        assert float((back[i] - seen / (i + 1 - first + blocks)).abs().max()) < 1e-12
    # at i = 9 the tokens 0..3 are one block and the tokens 4..9 the window; at i = 10 token 4 has left the window and
    # its block (4..7) is not yet behind it: it is not seen at all
    assert blocks >= 0 and max(0, (10 - W_ + 1) // P_) == 1 and max(0, 10 - W_ + 1) == 5
