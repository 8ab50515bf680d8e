"""Redudra without a GPU: configuration, plan and schedule of looped layers, what each layer run keeps, the cache
bookkeeping of a window that keeps a request's first tokens, the rotary table against the oracle's frequencies, and the
oracle's own parts by hand."""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest
import torch

import plain_redudra as pr
import redudra_util as ru
from acvram_b200.cache.manager import CacheManager, CachePlan, PagedNeed, StateNeed
from acvram_b200.config import ConfigError, RedudraConfig, family_of
from acvram_b200.models import needs_of_plan
from acvram_b200.models.decoder import DecoderModel
from acvram_b200.parts import Runtime
from acvram_b200.parts.position import Rotary


@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
def test_config_round_trip_plan_and_schedule(which):
    raw = ru.config(which)
    cfg = RedudraConfig.from_dict(raw)
    assert RedudraConfig.from_dict(cfg.to_dict()) == cfg
    family = family_of(raw)
    assert family.name == "Redudra"
    plan = family.build_plan(cfg)
    assert plan.residual_dtype == "float32" and plan.logit_softcap == raw.get("logit_softcap", 0.0)
    # the schedule is the oracle's run order, every run with a cache slot of its own, a pass's first run with its vector
    order = pr.run_order(raw)
    assert [e.layer for e in plan.schedule] == [i for i, _ in order]
    assert sorted(e.cache for e in plan.schedule) == list(range(len(order)))
    first = raw["loop"]["start"] if raw.get("loop") else -1
    assert [e.stream_add for e in plan.schedule] == [("loop.step", p) if p is not None and i == first else None for i, p in order]
    # the tensors asked for are exactly the design's names and shapes
    weights = ru.random_weights(raw, 0)
    needs = needs_of_plan(plan)
    assert set(needs) == set(weights)
    for name, t in weights.items():
        assert tuple(needs[name].shape) == tuple(t.shape), name


def test_config_errors_name_the_key():
    raw = ru.config("A")
    for change, word in ((lambda c: c["layers"][0].__setitem__("type", "attention"), "type"),
                         (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("heads", 3), "kv_heads"),
                         (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
                         (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "dims"),
                         (lambda c: c["layers"][1]["mixer"].__setitem__("blocks", 5), "blocks"),
                         (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "kind"),
                         (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
                         (lambda c: c.pop("norm"), "norm"), (lambda c: c.pop("vocab"), "vocab")):
        bad = copy.deepcopy(raw)
        change(bad)
        with pytest.raises(ConfigError, match=word):
            RedudraConfig.from_dict(bad)


def test_what_every_layer_run_keeps():
    raw = ru.config("A")
    model = DecoderModel(family_of(raw).build_plan(RedudraConfig.from_dict(raw)))
    plan = model.cache_plan()
    runs = pr.run_order(raw)
    # a parallel run keeps pages, a retention state and the shifted row; a recurrent run its state, its convolution's
    # inputs and the shifted row
    assert len(plan.needs) == 3 * len(runs)
    for slot, (layer, _) in enumerate(runs):
        names = [path for path, _ in model.slot_leaves[slot]]
        if raw["layers"][layer]["type"] == "parallel":
            assert names == [("mixer", "left"), ("mixer", "right"), ("shift",)]
        else:
            assert names == [("mixer", "state"), ("mixer", "conv"), ("shift",)]
    l0 = raw["layers"][0]["mixer"]["left"]
    assert PagedNeed(l0["kv_heads"], l0["dim"], 20, l0["vdim"], 0, 3) in plan.groups
    assert StateNeed((3, 8, 16), "float32") in plan.groups and StateNeed((2, 64), "float32") in plan.groups
    # the shifted rows of all runs share one group, the three passes of layer 0 each have their own pages
    shift = plan.groups.index(StateNeed((96,), "float32"))
    assert plan.slots_per_group[shift] == len(runs)
    assert plan.slots_per_group[plan.groups.index(PagedNeed(2, 16, 20, 24, 0, 3))] == 3
    # one tap: nothing of the convolution is kept
    b = ru.config("B")
    mb = DecoderModel(family_of(b).build_plan(RedudraConfig.from_dict(b)))
    mb.cache_plan()
    assert [path for path, _ in mb.slot_leaves[0]] == [("mixer", "state"), ("shift",)]


@pytest.mark.parametrize("window,keep,page", [(20, 3, 8), (7, 9, 4), (48, 4, 16), (10, 0, 4), (5, 16, 4)])
def test_window_gives_pages_back_but_keeps_the_first_tokens(window, keep, page):
    need = PagedNeed(1, 8, window, 0, 0, keep)
    m = CacheManager(CachePlan([need, StateNeed((4,))]), page, 64, 2)
    m.admit("r")
    length = 0
    for portion in (3, 30, 1, 1, 17, 2, 1, 1, 1, 40, 1):
        m.grow("r", length + portion)
        length += portion
        m.advance("r", length)
        m.trim("r")
        m.check()
        table = m.block_table("r", 0)
        # every position that a later query (at length or beyond) may read is still there, and nothing else but
        # what shares a page with such a position
        needed = {j // page for j in range(length) if pr.visible(length, j, window, keep)}
        held = {i for i, p in enumerate(table) if p >= 0}
        assert needed <= held, f"length {length}: pages {sorted(needed - held)} were given back too early"
        assert held == needed | {i for i in held if i >= (length - window + 1) // page}
    m.release("r")
    assert m.free_pages() == [64] and m.state_groups[0].num_free == 2


def test_state_slots_come_back_and_go_out_again():
    m = CacheManager(CachePlan([StateNeed((4,)), PagedNeed(1, 8, 6, 0, 0, 2)]), 4, 16, 2)
    a = m.admit("a")
    b = m.admit("b")
    assert not m.can_admit() and a[0] != b[0]
    m.release("a")
    c = m.admit("c")
    assert c[0] == a[0], "the freed slot is the one given out next"
    m.check()


@pytest.mark.parametrize("rot", [ru.rot(5000.0, 8, (3.0, 64, 8.0, 1.0)), ru.rot(30000.0, 64, (3.0, 128, 16.0, 1.0)),
                                 ru.rot(777.0, 10, (2.5, 40, 4.0, 0.5)), ru.rot(300.0, 16)])
def test_rotary_table_has_the_oracles_frequencies(rot):
    sc = rot.get("scaling")
    part = Rotary(0, rot["dims"], rot["base"], 300, tuple(sc[k] for k in ("factor", "original", "fast", "slow")) if sc else None,
                  exact=True)
    part.load({}, Runtime(torch.device("cpu"), torch.float32))
    f, mag = pr.rotary_frequencies(rot)
    ang = np.arange(300)[:, None] * f[None, :]
    want = np.concatenate([np.cos(ang), np.sin(ang)], axis=1) * mag
    assert np.abs(part.rotary_table().numpy() - want).max() < 1e-7
    if sc:      # the scaling does something: slow pairs turn more slowly than the plain ones, fast pairs as before
        plain, _ = pr.rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
        assert f[-1] < plain[-1] and f[0] == plain[0] and mag > 1.0


def test_oracle_parts_by_hand():
    assert [j for j in range(12) if pr.visible(11, j, 4, 2)] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(12) if pr.visible(11, j, 0, 0)] == list(range(12))
    assert [j for j in range(5) if pr.visible(2, j, 4, 2)] == [0, 1, 2]
    h = np.array([[1.0, 2.0], [3.0, 6.0], [5.0, 5.0]])
    np.testing.assert_allclose(pr.token_shift(h, np.array([0.5, 1.0])), [[0.5, 0.0], [2.0, 2.0], [4.0, 6.0]])
    x = np.arange(1.0, 5.0)[:, None]
    np.testing.assert_allclose(pr.causal_conv(x, np.array([[100.0, 10.0, 1.0]]), np.array([0.5]))[:, 0],
                               [1.5, 12.5, 123.5, 234.5])
    np.testing.assert_allclose(pr.layer_norm(np.array([[1.0, 3.0]]), np.array([2.0, 2.0]), np.array([1.0, 0.0]), 0.0), [[-1.0, 2.0]])
    assert abs(pr.gelu_tanh(np.array([1.0]))[0] - 0.8411919906082768) < 1e-12
    assert abs(pr.softplus(np.array([0.0]))[0] - math.log(2.0)) < 1e-15
    # a pair turned by a quarter turn
    q = np.array([[[1.0, 0.0, 7.0]]])
    out = pr.rotate(np.repeat(q, 2, axis=0), {"base": 1.0, "dims": 2}, [0, math.pi / 2])
    np.testing.assert_allclose(out[1, 0], [0.0, 1.0, 7.0], atol=1e-15)
    # retention with one head of one element: o_t = q_t sum_j decay^(t-j) k_j v_j
    W = {"p.q": np.eye(1), "p.k": np.eye(1), "p.v": np.eye(1), "p.g": np.eye(1), "p.o": np.eye(1)}
    hh = np.array([[1.0], [2.0], [3.0]])
    want = np.array([1.0, 2 * (0.5 + 4), 3 * (0.25 + 0.5 * 4 + 9)])[:, None]
    got = pr.retention(hh, W, "p.", {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5]}, 0.0)
    np.testing.assert_allclose(got, np.sign(want) * pr.silu(hh))
    cfg = {"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 2}}
    assert pr.run_order(cfg) == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (3, None)]
