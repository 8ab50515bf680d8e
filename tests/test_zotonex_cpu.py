"""Zotonex without a GPU: configuration, plan, cache bookkeeping of the chunked mask, and the oracle's own parts."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_zotonex as pz
import zotonex_util as zu
from acvram_b200.cache.manager import CacheManager, CachePlan, PagedNeed
from acvram_b200.config import ConfigError, ZotonexConfig, family_of
from acvram_b200.models import needs_of_plan
from acvram_b200.models.decoder import DecoderModel


@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_config_round_trip_and_plan(which):
    raw = zu.config(which)
    cfg = ZotonexConfig.from_dict(raw)
    assert ZotonexConfig.from_dict(cfg.to_dict()) == cfg
    family = family_of(raw)
    assert family.name == "Zotonex"
    plan = family.build_plan(cfg)
    assert plan.residual_dtype == "float32" and plan.embedding_scale == raw["embedding"]["scale"]
    # a reader runs on the slot of the layer it names and writes nothing
    slots = {}
    for i, (layer, entry) in enumerate(zip(raw["layers"], plan.schedule)):
        j = layer["mixer"].get("kv_from")
        if j is None:
            slots[i] = entry.cache
            assert entry.writes
        else:
            assert entry.cache == slots[j] and not entry.writes
    # the tensors asked for are exactly the design's names
    assert set(needs_of_plan(plan)) == set(zu.random_weights(raw, 0))
    for name, t in zu.random_weights(raw, 0).items():
        assert tuple(needs_of_plan(plan)[name].shape) == tuple(t.shape), name


def test_config_errors_name_the_key():
    raw = zu.config("A")
    for change, word in ((lambda c: c["layers"][0].__setitem__("type", "recurrent"), "type"),
                         (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 2), "kv_from"),
                         (lambda c: c["layers"][1]["mixer"].__setitem__("vdim", 32), "vdim"),
                         (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "kv_heads"),
                         (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
                         (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "kind"),
                         (lambda c: c.pop("norm"), "norm"), (lambda c: c.pop("vocab"), "vocab")):
        bad = copy.deepcopy(raw)
        change(bad)
        with pytest.raises(ConfigError, match=word):
            ZotonexConfig.from_dict(bad)


def test_cache_plan_groups_and_widening():
    # A: both slots have rows of other sizes (2 x 16 | 24 and 2 x 8 | 16) -> two groups; the reader shares the writer's slot
    plan = DecoderModel(family_of(zu.config("A")).build_plan(ZotonexConfig.from_dict(zu.config("A")))).cache_plan()
    assert plan.needs == [PagedNeed(2, 32, 0, 24, 24), PagedNeed(2, 16, 0, 0, 24)]
    # C: readers with chunks of 10 and none on a writer with chunks of 7: the slot keeps everything
    plan = DecoderModel(family_of(zu.config("C")).build_plan(ZotonexConfig.from_dict(zu.config("C")))).cache_plan()
    assert plan.needs == [PagedNeed(3, 48, 0, 40, 0)]
    assert PagedNeed(2, 32, 0, 24, 24).widened(PagedNeed(2, 32, 0, 24, 24)).chunk == 24
    with pytest.raises(ValueError):
        PagedNeed(2, 32, 0, 24, 24).widened(PagedNeed(2, 32, 0, 16, 24))


def test_chunked_need_gives_pages_back_at_chunk_borders():
    need = PagedNeed(1, 8, 0, 0, 10)
    assert [need.first_needed(n) for n in (0, 9, 10, 11, 19, 20, 35)] == [0, 0, 10, 10, 10, 20, 30]
    m = CacheManager(CachePlan([need]), 4, 6, 2)       # pages of 4 tokens, chunks of 10
    m.admit("a")
    g = m.paged_groups[0]
    held = lambda: [p for p in g.tables["a"] if p >= 0]
    for length, live_from in ((9, 0), (10, 2), (13, 2), (21, 5)):
        m.grow("a", length)
        m.advance("a", length)
        m.trim("a")
        # pages wholly before the chunk of the next token are gone, the page that the chunk starts in stays
        assert g.first_live["a"] == live_from, (length, g.first_live["a"])
        assert len(held()) == g.pages_for(length) - live_from
        m.paged_groups[0].pool.check()
    # a second request runs on the pages that the first gave back, in a pool too small for both in full
    m.admit("b")
    m.grow("b", 12)
    assert m.paged_groups[0].pool.num_free == 6 - 1 - 3
    m.release("a")
    m.release("b")
    assert m.paged_groups[0].pool.num_free == 6
    # a window and a chunk together: the later of the two bounds
    both = PagedNeed(1, 8, 6, 0, 10)
    assert [both.first_needed(n) for n in (5, 9, 12, 18, 20)] == [0, 4, 10, 13, 20]
    assert not both.takes_over and not need.takes_over and PagedNeed(1, 8).takes_over


def test_oracle_parts():
    """The oracle's own mechanisms against numbers worked out by hand."""
    # chunk mask: 5 positions, chunks of 2
    seen = pz.chunk_mask(5, 2)
    assert seen.int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 0, 1]]
    assert pz.chunk_mask(3, None).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    # expert: clamps and the +1 on the linear branch
    one = torch.ones(1, 1, dtype=torch.float64)
    x = torch.tensor([[4.0]], dtype=torch.float64)
    y = pz.expert(x, one, -one, one, 3.0)            # g = min(4, 3) = 3, u = clamp(-4) = -3: 3 * sigmoid(5.106) * (-2)
    assert abs(float(y) - 3.0 / (1.0 + pow(2.718281828459045, -5.106)) * -2.0) < 1e-9
    # routing: the scores themselves, not renormalised, largest first
    idx, w = pz.route(torch.tensor([[1.0, 0.0]], dtype=torch.float64), torch.tensor([[0.0, 0.0], [2.0, 0.0], [-1.0, 0.0]], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 0]] and abs(float(w[0, 0]) - 0.8807970779778823) < 1e-12 and float(w[0, 1]) == 0.5
    # differential attention: one query over two keys, maps with known weights
    q = torch.zeros(1, 1, 2, 2, dtype=torch.float64)
    k = torch.zeros(2, 1, 2, 2, dtype=torch.float64)
    q[0, 0, 1, 0] = 1.0
    k[1, 0, 1, 0] = 30.0                             # map 2 looks at key 1 alone; map 1 is uniform
    v = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]], dtype=torch.float64)
    o = pz.diff_core(q, k, v, torch.ones(1, 2, dtype=torch.bool), 1.0, 0.5, 0.25, 0.0)
    want = torch.tensor([0.5, 0.5 - 0.5])           # o1 = (.5, .5), o2 = (0, 1): o = (.5, 0) -> unit rms -> (sqrt 2, 0) * .75
    assert torch.allclose(o, torch.tensor([[2 ** 0.5 * 0.75, 0.0]], dtype=torch.float64), atol=1e-9), (o, want)
