"""The Nodopel design without a GPU: its configuration reads and writes back, its description names the tensors
of a model folder, looped layers appear once per run with a cache of their own, the cache keeps the pages of the
first positions that stay visible, and the rotation's frequencies follow the plain rule."""

from __future__ import annotations

import copy

import pytest
import torch

import nodopel_configs
import plain_nodopel as plain


@pytest.mark.parametrize("name", list(nodopel_configs.CONFIGS))
def test_config_round_trip_and_names(name):
    import vllm_from_scratch_b200 as engine
    from vllm_from_scratch_b200.parts.model import DecoderModel
    raw = nodopel_configs.CONFIGS[name][0]
    entry, typed = engine.load_model_config(raw)
    assert entry.name == "Nodopel"
    assert entry.config_class.from_dict(typed.to_dict()) == typed
    spec = entry.build_spec(typed)
    model = DecoderModel(spec, torch.float32, "cpu")
    weights = entry.random_weights(typed, 3)
    expected = model.expected_weights()
    assert set(weights) == set(expected)
    for key, info in expected.items():
        assert tuple(weights[key].shape) == tuple(info.shape), key
    assert model.graph_safe()
    assert [entry.layer for entry in spec.schedule] == plain.schedule_of(raw)
    assert spec.streams == raw.get("streams")


def test_looped_layers_own_a_cache_per_run():
    import vllm_from_scratch_b200 as engine
    from vllm_from_scratch_b200.cache import CacheStorage
    from vllm_from_scratch_b200.parts.model import DecoderModel
    entry, typed = engine.load_model_config(nodopel_configs.ND_A)
    spec = entry.build_spec(typed)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    model = DecoderModel(spec, torch.float32, "cpu")
    needs = model.cache_needs()
    assert all(need is not None for need in needs)
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].value_dim) == (2, 32, 24)       # both maps in a key row
    assert (needs[0].window, needs[0].keep_first) == (20, 3)
    assert (needs[5].window, needs[5].keep_first) == (None, 0)
    storage = CacheStorage(needs, [None] * len(needs), 4, 10, 2, torch.float32, "cpu")
    # the two runs of layer 1 share a group (the same need) and own a slice each
    views = storage.views
    assert views[1].group == views[3].group and views[1].keys.data_ptr() != views[3].keys.data_ptr()
    assert views[2].group == views[4].group != views[1].group
    assert storage.group_keep_first == [group.need.keep_first for group in storage.groups]


def test_first_pages_stay_while_the_window_moves():
    from vllm_from_scratch_b200.cache import RELEASED, CacheManager
    # group 0: window 10, the first 6 positions kept (two pages of 4); group 1: window 10, none kept; group 2: all keys
    manager = CacheManager([10, 10, None], 4, 16, 2, group_keep_first=[6, 0, 0])
    manager.admit("a")
    assert manager.allocate("a", 40)
    manager.commit("a", 40)
    kept, moving, full = (manager.block_table("a", group) for group in range(3))
    # the next query sits at 40 and reads from 31 on: pages 0 .. 6 lie wholly behind it
    assert [page != RELEASED for page in kept] == [True, True] + [False] * 5 + [True] * 3
    assert [page != RELEASED for page in moving] == [False] * 7 + [True] * 3
    assert all(page != RELEASED for page in full)
    assert manager.num_free_pages(0) == 16 - 5 and manager.num_free_pages(1) == 16 - 3
    manager.check_invariants()
    # pages that came back are handed out again, to the same request and to another
    manager.admit("b")
    assert manager.allocate("b", 8) and manager.allocate("a", 48)
    manager.commit("a", 48)
    assert [page != RELEASED for page in manager.block_table("a", 0)] == [True, True] + [False] * 7 + [True] * 3
    manager.check_invariants()
    manager.release("a")
    assert manager.num_free_pages(0) == 16 - 2
    # a request that is preempted starts again with its first pages kept
    manager.commit("b", 8)
    manager.drop_pages("b")
    assert manager.allocate("b", 30)
    manager.commit("b", 30)
    assert [page != RELEASED for page in manager.block_table("b", 0)] == [True, True] + [False] * 3 + [True] * 3
    manager.release("b")
    manager.check_invariants()
    assert all(manager.num_free_pages(group) == 16 for group in range(3))


@pytest.mark.parametrize("rot", [
    {"dims": 8, "base": 10000.0},
    {"dims": 24, "base": 500.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
    {"dims": 64, "base": 1.0e6, "scaling": {"factor": 3.0, "low": 0.5, "high": 1.5, "original": 20}},
])
def test_frequencies(rot):
    from vllm_from_scratch_b200.parts.base import POSITION_ENCODINGS, PartEnv
    scaling = rot.get("scaling")
    params = {"theta": rot["base"], "rotary_dim": rot["dims"],
              "frequency_scaling": None if scaling is None else tuple(scaling[k] for k in ("factor", "low", "high", "original"))}
    part = POSITION_ENCODINGS.get("rotary")(params, PartEnv(16, torch.float32, torch.device("cpu"), ""))
    want = torch.tensor(plain.rotary_frequencies(rot), dtype=torch.float64)
    got = part.inverse_frequencies().double()
    assert torch.allclose(got, want, rtol=2e-7, atol=0)
    if scaling is not None:
        plain_rule = torch.tensor(plain.rotary_frequencies({"dims": rot["dims"], "base": rot["base"]}), dtype=torch.float64)
        ratio = want / plain_rule
        # all three branches occur: kept, divided by the factor, and between the two
        assert (ratio == 1).any() and torch.isclose(ratio, torch.tensor(1 / scaling["factor"], dtype=torch.float64)).any()
        assert ((ratio < 1 - 1e-9) & (ratio > 1 / scaling["factor"] + 1e-9)).any()


def test_visibility_rule_of_the_plain_implementation():
    mask = {"size": 5, "keep_first": 2}
    assert [j for j in range(12) if plain.sees(9, j, mask)] == [0, 1, 5, 6, 7, 8, 9]
    assert [j for j in range(12) if plain.sees(3, j, mask)] == [0, 1, 2, 3]
    assert [j for j in range(12) if plain.sees(9, j, {"size": 5})] == [5, 6, 7, 8, 9]
    assert [j for j in range(12) if plain.sees(4, j, None)] == [0, 1, 2, 3, 4]


@pytest.mark.parametrize("change, message", [
    (lambda raw: raw["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=18), "exceeds dim"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda raw: raw["layers"][1]["mlp"]["router"].update(top=9), "top=9"),
    (lambda raw: raw["layers"][1]["mlp"].update(kind="other"), "part of the design"),
    (lambda raw: raw["layers"][1].update(type="mamba2"), "not a mixer of this design"),
    (lambda raw: raw["loop"].update(stop=7), "does not lie within"),
    (lambda raw: raw["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
])
def test_config_errors(change, message):
    import vllm_from_scratch_b200 as engine
    raw = copy.deepcopy(nodopel_configs.ND_A)
    change(raw)
    with pytest.raises(Exception, match=message):
        engine.load_model_config(raw)


def test_plain_model_feeds_token_by_token():
    """The plain implementation keeps a request's past itself: two requests fed in turns give what each gives alone."""
    import vllm_from_scratch_b200 as engine
    raw = nodopel_configs.ND_C
    entry, typed = engine.load_model_config(raw)
    weights = {k: v.double() for k, v in entry.random_weights(typed, 5, dtype=torch.float32).items()}
    tokens = {"x": [3, 9, 1, 40, 7, 7, 2], "y": [5, 0, 60, 11]}
    alone = {rid: plain.PlainNodopel(raw, weights).run(rid, seq) for rid, seq in tokens.items()}
    model = plain.PlainNodopel(raw, weights)
    rows = {"x": [], "y": []}
    for i in range(7):
        for rid in ("x", "y"):
            if i < len(tokens[rid]):
                rows[rid].append(model.step(rid, tokens[rid][i]))
    for rid in tokens:
        assert torch.equal(torch.stack(rows[rid]), alone[rid])
