"""What can be checked of the Mupuvik design without a GPU: the configuration reads and writes back, the
description names the checkpoint's tensors, the cache gives every part what it asked for (a layer that reads
another layer's keys the owner's pages, kept as long as the longest reader needs them), and the plain
implementation gives the same rows however a prompt is cut."""

from __future__ import annotations

import json
import math

import pytest
import torch

import mupuvik_configs
import plain_mupuvik


def typed(raw):
    import vllm_from_scratch_b200 as engine
    return engine.load_model_config(raw)


@pytest.mark.parametrize("name", list(mupuvik_configs.CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    raw, _ = mupuvik_configs.CONFIGS[name]
    entry, config = typed(raw)
    assert entry.name == "Mupuvik"
    again = entry.config_class.from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config
    from vllm_from_scratch_b200.parts.model import DecoderModel
    model = DecoderModel(entry.build_spec(config), torch.float32, "cpu")
    weights = entry.random_weights(config, 1, decay_rank=5)
    expected = model.expected_weights()
    assert set(expected) == set(weights)
    for key, info in expected.items():
        assert len(info.shape) == weights[key].dim(), key
        assert all(want is None or want == found for want, found in zip(info.shape, weights[key].shape)), key
    for index, layer in enumerate(raw["layers"]):
        assert (f"l{index}.norm2" in expected) == (layer["mlp"] is not None)
        reads = layer["mixer"].get("kv_from") is not None
        if layer["type"] == "attention":
            assert (f"l{index}.mix.k" in expected) == (not reads) and f"l{index}.mix.q.b" in expected
            assert (f"l{index}.mix.k.norm" in expected) == (not reads) and f"l{index}.mix.g" in expected
        if layer["mlp"] is not None:
            assert (f"l{index}.mlp.shared.up" in expected) == ("shared" in layer["mlp"])
    assert "head" not in expected and "head.weight" not in expected        # the logits use the embedding's table


def test_configuration_refuses_what_the_design_has_not():
    from vllm_from_scratch_b200.config import ConfigError
    def changed(edit):
        raw = json.loads(json.dumps(mupuvik_configs.MV_A))
        edit(raw)
        return raw
    for edit in (lambda raw: raw["layers"][0].update(type="convolution"),
                 lambda raw: raw["layers"][0]["mlp"].update(kind="dense"),
                 lambda raw: raw["layers"][0]["mlp"]["router"].update(top=9),
                 lambda raw: raw["layers"][1]["mixer"].update(kv_from=3),              # not an earlier layer
                 lambda raw: raw["layers"][4]["mixer"].update(kv_from=1),              # a layer that owns no keys
                 lambda raw: raw["layers"][1]["mixer"].update(dim=8),                  # other sizes than the owner's
                 lambda raw: raw["layers"][2]["mixer"]["left"]["rot"].update(dims=7),
                 lambda raw: raw["layers"][2]["mixer"]["right"].update(tau=0.0),
                 lambda raw: raw.pop("norm"),
                 lambda raw: raw["embedding"].pop("scale")):
        with pytest.raises(ConfigError):
            typed(changed(edit))


def test_cache_lends_pages_and_keeps_them_for_the_longest_reader():
    from vllm_from_scratch_b200.cache import CacheStorage
    from vllm_from_scratch_b200.parts.model import DecoderModel
    entry, config = typed(mupuvik_configs.MV_A)
    spec = entry.build_spec(config)
    assert [e.cache_from for e in spec.schedule] == [None, 0, None, None, 0]
    model = DecoderModel(spec, torch.float32, "cpu")
    storage = CacheStorage(model.cache_needs(), [e.cache_from for e in spec.schedule], 16, 6, 3, torch.float32, "cpu",
                           embedding_need=model.embedding.cache_need())
    # the owner's window is 24, its readers' 40 and 9: the pages are kept for 40 positions
    assert sorted(storage.group_windows, key=str) == [40, None]
    owner, longer, pair, scan, shorter = storage.views
    assert owner.writable and not longer.writable and not shorter.writable
    assert longer.keys.data_ptr() == owner.keys.data_ptr() == shorter.keys.data_ptr()
    assert owner.keys.shape == (6, 2, 16, 16) and owner.values.shape == (6, 2, 16, 24)
    assert pair.kind == "pages" and set(pair.states) == {"right.state"} and pair.states["right.state"].shape == (4, 2, 8, 16)
    assert set(scan.states) == {"state", "conv"}
    assert storage.embedding_view.state.dtype == torch.int32
    for tensor in storage.states.values():
        tensor.fill_(7)
    storage.zero_slots([2])
    for tensor in storage.states.values():
        assert not tensor[2].any() and tensor[0].eq(7).all()


def test_an_unknown_rank_is_the_checkpoints_to_give():
    from vllm_from_scratch_b200.parts.model import DecoderModel
    from vllm_from_scratch_b200.weights.loader import WeightLoadError, load_weights_from_tensors
    entry, config = typed(mupuvik_configs.MV_A)
    for rank in (1, 7):
        model = DecoderModel(entry.build_spec(config), torch.float32, "cpu")
        load_weights_from_tensors(model, entry.random_weights(config, 3, decay_rank=rank, dtype=torch.float32))
        assert model.layers[2].mixer.branches[1].down.shape[0] == rank
    weights = entry.random_weights(config, 3, decay_rank=4, dtype=torch.float32)
    weights["l2.mix.right.a2"] = weights["l2.mix.right.a2"][:, :3].contiguous()     # the two ranks differ
    with pytest.raises(ValueError):
        load_weights_from_tensors(DecoderModel(entry.build_spec(config), torch.float32, "cpu"), weights)
    weights = entry.random_weights(config, 3, dtype=torch.float32)
    weights["l2.mix.right.a1"] = weights["l2.mix.right.a1"][:, :5].contiguous()     # a size that is known
    with pytest.raises(WeightLoadError):
        load_weights_from_tensors(DecoderModel(entry.build_spec(config), torch.float32, "cpu"), weights)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_plain_implementation_does_not_depend_on_the_cut(name):
    raw, _ = mupuvik_configs.CONFIGS[name]
    entry, config = typed(raw)
    weights = entry.random_weights(config, 5, dtype=torch.float32)
    model = plain_mupuvik.PlainMupuvik(raw, weights, torch.float64)
    tokens = torch.randint(0, raw["vocab"], (23,), generator=torch.Generator().manual_seed(2)).tolist()
    trail = []
    whole = model.feed(model.new_state(), tokens, trail)
    state, rows, done = model.new_state(), [], 0
    for size in (1, 2, 5, 1, 1, 7, 6):
        rows.append(model.feed(state, tokens[done:done + size]))
        done += size
    cut = torch.cat(rows)
    assert cut.shape == whole.shape == (len(tokens), raw["vocab"]) and len(trail) == len(tokens)
    assert trail[0].shape == (len(raw["layers"]), raw["width"])
    assert float((cut - whole).abs().max()) < 1e-9


def test_plain_pieces():
    # neighbours are turned, what lies behind the rotated part stays, and position 0 turns nothing
    x = torch.arange(12, dtype=torch.float64).view(1, 12) + 1.0
    assert torch.equal(plain_mupuvik.rotate_pairs(x, 0, 10.0, 8), x)
    turned = plain_mupuvik.rotate_pairs(x, 3, 10.0, 8)
    assert torch.equal(turned[:, 8:], x[:, 8:])
    assert math.isclose(float(turned[0, 0]), 1.0 * math.cos(3.0) - 2.0 * math.sin(3.0))
    assert math.isclose(float(turned[0, 3]), 4.0 * math.cos(3.0 * 10 ** -0.25) + 3.0 * math.sin(3.0 * 10 ** -0.25))
    # one more in the denominator: with a single key of score 0 half of its value comes through
    q, keys, values = torch.zeros(1, 4, dtype=torch.float64), torch.ones(1, 1, 4, dtype=torch.float64), torch.ones(1, 1, 2, dtype=torch.float64)
    assert torch.allclose(plain_mupuvik.attend(q, keys, values, 1.0, 1, 0, True), torch.full((1, 2), 0.5, dtype=torch.float64))
    assert torch.allclose(plain_mupuvik.attend(q, keys, values, 1.0, 1, 0, False), torch.ones(1, 2, dtype=torch.float64))
    # the first token of a sequence takes the table's last row
    assert plain_mupuvik.bigram_row(None, 5, 3, 7, 11) == 11 and plain_mupuvik.bigram_row(4, 5, 3, 7, 11) == (12 + 35) % 11
