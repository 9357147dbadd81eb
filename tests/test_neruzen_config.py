"""The Neruzen configuration and description without a GPU: the round trip of config.json, the errors, which parts a
layer gets and what the cache is asked to hold."""
from __future__ import annotations

import copy

import pytest
import torch

from neruzen_models import CONFIGS


def test_round_trip_and_description():
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel

    for name, raw in CONFIGS.items():
        arch, config = load_config(copy.deepcopy(raw))
        assert arch.name == "Neruzen" and config.to_dict() == raw, name
        spec = arch.describe(config)
        assert all(layer.arrangement == "parallel" for layer in spec.layers)
        model = DecoderModel(spec, torch.float32, None)
        declared = model.weight_declarations()
        assert ("bigram" in declared) == ("embedding" in raw)
        for index, layer in enumerate(raw["layers"]):
            assert declared[f"l{index}.shift"].shape == (raw["width"],)
            assert (f"l{index}.mlp.router" in declared) == (layer["mlp"] is not None)
            if layer["type"] == "lightning":
                assert declared[f"l{index}.mix.norm"].shape == (layer["mixer"]["heads"] * layer["mixer"]["vdim"],)
            if layer["type"] == "retention":
                assert f"l{index}.mix.norm" not in declared
            if layer["mlp"] is not None:
                assert (f"l{index}.mlp.shared.gate" in declared) == ("shared" in layer["mlp"])


def test_what_the_cache_is_asked_for():
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.parts.base import KVNeed

    arch, config = load_config(copy.deepcopy(CONFIGS["a"]))
    model = DecoderModel(arch.describe(config), torch.float32, None)
    kv, state, source = model.cache_needs()
    # per layer: the mixer's entry, then the arrangement's own (the shifted row); last the embedding's previous token
    assert kv[0] == KVNeed(1, 64 + 16, 21, 0) and all(k is None for k in kv[1:])
    assert [tuple(s.shape) for s in state[1]] == [(96,)] and [tuple(s.shape) for s in state[2]] == [(3, 40, 24)]
    assert [(tuple(s.shape), s.dtype) for s in state[-1]] == [((), torch.int32)]
    assert model.embedding_entry == len(kv) - 1 and all(s is None for s in source)
    cache = model.new_cache(8, 2, device=None)
    assert len(cache.kv_groups) == 1 and cache.kv_groups[0].need.v_dim == 0


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="attention"), "known"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rotated part"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][2]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_errors(change, needle):
    from thintensor_b200.config.base import ConfigError
    from thintensor_b200.config.registry import load_config

    raw = copy.deepcopy(CONFIGS["a"])
    change(raw)
    with pytest.raises(ConfigError) as err:
        load_config(raw)
    assert needle in str(err.value)
