"""The Famalorn configuration, its description as parts, and what the cache is asked to hold (no GPU)."""
from __future__ import annotations

import copy

import pytest
import torch

from famalorn_models import CONFIGS


def test_round_trip_and_registry():
    from thintensor_b200.config import ConfigError, FamalornConfig, load_config

    for raw in CONFIGS.values():
        arch, config = load_config(raw)
        assert arch.name == "Famalorn" and isinstance(config, FamalornConfig)
        assert config.to_dict() == raw
        assert load_config(config.to_dict())[1] == config
    broken = copy.deepcopy(CONFIGS["p"])
    broken["layers"][1]["type"] = "retention"
    with pytest.raises(ConfigError, match="retention"):
        load_config(broken)
    broken = copy.deepcopy(CONFIGS["p"])
    del broken["layers"][2]["mixer"]["state"]
    with pytest.raises(ConfigError, match="state"):
        load_config(broken)
    broken = copy.deepcopy(CONFIGS["p"])
    broken["layers"][0]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="multiple"):
        load_config(broken)
    broken = copy.deepcopy(CONFIGS["p"])
    broken["layers"][0]["mlp"]["kind"] = "routed"
    with pytest.raises(ConfigError, match="mlp"):
        load_config(broken)


def test_description_and_cache_needs():
    from thintensor_b200.config import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.parts.base import KVNeed, StateNeed

    arch, config = load_config(CONFIGS["p"])
    spec = arch.describe(config)
    assert [layer.arrangement for layer in spec.layers] == ["pre_norm_pair", "pre_norm", "pre_norm"]
    assert "ffn" not in spec.layers[1].parts and "ffn" in spec.layers[2].parts
    assert spec.layers[0].params == {"left_scale": 0.7, "right_scale": 1.3}
    model = DecoderModel(spec, torch.float32, None)
    names = model.weight_declarations()
    assert names["l0.mix.left.sink"].shape == (4,) and names["l0.mix.left.q.norm"].shape == (32,)
    assert names["l0.mix.left.v"].shape == (2 * 24, 96) and names["l0.mix.left.o"].shape == (96, 4 * 24)
    assert names["l0.mix.right.in"].shape == (2 * 48 + 2 * 3 * 24 + 3, 96) and names["l0.mix.right.conv"].shape == (48 + 144, 4)
    assert names["l1.mix.q.conv"].shape == (48, 3) and names["l1.mix.g"].shape == (160, 96) and names["l1.mix.norm"].shape == (40,)
    assert "l1.norm2" not in names and "l2.norm2" in names and names["final.norm"].shape == (96,) and names["head"].shape == (211, 96)
    kv, state, source = model.cache_needs()
    # the pair layer has two entries (attention, then Mamba-2); the others one each
    assert kv == [KVNeed(2, 32, None, 24), None, None, None] and source == [None] * 4
    assert state[0] == [] and state[1] == [StateNeed((3, 16, 24)), StateNeed((3, 192))]
    assert state[2] == [StateNeed((4, 40, 24)), StateNeed((2, 2 * 48 + 160))]
    assert state[3] == [StateNeed((4, 40, 72)), StateNeed((1, 160 + 288))]
    cache = model.new_cache(4, 2, device=None)
    assert len(cache.kv_groups) == 1 and len(cache.state_groups) == 6

    arch, config = load_config(CONFIGS["s"])
    kv, _, _ = DecoderModel(arch.describe(config), torch.float32, None).cache_needs()
    assert kv == [KVNeed(3, 16, None, None), None, KVNeed(1, 20, None, 36), None]      # two groups with tables of their own


def test_a_pre_norm_layer_needs_both_or_neither_of_its_feed_forward_parts():
    from thintensor_b200.config import load_config
    from thintensor_b200.engine.model import DecoderModel
    from dataclasses import replace

    arch, config = load_config(CONFIGS["r"])
    spec = arch.describe(config)
    parts = dict(spec.layers[1].parts)
    del parts["ffn_norm"]
    with pytest.raises(ValueError, match="feed-forward"):
        DecoderModel(replace(spec, layers=(spec.layers[0], replace(spec.layers[1], parts=parts), spec.layers[2])), torch.float32, None)
