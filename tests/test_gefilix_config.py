"""The Gefilix configuration and model description, without a device: keys and rejections,
the tensor list against the plain implementation's, and what each layer asks of the cache."""

import copy

import pytest

import plain_gefilix as plain
from atomserve_b200.config import ModelConfigError
from atomserve_b200.config.registry import config_from_dict
from atomserve_b200.parts import build_model
from tiny_gefilix import GEFILIX, calm


@pytest.mark.parametrize("name", list(GEFILIX))
def test_round_trip_and_tensor_list(name):
    raw = GEFILIX[name][0]
    arch, config = config_from_dict(raw)
    assert arch.name == "Gefilix"
    assert config_from_dict(config.to_dict())[1] == config
    model = build_model(arch.build_spec(config))
    assert {s.name: tuple(s.shape) for s in model.tensor_specs()} == plain.tensor_shapes(raw)
    needs = model.cache_requirements()
    for layer, (pages, state) in zip(raw["layers"], needs):
        m = layer["mixer"]
        if layer["type"] == "lightning":
            assert pages is None and [s.shape for s in state] == [(m["heads"], m["dim"], m["vdim"])]
        elif m.get("kv_from") is None:
            assert not state and pages.values_per_token == m["kv_rank"] + m["rot_dim"]
        else:
            assert pages is None and not state
    for call, layer in zip(model.schedule, raw["layers"]):
        assert call.cache_from == layer["mixer"].get("kv_from")
    assert config_from_dict(calm(raw))[1] != config or name == "none"


def test_both_spellings_of_the_architecture_key():
    raw = copy.deepcopy(GEFILIX["b"][0])
    raw["architectures"] = [raw.pop("architecture")]
    assert config_from_dict(raw)[0].name == "Gefilix"


def broken(change):
    raw = copy.deepcopy(GEFILIX["a"][0])
    change(raw)
    return raw


@pytest.mark.parametrize("change", [
    lambda r: r.pop("postln_alpha"),
    lambda r: r["layers"][0]["mixer"].pop("decay"),
    lambda r: r["layers"][0]["mixer"]["decay"].append(0.5),
    lambda r: r["layers"][0].update(type="convolution"),
    lambda r: r["layers"][3]["mixer"].update(kv_from=3),
    lambda r: r["layers"][3]["mixer"].update(kv_from=0),
    lambda r: r["layers"][3]["mixer"].update(kv_rank=48),
    lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7),
    lambda r: r["layers"][1]["mlp"]["router"].update(experts=7),
    lambda r: r["layers"][1]["mlp"].update(kind="sparse"),
    lambda r: r["layers"][1]["mlp"]["expert"].pop("limit"),
])  # fmt: skip
def test_rejections(change):
    with pytest.raises(ModelConfigError):
        config_from_dict(broken(change))
