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


def test_segments_of_a_step():
    """Requests of 256 tokens and more are cut into segments of 64; shorter ones stay whole."""
    import torch

    from atomserve_b200.ops.recurrent import SEGMENT_FROM, SEGMENT_TOKENS, plan_segments

    assert plan_segments([1, SEGMENT_FROM - 1], torch.device("cpu")) is None
    lens = [300, 1, 5, SEGMENT_FROM]
    seg = plan_segments(lens, torch.device("cpu"))
    bounds, starts = seg.bounds.tolist(), seg.req_start.tolist()
    assert bounds[0] == 0 and bounds[-1] == sum(lens) and seg.count == len(bounds) - 1
    assert all(0 < b - a <= SEGMENT_TOKENS or (b - a) in lens for a, b in zip(bounds, bounds[1:]))
    row = 0
    for r, n in enumerate(lens):  # each request's segments tile its rows exactly
        assert bounds[starts[r]] == row and bounds[starts[r + 1]] == row + n
        row += n
    assert seg.index.tolist() == list(range(seg.count))


def test_state_buffers_have_a_row_that_belongs_to_no_request():
    import torch

    from atomserve_b200.cache.state_slots import StateSlots

    slots = StateSlots(3)
    buf = slots.register("s", (2, 2), torch.float32)
    assert buf.shape == (4, 2, 2) and slots.pad_slot == 3
    taken = [slots.take() for _ in range(3)]
    assert sorted(taken) == [0, 1, 2] and slots.num_free == 0
    buf[1] = 7.0
    slots.give_back(1)
    assert slots.take() == 1 and not buf[1].any()  # zeroed when handed out again
