"""The Zogepel configuration and model description on the CPU: keys, rejections, the round trip
through config.json, tensor names and shapes, what each layer keeps between steps."""

import copy

import pytest

import plain_zogepel as plain
from tiny_zogepel import ZOGEPEL


def parse(raw):
    from atomserve_b200.config.registry import config_from_dict

    return config_from_dict(raw)


@pytest.mark.parametrize("name", list(ZOGEPEL))
def test_round_trip_and_tensor_list(name):
    from atomserve_b200.parts.model import build_model

    raw = ZOGEPEL[name][0]
    arch, config = parse(raw)
    assert arch.name == "Zogepel"
    assert parse(config.to_dict())[1] == config
    assert ("token_side" in config.to_dict()) == ("token_side" in raw)
    model = build_model(arch.build_spec(config))
    got = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert got == plain.tensor_shapes(raw)
    kinds = {s.name: s.kind for s in model.tensor_specs()}
    assert all(kinds[n] == ("matrix" if len(shape) == 2 else "gain") for n, shape in got.items())


def test_what_layers_keep_between_steps():
    from atomserve_b200.parts.model import build_model

    raw = ZOGEPEL["a"][0]
    arch, config = parse(raw)
    needs = build_model(arch.build_spec(config)).cache_requirements()
    pages, state = needs[0]
    assert pages.window == 20 and [(t.name, t.heads, t.width) for t in pages.tensors] == [("k", 2, 24), ("v", 2, 24)]
    assert [(s.name, tuple(s.shape)) for s in state] == [("s", (3, 16, 40))]
    pages, state = needs[1]
    assert pages is None and [(s.name, tuple(s.shape)) for s in state] == [("s", (3, 24, 40)), ("n", (3, 24)), ("top", (3,))]
    assert needs[2][0].window == 7


def test_a_layer_without_feed_forward_ignores_its_second_norm():
    from atomserve_b200.weights.loader import check_names_and_shapes
    from atomserve_b200.parts.model import build_model

    raw = ZOGEPEL["a"][0]
    arch, config = parse(raw)
    spec = arch.build_spec(config)
    found = dict(plain.tensor_shapes(raw), **{"l1.norm2": (96,), "l1.ls2": (96,)})
    check_names_and_shapes(found, build_model(spec).tensor_specs(), spec.ignored_tensors)


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "not one of"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 4), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("vdim", 8), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decays"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].__setitem__("dims", 18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "dense"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["token_side"].pop("dim"), "dim"),
])  # fmt: skip
def test_rejections(change, text):
    from atomserve_b200.config.model_config import ModelConfigError

    raw = copy.deepcopy(ZOGEPEL["a"][0])
    change(raw)
    with pytest.raises(ModelConfigError, match=text):
        parse(raw)
