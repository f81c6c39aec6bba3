"""The Vapelix configuration: parsing, the layer specs and plan it gives the generic decoder, the
tensors it expects, and the errors that name the key."""

import copy

import pytest

import plain_vapelix as pv
import vapelix_configs as vc
from distengine_b200.config import ConfigError
from distengine_b200.config.vapelix import VapelixConfig
from distengine_b200.models import expected_tensors
from distengine_b200.registry import resolve


@pytest.mark.parametrize("name", sorted(vc.ALL))
def test_round_trip_and_tensors(name):
    architecture, config = resolve(vc.ALL[name])
    assert architecture.name == "Vapelix" and isinstance(config, VapelixConfig)
    assert config.to_json() == vc.ALL[name]
    assert VapelixConfig.from_json(config.to_json()) == config
    expected, vectors, optional = expected_tensors(config)
    assert {k: tuple(v) for k, v in expected.items()} == pv.tensor_shapes(vc.ALL[name])
    assert "final.norm" in vectors and "l0.norm1" in vectors and not optional
    assert config.tied_output


def test_the_plan_repeats_the_looped_layers():
    config = VapelixConfig.from_json(vc.VAP_A)
    plan = [(e.layer, e.adds_embedding) for e in config.plan()]
    assert plan == pv.run_order(vc.VAP_A)
    assert plan == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True),
                    (2, False), (3, False)]
    whole = VapelixConfig.from_json(vc.VAP_C)
    assert [(e.layer, e.adds_embedding) for e in whole.plan()] == [(0, False), (1, False),
                                                                   (0, True), (1, False)]
    assert [e.layer for e in VapelixConfig.from_json(vc.VAP_B).plan()] == [0, 1, 2]
    once = copy.deepcopy(vc.VAP_A)
    once["loop"]["times"] = 1
    assert [e.layer for e in VapelixConfig.from_json(once).plan()] == [0, 1, 2, 3]


def test_layer_specs_name_the_parts():
    specs = VapelixConfig.from_json(vc.VAP_A).layer_specs()
    assert [s.block for s in specs] == ["parallel_norms"] * 4
    assert [s.feed_forward.kind if s.feed_forward else None for s in specs] == [
        "routed_experts", "gated_mlp", None, "routed_experts"]
    assert all(s.side_input.kind == "token_side" for s in specs)
    assert specs[2].side_input.params["index"] == 2
    assert specs[1].mixer.params["scaling"] == (4.0, 64.0, 8.0, 1.0)
    assert specs[0].mixer.params["scaling"] is None
    assert all(s.side_input is None for s in VapelixConfig.from_json(vc.VAP_B).layer_specs())


def test_every_run_of_a_layer_has_a_cache_of_its_own():
    from distengine_b200.models.decoder import DecoderModel
    model = DecoderModel(VapelixConfig.from_json(vc.VAP_A), "float32", "meta")
    specs = model.cache_specs()
    assert len(specs) == 8 and all(s is not None for s in specs)
    assert specs[1] == specs[3] == specs[5] and specs[0] == specs[7] and specs[0] != specs[1]
    assert specs[1].values_in_keys and specs[1].head_dim == 24 and specs[1].v_dim == 18


def _broken(change):
    config = copy.deepcopy(vc.VAP_A)
    change(config)
    return config


@pytest.mark.parametrize("change, key", [
    (lambda c: c["layers"][0].update(type="attention"), "layers[0].type"),
    (lambda c: c["layers"][1]["mixer"].update(rot_dim=5), "layers[1].mixer.rot_dim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "layers[1].mixer.rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "layers[1].mixer.kv_rank"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "layers[0].mlp.router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "layers[0].mlp.kind"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0), "rot.scaling"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["norm"].update(eps=0), "norm.eps"),
    (lambda c: c["token_side"].update(dim=0), "token_side.dim"),
])
def test_errors_name_the_key(change, key):
    with pytest.raises(ConfigError) as error:
        VapelixConfig.from_json(_broken(change))
    assert key in str(error.value)
