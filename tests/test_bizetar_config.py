"""The Bizetar configuration: parsing, the layer specs it gives the generic decoder, the tensors
it expects, what every layer keeps per request, and the errors that name the key."""

import copy

import pytest

import bizetar_configs as bc
import plain_bizetar as pb
from distengine_b200.config import ConfigError
from distengine_b200.config.bizetar import BizetarConfig
from distengine_b200.models import expected_tensors
from distengine_b200.registry import resolve


def _same(a, b):
    """Equal but for keys that are absent on one side and empty on the other."""
    if isinstance(a, dict) and isinstance(b, dict):
        return all(_same(a.get(k), b.get(k)) for k in set(a) | set(b))
    if isinstance(a, list) and isinstance(b, list):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    empty = (None, False, 0)
    return a == b or (a in empty and b in empty)


@pytest.mark.parametrize("name", sorted(bc.ALL))
def test_round_trip_and_tensors(name):
    architecture, config = resolve(bc.ALL[name])
    assert architecture.name == "Bizetar" and isinstance(config, BizetarConfig)
    assert _same(config.to_json(), bc.ALL[name])
    assert BizetarConfig.from_json(config.to_json()) == config
    expected, vectors, optional = expected_tensors(config)
    assert {k: tuple(v) for k, v in expected.items()} == pb.tensor_shapes(bc.ALL[name])
    assert {"final.norm", "embed.norm", "l0.norm1", "l0.dwa"} <= vectors and not optional
    assert not config.tied_output and "head" in expected


def test_layer_specs_name_the_parts():
    specs = BizetarConfig.from_json(bc.BIZ_A).layer_specs()
    assert [s.block for s in specs] == ["sublayer_norm"] * 4
    assert [dict(s.block_params)["depth"] for s in specs] == [2, 3, 4, 5]
    assert all(s.mixer.kind == "sink_attention" for s in specs)
    assert [s.feed_forward.kind if s.feed_forward else None for s in specs] == [
        "routed_experts", "polynorm_mlp", None, "routed_experts"]
    # the first layer that mixes values gives them, the later ones take, one stays out
    assert [s.mixer.params["value_mix"] for s in specs] == ["give", "take", None, "take"]
    first, second = specs[0].mixer.params, specs[1].mixer.params
    assert first["norm"] == "whole" and first["gate"] == "head" and first["slopes"]
    assert first["temperature"] == (0.7, 4) and specs[3].mixer.params["temperature"] is None
    assert second["norm"] == "head" and second["gate"] == "feature" and second["biased"]
    assert second["taps"] == 2 and second["stretch"] == (4.0, 16.0, 8.0, 1.0)
    assert specs[2].mixer.params["stretch"] is None and specs[2].mixer.params["taps"] == 4
    routed = specs[0].feed_forward.params
    assert routed["identity"] == 2 and routed["gated"] and routed["scoring"] == "corrected_scores"


def test_what_a_layer_keeps():
    """Pages for every layer, and a state slot for the kept rows of a convolution of two taps or
    more."""
    from distengine_b200.models.decoder import DecoderModel
    from distengine_b200.parts.base import PagedKVSpec, StateSpec
    model = DecoderModel(BizetarConfig.from_json(bc.BIZ_A), "float32", "meta")
    specs = model.cache_specs()
    assert specs[0] == PagedKVSpec(2, 5, None, value_dim=3)
    assert specs[1] == (PagedKVSpec(2, 10, None, value_dim=3),
                        StateSpec(((6 + 2) * 10 + 2 * 3,)))
    assert specs[2][1] == StateSpec((3 * ((3 + 1) * 6 + 7),))
    assert model.history_depth == 5
    one_tap = DecoderModel(BizetarConfig.from_json(bc.BIZ_B), "float32", "meta").cache_specs()
    assert all(isinstance(s, PagedKVSpec) for s in one_tap)


def test_null_keys_of_the_other_form_and_unused_tensors(tmp_path):
    """A key of the other mixer form may stand with null; a weight file may hold the mixing
    weight of a layer outside the mixing and the second sublayer's tensors of a layer without a
    feed-forward - they are passed over, anything else unexpected is still reported."""
    import torch
    from distengine_b200.weights import save_tensors
    from distengine_b200.weights.loader import WeightMismatchError, load_checked
    config = copy.deepcopy(bc.BIZ_A)
    config["layers"][0]["mixer"].update(conv=None, rot=None)
    config["layers"][1]["mixer"].update(q_temp=None)
    parsed = BizetarConfig.from_json(config)
    assert parsed == BizetarConfig.from_json(bc.BIZ_A)
    assert parsed.unused_tensors() == {"l2.mix.vmix", "l2.norm2", "l2.rg2", "l2.rg2.b"}
    expected, _, optional = expected_tensors(parsed)
    tensors = {k: torch.zeros(v) for k, v in expected.items()}
    tensors.update({"l2.mix.vmix": torch.zeros(()), "l2.norm2": torch.zeros(42),
                    "l2.rg2": torch.zeros(42, 42), "l2.rg2.b": torch.zeros(42)})
    save_tensors(str(tmp_path / "model.safetensors"), tensors)
    loaded = load_checked(str(tmp_path), expected, optional, torch.float32,
                          unused=parsed.unused_tensors())
    assert set(loaded) == set(expected)
    with pytest.raises(WeightMismatchError) as error:
        load_checked(str(tmp_path), expected, optional, torch.float32)
    assert "l2.rg2.b" in str(error.value)
    tensors["l0.mix.q.b"] = torch.zeros(30)
    save_tensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightMismatchError) as error:
        load_checked(str(tmp_path), expected, optional, torch.float32,
                     unused=parsed.unused_tensors())
    assert "l0.mix.q.b" in str(error.value) and "l2.rg2" not in str(error.value)


def _broken(change):
    config = copy.deepcopy(bc.BIZ_A)
    change(config)
    return config


@pytest.mark.parametrize("change, key", [
    (lambda c: c["layers"][0].update(type="latent_attention"), "layers[0].type"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "layers[1].mixer.rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=12), "layers[1].mixer.rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "layers[1].mixer.vdim"),
    (lambda c: c["layers"][1]["mixer"].update(heads=5), "layers[1].mixer.heads"),
    (lambda c: c["layers"][1]["mixer"].update(conv=0), "layers[1].mixer.conv"),
    (lambda c: c["layers"][0]["mixer"].update(conv=3), "layers[0].mixer."),
    (lambda c: c["layers"][1]["mixer"].update(q_temp={"coef": 1.0, "every": 2}), "layers[1].mixer."),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "layers[0].mixer.q_temp.every"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "layers[0].mlp.router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "layers[0].mlp.kind"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0), "rot.scaling"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=4), "v_mix"),
    (lambda c: c["layers"][0]["mixer"].update(rot={"base": 10.0, "dims": 2}), "layers[0].mixer."),
    (lambda c: c["norm"].update(eps=0), "norm.eps"),
])
def test_errors_name_the_key(change, key):
    with pytest.raises(ConfigError) as error:
        BizetarConfig.from_json(_broken(change))
    assert key in str(error.value)
