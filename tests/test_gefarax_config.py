"""Gefarax without a GPU: its configuration, the model specification built from it, the tensors it declares, and a
few properties of the plain implementation the GPU tests compare against."""
import copy
import math

import pytest
import torch

import plain_gefarax as plain
from gefarax_configs import GEFARAX, LOOP_FROM_START, LOOP_IN_THE_MIDDLE, NO_LOOP

import llmserver_b200.models  # noqa: F401  (registers the architectures)
from llmserver_b200.cache import CacheManager
from llmserver_b200.config import GefaraxConfig, UnsupportedModelError, architecture_of
from llmserver_b200.parts import BLOCKS, MIXERS
from llmserver_b200.weights.declare import declared_weights


@pytest.mark.parametrize("name", sorted(GEFARAX))
def test_round_trip_and_registry(name):
    raw = GEFARAX[name][0]
    config = GefaraxConfig.from_dict(raw)
    assert GefaraxConfig.from_dict(config.to_dict()) == config
    architecture = architecture_of(raw)            # found through the singular "architecture" key
    assert architecture.config_class is GefaraxConfig
    architecture.build_spec(config).validate()


def test_layer_runs_and_schedule():
    config = GefaraxConfig.from_dict(LOOP_IN_THE_MIDDLE)
    assert config.layer_runs() == [(0, False), (1, False), (1, True), (1, True), (2, False)]
    spec = architecture_of(LOOP_IN_THE_MIDDLE).build_spec(config)
    assert [(entry.layer, entry.add_embedding, entry.cache_from) for entry in spec.schedule] == [
        (0, False, None), (1, False, None), (1, True, None), (1, True, None), (2, False, None)]
    assert GefaraxConfig.from_dict(LOOP_FROM_START).layer_runs() == [(0, False), (1, False), (0, True), (1, False), (2, False)]
    assert GefaraxConfig.from_dict(NO_LOOP).layer_runs() == [(0, False), (1, False)]
    once = copy.deepcopy(LOOP_FROM_START)
    once["loop"]["times"] = 1
    assert GefaraxConfig.from_dict(once).layer_runs() == [(0, False), (1, False), (2, False)]


def test_every_layer_run_has_a_cache_of_its_own():
    config = GefaraxConfig.from_dict(LOOP_FROM_START)
    spec = architecture_of(LOOP_FROM_START).build_spec(config)
    needs = []
    for entry in spec.schedule:
        layer = spec.layers[entry.layer]
        mixer = layer.part(BLOCKS.get(layer.block.kind).mixer_role(layer.block.as_dict()))
        needs.append(MIXERS.get(mixer.kind).cache_need(mixer.as_dict()))
    cache = CacheManager(needs, page_size=4, num_pages=8, num_slots=2)
    assert sum(len(group.entries) for group in cache.groups) == len(spec.schedule) == 5
    # layers 0 (twice) share a group, layer 1 (twice; keys and values of one size) another, layer 2 a third
    assert sorted(len(group.entries) for group in cache.groups) == [1, 2, 2]
    sizes = {(group.need.head_dim, group.need.value_dim) for group in cache.groups}
    assert sizes == {(32, 16), (16, None), (24, 40)}


def test_declared_tensors():
    config = GefaraxConfig.from_dict(LOOP_FROM_START)
    wanted = declared_weights(architecture_of(LOOP_FROM_START).build_spec(config))
    assert wanted["embed"].shape == (300, 64) and wanted["head"].shape == (300, 64) and wanted["final.norm"].shape == (64,)
    assert wanted["l0.mix.q"].shape == (128, 64) and wanted["l0.mix.k"].shape == (64, 64)
    assert wanted["l0.mix.v"].shape == (32, 64) and wanted["l0.mix.o"].shape == (64, 64) and wanted["l0.mix.sink"].shape == (4,)
    assert wanted["l2.mix.o"].shape == (64, 240)
    assert wanted["l0.mlp.e3.gate"].shape == (48, 64) and wanted["l0.mlp.e3.down"].shape == (64, 48)
    assert wanted["l0.mlp.router"].shape == (4, 64) and wanted["l0.mlp.correction"].shape == (4,)
    assert wanted["l0.mlp.shared.up"].shape == (32, 64) and "l2.mlp.shared.up" not in wanted
    assert "l1.mlp.router" not in wanted and "l1.norm2" not in wanted and "l1.norm1b" in wanted
    assert {"l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b"} <= set(wanted)


def test_refusals():
    for change, message in (
            (lambda raw: raw["layers"][0].__setitem__("type", "convolution"), "unknown mixer type"),
            (lambda raw: raw["layers"][0]["mixer"].__setitem__("kv_heads", 3), "no multiple"),
            (lambda raw: raw["layers"][0]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
            (lambda raw: raw["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top must lie"),
            (lambda raw: raw["layers"][0]["mlp"].__setitem__("kind", "dense"), "unknown kind"),
            (lambda raw: raw["loop"].__setitem__("stop", 7), "does not fit"),
            (lambda raw: raw.pop("width"), "lacks width")):
        raw = copy.deepcopy(LOOP_FROM_START)
        change(raw)
        with pytest.raises(UnsupportedModelError, match=message):
            GefaraxConfig.from_dict(raw)


# ------------------------------------------------------------------ the plain implementation itself
def _random_weights(raw, seed):
    config = GefaraxConfig.from_dict(raw)
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, declaration in declared_weights(architecture_of(raw).build_spec(config)).items():
        values = torch.randn(declaration.shape, generator=generator, dtype=torch.float64)
        weights[name] = 1.0 + 0.1 * values if declaration.kind == "norm" else 0.3 * values
    return weights


def test_plain_model_is_causal_and_loops():
    weights = _random_weights(LOOP_IN_THE_MIDDLE, 5)
    tokens = [3, 17, 150, 9, 9, 42, 77, 1, 0, 189, 5, 64]
    whole, layers = plain.forward(LOOP_IN_THE_MIDDLE, weights, tokens, keep_layers=True)
    assert layers.shape == (5, len(tokens), 48)
    prefix = plain.forward(LOOP_IN_THE_MIDDLE, weights, tokens[:7])
    assert torch.allclose(whole[:7], prefix, atol=1e-12)
    once = copy.deepcopy(LOOP_IN_THE_MIDDLE)
    once["loop"] = None
    assert not torch.allclose(plain.forward(once, weights, tokens), whole, atol=1e-3)


def test_plain_sink_and_rotation():
    # with one visible key the attention weight is 1 / (1 + exp(sink - score))
    mixer = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 2, "scale": 0.5, "rot": None}
    eye = torch.eye(4, dtype=torch.float64)
    weights = {"a.q": eye, "a.k": eye, "a.v": torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0]], dtype=torch.float64),
               "a.o": torch.eye(2, dtype=torch.float64), "a.sink": torch.tensor([0.7], dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0, 0.0, -1.0]], dtype=torch.float64)
    out = plain.attention_mixer(h, torch.arange(1), mixer, weights, "a.")
    score = 0.5 * float(h[0] @ h[0])
    assert torch.allclose(out, h[:, :2] / (1.0 + math.exp(0.7 - score)), atol=1e-12)
    # rotation: position 0 only scales by the magnitude; the part beyond rot.dims is untouched at any position
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 8.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    x = torch.arange(12, dtype=torch.float64).view(2, 1, 6) + 1.0
    turned = plain.rotate(x, torch.tensor([0, 5]), rot)
    magnitude = 0.1 * math.log(8.0) + 1.0
    assert torch.allclose(turned[0, 0, :4], x[0, 0, :4] * magnitude) and torch.equal(turned[:, :, 4:], x[:, :, 4:])
    assert torch.allclose(turned[1, 0, :4].norm(), x[1, 0, :4].norm() * magnitude)
