"""Dikusun without a GPU: configuration, refusals, schedule, cache needs, declared tensors, and properties of the plain
implementation that the GPU tests lean on."""
import copy

import pytest
import torch

import plain_dikusun as plain
from dikusun_configs import ALL_KINDS, DIKUSUN, GLA_ONLY


def _spec(raw):
    import llmserver_b200.models  # noqa: F401
    from llmserver_b200.config import DikusunConfig
    from llmserver_b200.config.registry import architecture_of
    config = DikusunConfig.from_dict(raw)
    return config, architecture_of(raw).build_spec(config)


@pytest.mark.parametrize("name", sorted(DIKUSUN))
def test_configuration_round_trips(name):
    from llmserver_b200.config import DikusunConfig
    raw = DIKUSUN[name][0]
    config = DikusunConfig.from_dict(raw)
    assert DikusunConfig.from_dict(config.to_dict()) == config
    assert config.vocab_size == raw["vocab"] and config.hidden_size == raw["width"]


def test_refusals():
    from llmserver_b200.config import DikusunConfig, UnsupportedModelError
    def broken(change):
        raw = copy.deepcopy(ALL_KINDS)
        change(raw)
        with pytest.raises(UnsupportedModelError):
            DikusunConfig.from_dict(raw)
    broken(lambda raw: raw["layers"][1].update(type="convolution"))
    broken(lambda raw: raw["layers"][1]["mixer"].update(kv_heads=3))
    broken(lambda raw: raw["layers"][1]["mixer"]["rot"].update(dims=18))
    broken(lambda raw: raw["layers"][1]["mixer"].pop("diff"))
    broken(lambda raw: raw["layers"][2]["mixer"].pop("kv_rank"))
    broken(lambda raw: raw["layers"][3]["mixer"].update(tau=0.0))
    broken(lambda raw: raw["layers"][3]["mlp"].update(kind="moe"))
    broken(lambda raw: raw["layers"][4].update(weights_of=4))
    broken(lambda raw: raw["layers"][4].update(weights_of=5))       # layer 5 has no weights of its own
    broken(lambda raw: raw["layers"][4].update(weights_of=2))       # another kind of layer
    broken(lambda raw: raw.pop("norm"))


def test_layers_that_use_another_layers_weights_are_schedule_entries_of_it():
    config, spec = _spec(ALL_KINDS)
    assert [layer.prefix for layer in spec.layers] == ["l1.", "l2.", "l3."]
    assert [entry.layer for entry in spec.schedule] == [2, 0, 1, 2, 0, 0]
    assert all(entry.cache_from is None for entry in spec.schedule)      # each run keeps a cache or state of its own
    assert spec.embedding_scale == 0.7


def test_cache_needs_and_declared_tensors():
    from llmserver_b200.cache import CacheManager, KVPagesNeed, StateNeed
    from llmserver_b200.parts import BLOCKS, MIXERS
    from llmserver_b200.weights.declare import declared_weights
    config, spec = _spec(ALL_KINDS)
    needs = []
    for entry in spec.schedule:
        layer = spec.layers[entry.layer]
        mixer = layer.part(BLOCKS.get(layer.block.kind).mixer_role(layer.block.as_dict()))
        needs.append(MIXERS.get(mixer.kind).cache_need(mixer.as_dict()))
    assert needs[0] == StateNeed((3, 16, 32), "float32") and needs[3] == needs[0]
    assert needs[1] == KVPagesNeed(2, 32, 23, 16) and needs[4] == needs[5] == needs[1]     # both maps in one key row
    assert needs[2] == KVPagesNeed(1, 56, None, None, keys_only=True)
    cache = CacheManager(needs, 8, 10, num_slots=2, prefix_sharing=True)
    assert len(cache.groups) == 2 and sorted(cache.state_entries) == [0, 3]
    assert [len(group.entries) for group in cache.groups] == [3, 1]
    assert not cache.prefix_sharing       # a window and a state both rule shared prefixes out
    names = declared_weights(spec)
    assert not any(name.startswith(("l0.", "l4.", "l5.")) for name in names)
    assert names["l1.mix.q"].shape == (4 * 2 * 16, 96) and names["l1.mix.k"].shape == (2 * 2 * 16, 96)
    assert names["l1.mix.g"].shape == (4, 96) and names["l1.mix.o.b"].shape == (96,) and names["l1.mix.lq2"].shape == (16,)
    assert names["l2.mix.uk"].shape == (2 * 32, 56) and names["l2.mix.dq.norm"].shape == (40,)
    assert names["l3.mix.a1"].shape == (12, 96) and names["l3.mix.a2.b"].shape == (3 * 16,)
    assert "l2.norm2" not in names and "l3.norm2" in names and names["final.norm"].shape == (96,)


def test_a_decay_rank_the_configuration_does_not_name_is_taken_from_the_tensor():
    from llmserver_b200.weights.declare import declared_weights
    from llmserver_b200.weights.loader import shape_fits
    raw = copy.deepcopy(GLA_ONLY)
    for layer in raw["layers"]:
        del layer["mixer"]["a_rank"]
    _, spec = _spec(raw)
    names = declared_weights(spec)
    assert names["l0.mix.a1"].shape == (-1, 40) and names["l0.mix.a2"].shape == (48, -1)
    assert shape_fits((7, 40), names["l0.mix.a1"].shape) and not shape_fits((7, 41), names["l0.mix.a1"].shape)


# ------------------------------------------------------------------------------------------------ the plain implementation
def _random_weights(raw, seed):
    from llmserver_b200.weights.declare import declared_weights
    from llmserver_b200.weights.random_init import random_tensor
    _, spec = _spec(raw)
    return {name: random_tensor(name, declaration, seed).to(torch.float64) for name, declaration in declared_weights(spec).items()}


def test_plain_gla_state_carries_over_portions():
    raw = GLA_ONLY
    weights = _random_weights(raw, 1)
    h = torch.randn((19, raw["width"]), dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    mixer = raw["layers"][0]["mixer"]
    whole, last = plain.gla_mixer(h, mixer, weights, "l0.mix.", 1e-5)
    first, state = plain.gla_mixer(h[:7], mixer, weights, "l0.mix.", 1e-5)
    second, end = plain.gla_mixer(h[7:], mixer, weights, "l0.mix.", 1e-5, state=state)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-12) and torch.allclose(end, last, atol=1e-12)
    alpha = plain.gla_decay(h, mixer, weights, "l0.mix.")
    assert alpha.shape == (19, 2, 24) and bool(((alpha > 0) & (alpha < 1)).all())


def test_plain_window_and_latent_identity():
    positions = torch.arange(9)
    seen = plain.visible(positions, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True, False, False, False]
    assert plain.visible(positions)[5].tolist() == [True] * 6 + [False] * 3
    # attention through the cached latent alone equals attention over keys and values made from it
    raw = DIKUSUN["latent_only"][0]
    weights = _random_weights(raw, 3)
    mixer = raw["layers"][0]["mixer"]
    h = torch.randn((11, raw["width"]), dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    want = plain.latent_attention_mixer(h, torch.arange(11), mixer, weights, "l0.mix.", 1e-6)
    heads, dim, vdim, rank = mixer["heads"], mixer["dim"], mixer["vdim"], mixer["kv_rank"]
    c = plain.latent_of(h, weights, "l0.mix.", 1e-6)
    c_q = plain.rms_norm(h @ weights["l0.mix.dq"].T, weights["l0.mix.dq.norm"], 1e-6)
    q = (c_q @ weights["l0.mix.uq"].T).view(11, heads, dim)
    q_latent = torch.einsum("thd,hdr->thr", q, weights["l0.mix.uk"].view(heads, dim, rank))
    out = torch.zeros(11, heads, vdim, dtype=torch.float64)
    for head in range(heads):
        p = plain.softmax_rows(q_latent[:, head] @ c.T * mixer["scale"], plain.visible(torch.arange(11)))
        out[:, head] = (p @ c) @ weights["l0.mix.uv"].view(heads, vdim, rank)[head].T
    assert torch.allclose(out.reshape(11, -1) @ weights["l0.mix.o"].T, want, atol=1e-10)


def test_plain_forward_runs_every_configuration():
    for name, (raw, seed) in DIKUSUN.items():
        weights = _random_weights(raw, seed)
        tokens = [(7 * i + 3) % raw["vocab"] for i in range(13)]
        logits, streams = plain.forward(raw, weights, tokens, return_layers=True)
        assert logits.shape == (13, raw["vocab"]) and streams.shape == (len(raw["layers"]), 13, raw["width"])
        assert bool(torch.isfinite(logits).all())
        # causal: a later token changes no earlier row
        changed = plain.forward(raw, weights, tokens[:-1] + [(tokens[-1] + 1) % raw["vocab"]])
        assert torch.allclose(changed[:-1], logits[:-1], atol=1e-12) and not torch.allclose(changed[-1], logits[-1], atol=1e-9)
