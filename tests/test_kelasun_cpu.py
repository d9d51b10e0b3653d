"""Kelasun without a GPU: configuration, spec, tensor names, cache bookkeeping, the oracle's own parts."""

import json
import math

import pytest
import torch

import plain_kelasun as plain
from kelasun_configs import KELASUN_CONFIGS, KELASUN_SEEDS, tensors_of
from tinyvllm_b200.config.registry import ConfigError, parse_model_config
from tinyvllm_b200.engine.model import Model
from tinyvllm_b200.cache.storage import bytes_per_page, group_runs
from tinyvllm_b200.models import KelasunConfig
from tinyvllm_b200.parts.base import BuildContext, KVNeed
from tinyvllm_b200.parts.rope import RopeInterleaved


@pytest.mark.parametrize("name", sorted(KELASUN_CONFIGS))
def test_config_round_trip_and_registry(name):
    config = KELASUN_CONFIGS[name]
    data = json.loads(json.dumps(config.to_json()))
    assert data["architecture"] == "Kelasun"
    again = parse_model_config(data)
    assert isinstance(again, KelasunConfig) and again == config


def test_config_refusals():
    good = KELASUN_CONFIGS["a"].to_json()
    for change in (lambda d: d.pop("postln_alpha"), lambda d: d.pop("logit_scale"),
                   lambda d: d["layers"][0].update(type="conv"),
                   lambda d: d["layers"][0]["mixer"].pop("kv_heads"),
                   lambda d: d["layers"][0]["mixer"].update(heads=3),
                   lambda d: d["layers"][1]["mixer"].pop("kv_rank"),
                   lambda d: d["layers"][1]["mixer"]["rot"].update(dims=6),
                   lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"),
                   lambda d: d["layers"][0]["mlp"].update(kind="dense"),
                   lambda d: d["layers"][0]["mlp"]["router"].update(top=9)):
        data = json.loads(json.dumps(good))
        change(data)
        with pytest.raises(ConfigError):
            parse_model_config(data)


@pytest.mark.parametrize("name", sorted(KELASUN_CONFIGS))
def test_the_model_declares_exactly_the_checkpoint_tensors(name):
    config = KELASUN_CONFIGS[name]
    model = Model(config.to_spec(), device="cpu", dtype=torch.float32)
    declared, may_lack = {}, set()
    for _, spec in model.param_targets():
        for source in spec.sources:
            declared[source.name] = declared.get(source.name, 0) + 1
            if spec.optional:
                may_lack.add(source.name)
    tensors = tensors_of(config, KELASUN_SEEDS[name])
    assert set(declared) - may_lack == set(tensors)
    assert all(count == 1 for count in declared.values())
    # a layer without a feed-forward may hold a second norm all the same, and only such a layer
    assert may_lack == {f"l{i}.norm2" for i, layer in enumerate(config.layers) if layer.mlp is None}
    assert set(declared) == set(tensors_of(config, KELASUN_SEEDS[name], second_norms=True))


def test_a_tensor_a_part_declares_optional_may_be_absent():
    from tinyvllm_b200.parts.base import ParamSpec, Part
    from tinyvllm_b200.weights.loader import WeightsError, bind_tensors

    part = Part()
    targets = [(part, ParamSpec.single("a", "x.a", (3,), role="vector")),
               (part, ParamSpec.single("b", "x.b", (2,), role="vector", optional=True))]
    bind_tensors(targets, {"x.a": torch.ones(3)}, dtype=torch.float32, device="cpu")
    assert part.b is None and part.a.shape == (3,)
    bind_tensors(targets, {"x.a": torch.ones(3), "x.b": torch.zeros(2)}, dtype=torch.float32, device="cpu")
    assert part.b.shape == (2,)
    with pytest.raises(WeightsError):
        bind_tensors(targets, {"x.b": torch.zeros(2)}, dtype=torch.float32, device="cpu")


def test_cache_groups_hold_latents_once():
    """A latent layer caches one row [latent | rotated key part] a token and no values; the attention
    layers cache keys and values; layers of equal geometry share a group."""
    config = KELASUN_CONFIGS["a"]
    model = Model(config.to_spec(), device="cpu", dtype=torch.float32)
    needs = model.cache_needs()
    assert needs[1] == KVNeed(1, 32 + 8, None, 32, 0, value_offset=0)
    groups, where = group_runs(needs, model.cache_sources())
    assert len(groups) == 2 and where[0][0] == where[2][0] and where[1][0] == where[3][0]
    latent = groups[where[1][0]]
    assert bytes_per_page(latent, 16, 2) == 2 * 16 * (32 + 8) * 2          # two runs, no value pages
    plain_group = groups[where[0][0]]
    assert bytes_per_page(plain_group, 16, 2) == 2 * 16 * 2 * (16 + 32) * 2


def test_stretched_frequencies_follow_the_oracle():
    for rot in ({"dims": 8, "base": 10000.0, "scaling": {"factor": 8.0, "original": 64.0, "fast": 16.0, "slow": 2.0}},
                {"dims": 64, "base": 200000.0, "scaling": {"factor": 3.0, "original": 128.0, "fast": 16.0, "slow": 1.0}},
                {"dims": 4, "base": 500.0}):
        part = RopeInterleaved(BuildContext(torch.device("cpu"), torch.float32), dims=rot["dims"], base=rot["base"],
                               scaling=rot.get("scaling"))
        freqs, magnitude = plain.rotary_frequencies(rot)
        assert torch.allclose(part.inverse_frequencies().double(), torch.tensor(freqs, dtype=torch.float64), rtol=1e-6)
        assert part.magnitude == pytest.approx(magnitude)
    # the ramp really lies inside: the first pair keeps its frequency, the last is divided by the factor
    freqs, _ = plain.rotary_frequencies({"dims": 8, "base": 10000.0,
                                         "scaling": {"factor": 8.0, "original": 64.0, "fast": 16.0, "slow": 2.0}})
    assert freqs[0] == pytest.approx(1.0) and freqs[-1] == pytest.approx(10000.0 ** (-6 / 8) / 8.0)


def test_oracle_sink_and_causality():
    scores = torch.zeros(3, 3, dtype=torch.float64)
    weights = plain.causal_softmax_rows(scores, sink=0.0)
    assert torch.allclose(weights[2], torch.full((3,), 0.25, dtype=torch.float64))      # three keys and the sink
    assert weights[0, 1] == 0 and weights[0, 0] == pytest.approx(0.5)
    no_sink = plain.causal_softmax_rows(scores)
    assert no_sink[1, 0] == pytest.approx(0.5)


def test_oracle_routing_weights_are_a_softmax_over_the_chosen():
    h = torch.eye(4, dtype=torch.float64)[:1] * 2.0
    w = {"m.router": torch.tensor([[1.0, 0, 0, 0], [3.0, 0, 0, 0], [2.0, 0, 0, 0]], dtype=torch.float64),
         **{f"m.e{e}.up": torch.eye(4, dtype=torch.float64) for e in range(3)},
         **{f"m.e{e}.down": torch.eye(4, dtype=torch.float64) * (e + 1) for e in range(3)}}
    out = plain.routed_experts(h, w, "m", {"router": {"experts": 3, "top": 2}})
    share = math.exp(6.0) / (math.exp(6.0) + math.exp(4.0))
    assert out[0, 0].item() == pytest.approx(4.0 * (share * 2 + (1 - share) * 3))
