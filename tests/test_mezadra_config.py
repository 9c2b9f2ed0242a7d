"""Mezadra's configuration on the CPU: parts and their parameters, expected tensors, refusals, and that every
mechanism of the plain implementation moves the logits of the test models (so a comparison with it has teeth)."""

from __future__ import annotations

import copy
import math

import pytest
import torch
from mezadra_models import CONFIGS, as_double, attention_layer, dense, make_config, make_weights, tensor_shapes
from plain_mezadra import forward

from rapid_llm_b200.config import MezadraConfig, resolve_architecture
from rapid_llm_b200.models.causal_lm import CausalLM


def test_the_registry_finds_the_architecture():
    assert resolve_architecture({"architecture": "Mezadra"}) is MezadraConfig


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_model_expects_the_files_tensors(name):
    config = CONFIGS[name]
    model = CausalLM(MezadraConfig.from_dict(config).to_spec(), torch.float32, "cpu")
    assert {n: tuple(s.shape) for n, s in model.tensor_specs().items()} == tensor_shapes(config)


def test_parts_and_their_parameters():
    spec = MezadraConfig.from_dict(CONFIGS["blend"]).to_spec()
    assert [layer.arrangement for layer in spec.layers] == ["outnorm"] * 5
    assert [layer.mixer.kind for layer in spec.layers] == ["gqa_attention", "lightning", "gqa_attention", "gqa_attention", "gqa_attention"]
    assert [layer.mixer.params.get("value_mix") for layer in spec.layers] == ["first", None, "later", None, "later"]
    assert [None if layer.feed_forward is None else layer.feed_forward.kind for layer in spec.layers] == [
        "routed_experts", None, "clamped_glu", None, "routed_experts"]
    first = spec.layers[0].mixer.params
    assert (first["conv_width"], first["softcap"], first["sink"], first["unit_after_rotation"]) == (2, 6.0, True, True)
    assert first["position"].params["rotary_dim"] == 48 and spec.layers[2].mixer.params["position"].params["rotary_dim"] == 0
    last = spec.layers[4].feed_forward.params
    assert (last["num_experts"], last["top_k"], last["expert_size"], last["shared_size"], last["shared_gate"]) == (4, 4, 8, 8, True)
    assert spec.layers[0].feed_forward.params["shared_size"] is None
    assert spec.embedding.params["scale"] == 3.0 and spec.embedding.params["opens_stream"]
    model = CausalLM(spec, torch.float32, "cpu")
    assert [need is not None for need in model.cache_needs()] == [True, False, True, True, True]
    # state: the convolution's tail (none for one tap), the recurrence's matrix
    assert [None if need is None else need.shape[0] for need in model.state_needs()] == [
        1 * (2 + 2) * 64, 3 * 16 * 24, None, 3 * (4 + 8) * 16, 4 * (1 + 2) * 64]


def test_refusals():
    config = copy.deepcopy(CONFIGS["attention"])
    config["layers"][0]["type"] = "window"
    with pytest.raises(ValueError, match="unknown mixer type"):
        MezadraConfig.from_dict(config)
    config = copy.deepcopy(CONFIGS["attention"])
    config["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(ValueError, match="unknown feed-forward kind"):
        MezadraConfig.from_dict(config)
    config = make_config([attention_layer(v_mix=True, mlp=dense()), attention_layer(v_mix=True, vdim=32, mlp=None)])
    with pytest.raises(ValueError, match="blend"):
        MezadraConfig.from_dict(config)
    config = copy.deepcopy(CONFIGS["lightning"])
    del config["width"]
    with pytest.raises(ValueError, match="width"):
        MezadraConfig.from_dict(config)


def test_every_mechanism_moves_the_logits():
    """Leaving one mechanism out of the plain implementation changes the logits by far more than the engine's bound."""
    config = CONFIGS["blend"]
    weights = as_double(make_weights(config, seed=11))
    tokens = torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(3)).tolist()
    reference = forward(config, weights, tokens)

    def moved(other_config=None, other_weights=None):
        logits = forward(other_config or config, other_weights or weights, tokens)
        return float((logits - reference).abs().max())

    def changed(path, value):
        other = copy.deepcopy(config)
        node = other
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        return other

    without_sink = {name: (value - 50.0 if name.endswith("sink") else value) for name, value in weights.items()}
    no_blend = {name: (value * 0 if name.endswith("vmix") else value) for name, value in weights.items()}
    flat_taps = dict(weights)
    for name, value in weights.items():
        if name.endswith(".conv"):
            flat_taps[name] = torch.zeros_like(value)
            flat_taps[name][:, -1] = value[:, -1]
    assert moved(other_weights=without_sink) > 0.05
    assert moved(other_weights=no_blend) > 0.05
    assert moved(other_weights=flat_taps) > 0.05
    assert moved(changed(("layers", 2, "mixer", "softcap"), 0.0)) > 0.02
    assert moved(changed(("layers", 0, "mixer", "rot", "dims"), 0)) > 0.05
    assert moved(changed(("layers", 2, "mlp", "limit"), 100.0)) > 0.02
    assert moved(changed(("embedding", "scale"), 1.0)) > 0.05
    assert moved(changed(("layers", 1, "mixer", "decay"), [0.5, 0.5, 0.5])) > 0.05
    assert math.isfinite(moved())
