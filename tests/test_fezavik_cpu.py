"""Fezavik without a GPU: configuration, spec, tensor names, cache and state bookkeeping, the oracle's own parts."""

import json
import math

import pytest
import torch

import plain_fezavik as plain
from fezavik_configs import FEZAVIK_CONFIGS, FEZAVIK_SEEDS, tensors_of
from tinyvllm_b200.config.registry import ConfigError, parse_model_config
from tinyvllm_b200.engine.model import Model
from tinyvllm_b200.models import FezavikConfig
from tinyvllm_b200.parts.base import BuildContext, KVNeed, StateNeed
from tinyvllm_b200.parts.rope import RopeHalfSplitComputed, RopeInterleaved


@pytest.mark.parametrize("name", sorted(FEZAVIK_CONFIGS))
def test_config_round_trip_and_registry(name):
    config = FEZAVIK_CONFIGS[name]
    data = json.loads(json.dumps(config.to_json()))
    assert data["architecture"] == "Fezavik"
    again = parse_model_config(data)
    assert isinstance(again, FezavikConfig) and again == config and again.to_json() == data


def test_config_refusals():
    good = FEZAVIK_CONFIGS["a"].to_json()
    for change in (lambda d: d.pop("norm"), lambda d: d.pop("width"),
                   lambda d: d["layers"][0].update(type="conv"),
                   lambda d: d["layers"][0]["mixer"].pop("kv_heads"),
                   lambda d: d["layers"][0]["mixer"].update(kv_heads=3),
                   lambda d: d["layers"][0]["mixer"].pop("scale"),
                   lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7),
                   lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18),
                   lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("low"),
                   lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].update(high=0.5),
                   lambda d: d["layers"][0]["mixer"]["mask"].update(size=0),
                   lambda d: d["layers"][1]["mixer"].pop("vdim"),
                   lambda d: d["layers"][2]["mixer"].pop("kv_rank"),
                   lambda d: d["layers"][2]["mixer"].update(rot_dim=8),
                   lambda d: d["layers"][2]["mixer"].pop("rot"),
                   lambda d: d["layers"][1]["mlp"].update(kind="dense"),
                   lambda d: d["layers"][1]["mlp"]["router"].update(top=11),
                   lambda d: d["layers"][1]["mlp"]["router"].update(identity=-1)):
        data = json.loads(json.dumps(good))
        change(data)
        with pytest.raises(ConfigError):
            parse_model_config(data)


@pytest.mark.parametrize("name", sorted(FEZAVIK_CONFIGS))
def test_the_model_declares_exactly_the_checkpoint_tensors(name):
    config = FEZAVIK_CONFIGS[name]
    model = Model(config.to_spec(), device="cpu", dtype=torch.float32)
    declared, shapes = {}, {}
    for _, spec in model.param_targets():
        assert not spec.optional
        for source in spec.sources:
            declared[source.name] = declared.get(source.name, 0) + 1
            shapes[source.name] = (source.rows,) + (tuple(spec.shape[1:]) if source.cols is None else (source.cols,))
    tensors = tensors_of(config, FEZAVIK_SEEDS[name])
    assert set(declared) == set(tensors)
    assert all(count == 1 for count in declared.values())
    assert all(tuple(tensors[n].shape) == shapes[n] for n in tensors)
    # a layer without a feed-forward owns neither the feed-forward's norms nor a router
    for index, layer in enumerate(config.layers):
        assert any(n.startswith(f"l{index}.norm2") for n in tensors) == (layer.mlp is not None)


@pytest.mark.parametrize("name", sorted(FEZAVIK_CONFIGS))
def test_every_layer_has_pages_or_a_state(name):
    """Attention layers need pages for keys and values with their window, latent layers one row a token whose
    first elements are the values, recurrent layers a float32 state a request."""
    config = FEZAVIK_CONFIGS[name]
    needs = Model(config.to_spec(), device="cpu", dtype=torch.bfloat16).cache_needs()
    assert len(needs) == len(config.layers)
    for layer, need in zip(config.layers, needs):
        if layer.type == "attention":
            assert need == KVNeed(layer.kv_heads, layer.dim, layer.window, layer.vdim, 0)
        elif layer.type == "latent_attention":
            assert need == KVNeed(1, layer.kv_rank + layer.rot_dim, layer.window, layer.kv_rank, 0, value_offset=0)
        else:
            assert need == StateNeed((layer.heads, layer.dim, layer.vdim), torch.float32)


@pytest.mark.parametrize("kind", [RopeInterleaved, RopeHalfSplitComputed])
@pytest.mark.parametrize("rot", [
    {"dims": 8, "base": 100.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}},
    {"dims": 32, "base": 10000.0, "scaling": {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 128.0}},
    {"dims": 64, "base": 300000.0, "scaling": {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 8192.0}},
    {"dims": 6, "base": 40.0}])
def test_slowed_waves_by_wavelength(rot, kind):
    """The position part's frequencies are the plain implementation's; where waves are slowed, pairs of all three
    bands occur (kept, blended, slowed by the whole factor)."""
    part = kind(BuildContext(torch.device("cpu"), torch.float32), dims=rot["dims"], base=rot["base"],
                scaling=rot.get("scaling"))
    got = part.inverse_frequencies().double()
    want = plain.frequencies(rot, torch.float64)
    assert torch.allclose(got, want, rtol=1e-6, atol=0)
    assert part.magnitude == 1.0
    if "scaling" in rot:
        plainly = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
        ratio = want / plainly
        factor = rot["scaling"]["factor"]
        assert (ratio == 1.0).any() and torch.isclose(ratio, torch.tensor(1.0 / factor, dtype=torch.float64)).any()
        assert ((ratio < 1.0 - 1e-9) & (ratio > 1.0 / factor + 1e-9)).any()


def test_the_oracles_window_and_sink():
    seen = plain.window_mask(6, 3)
    assert seen.tolist() == [[j <= i and i - j < 3 for j in range(6)] for i in range(6)]
    assert plain.window_mask(4, None).tolist() == [[j <= i for j in range(4)] for i in range(4)]
    scores = torch.zeros(1, 4, 4, dtype=torch.float64)
    p = plain.softmax_with_sink(scores, plain.window_mask(4, 2), torch.tensor([math.log(2.0)], dtype=torch.float64))
    # query 0 sees one key of score 0 beside a sink worth two such keys; later queries two keys
    assert torch.allclose(p[0, 0], torch.tensor([1 / 3, 0, 0, 0], dtype=torch.float64))
    assert torch.allclose(p[0, 3], torch.tensor([0, 0, 1 / 4, 1 / 4], dtype=torch.float64))


def test_the_oracles_routing():
    z = torch.tensor([2.0, 1.0, 0.0, 1.5, -1.0], dtype=torch.float64)
    s = torch.softmax(z, -1)
    none = torch.zeros(5, dtype=torch.float64)
    assert [e for e, _ in plain.route(z, none, {"top": 2})] == [0, 3]
    # the correction changes the choice, not the weights, which are the scores as they are and do not sum to 1
    chosen = plain.route(z, torch.tensor([0.0, 0.0, 1.0, 0.0, 0.0], dtype=torch.float64), {"top": 2})
    assert [e for e, _ in chosen] == [2, 0]
    assert torch.allclose(torch.stack([w for _, w in chosen]), s[[2, 0]])
    # a pass-through slot hands the input on, times its weight
    w = {"m.router": torch.tensor([[0.0, 0.0], [5.0, 0.0]], dtype=torch.float64), "m.correction": torch.zeros(2, dtype=torch.float64),
         "m.e0.gate": torch.ones(3, 2, dtype=torch.float64), "m.e0.up": torch.ones(3, 2, dtype=torch.float64),
         "m.e0.down": torch.ones(2, 3, dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0]], dtype=torch.float64)
    out = plain.moe_ff(h, w, "m", {"router": {"experts": 1, "identity": 1, "top": 1}})
    assert torch.allclose(out, h * torch.softmax(torch.tensor([0.0, 5.0], dtype=torch.float64), -1)[1])


def test_the_oracles_recurrence_carries_its_state():
    g = torch.Generator().manual_seed(1)
    heads, dim, vdim, width = 2, 3, 4, 5
    w = {"m.q": torch.randn(heads * dim, width, generator=g, dtype=torch.float64),
         "m.f": torch.randn(heads * dim, width, generator=g, dtype=torch.float64),
         "m.f.b": torch.randn(heads * dim, generator=g, dtype=torch.float64),
         "m.lower": torch.rand(heads * dim, generator=g, dtype=torch.float64),
         "m.v": torch.randn(heads * vdim, width, generator=g, dtype=torch.float64),
         "m.norm": torch.ones(vdim, dtype=torch.float64), "m.o": torch.eye(heads * vdim, dtype=torch.float64)}
    mixer = {"heads": heads, "dim": dim, "vdim": vdim}
    h = torch.randn(9, width, generator=g, dtype=torch.float64)
    whole, last = plain.gated_recurrence(h, w, "m", mixer, 1e-6)
    first, state = plain.gated_recurrence(h[:4], w, "m", mixer, 1e-6)
    second, again = plain.gated_recurrence(h[4:], w, "m", mixer, 1e-6, state=state)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(again, last)
    gates = plain.forget_gates(h, w, "m")
    assert (gates >= w["m.lower"]).all() and (gates <= 1.0).all()
