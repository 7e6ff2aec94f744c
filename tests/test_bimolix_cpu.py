"""Bimolix without a GPU: configuration, spec, tensor names, cache and state bookkeeping, the oracle's own parts."""

import json
import math

import pytest
import torch

import plain_bimolix as plain
from bimolix_configs import BIMOLIX_CONFIGS, BIMOLIX_SEEDS, tensors_of
from tinyvllm_b200.config.registry import ConfigError, parse_model_config
from tinyvllm_b200.engine.model import Model
from tinyvllm_b200.models import BimolixConfig
from tinyvllm_b200.parts.attention import distance_buckets
from tinyvllm_b200.parts.base import KVNeed, StateNeed


@pytest.mark.parametrize("name", sorted(BIMOLIX_CONFIGS))
def test_config_round_trip_and_registry(name):
    config = BIMOLIX_CONFIGS[name]
    data = json.loads(json.dumps(config.to_json()))
    assert data["architecture"] == "Bimolix"
    again = parse_model_config(data)
    assert isinstance(again, BimolixConfig) and again.to_json() == data
    assert [layer.weights_of for layer in again.layers] == [layer.weights_of for layer in config.layers]
    # a layer that names another's weights repeats that layer's entry
    for index, layer in enumerate(data["layers"]):
        if "weights_of" in layer:
            owner = data["layers"][again.owner(index)]
            assert {k: v for k, v in layer.items() if k != "weights_of"} == {k: v for k, v in owner.items() if k != "weights_of"}


def test_config_refusals():
    good = BIMOLIX_CONFIGS["a"].to_json()
    for change in (lambda d: d.pop("norm"), lambda d: d.pop("vocab"),
                   lambda d: d["layers"][0].update(type="conv"),
                   lambda d: d["layers"][0]["mixer"].pop("decay"),
                   lambda d: d["layers"][0]["mixer"].update(decay=[0.5]),
                   lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7),
                   lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18),
                   lambda d: d["layers"][1]["mixer"].pop("kv_heads"),
                   lambda d: d["layers"][1]["mixer"].update(kv_heads=3),
                   lambda d: d["layers"][1]["mixer"].update(vdim=8),
                   lambda d: d["layers"][1]["mixer"].pop("bias_max"),
                   lambda d: d["layers"][1]["mlp"].update(kind="sparse"),
                   lambda d: d["layers"][1]["mlp"]["router"].update(top=9),
                   lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=3),
                   lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(keep=5),
                   lambda d: d["layers"][2].update(weights_of=1),
                   lambda d: d["layers"][2].update(weights_of=2)):
        data = json.loads(json.dumps(good))
        change(data)
        with pytest.raises(ConfigError):
            parse_model_config(data)


@pytest.mark.parametrize("name", sorted(BIMOLIX_CONFIGS))
def test_the_model_declares_exactly_the_checkpoint_tensors(name):
    config = BIMOLIX_CONFIGS[name]
    model = Model(config.to_spec(), device="cpu", dtype=torch.float32)
    declared = {}
    for _, spec in model.param_targets():
        assert not spec.optional
        for source in spec.sources:
            declared[source.name] = declared.get(source.name, 0) + 1
    tensors = tensors_of(config, BIMOLIX_SEEDS[name])
    assert set(declared) == set(tensors)
    assert all(count == 1 for count in declared.values())
    # layers that run another layer's weights own none
    for index, layer in enumerate(config.layers):
        assert any(n.startswith(f"l{index}.") for n in tensors) == (layer.weights_of is None)


@pytest.mark.parametrize("name", sorted(BIMOLIX_CONFIGS))
def test_every_layer_run_has_a_cache_or_state_of_its_own(name):
    """Attention runs need pages for keys and values, retention runs a float32 state a request; a layer
    that runs another's weights shares the parts and nothing of the memory."""
    config = BIMOLIX_CONFIGS[name]
    spec = config.to_spec()
    assert len(spec.order) == len(config.layers)
    assert len(spec.layers) == sum(layer.weights_of is None for layer in config.layers)
    model = Model(spec, device="cpu", dtype=torch.float32)
    needs = model.cache_needs()
    assert len(needs) == len(config.layers)
    for layer, need in zip(config.layers, needs):
        if layer.type == "retention":
            assert isinstance(need, StateNeed) and need.dtype == torch.float32
            assert tuple(need.shape) == (layer.heads, layer.dim, layer.vdim)
        else:
            assert isinstance(need, KVNeed)
            assert (need.num_kv_heads, need.head_dim, need.value_size) == (layer.kv_heads, layer.dim, layer.vdim)
            assert need.window is None          # a chunk's keys stay: a later query of the chunk reads them
    for index, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            assert spec.order[index].layer == spec.order[config.owner(index)].layer


@pytest.mark.parametrize("rows,far", [(2, 3.0), (5, 11.0), (6, 9.0), (12, 40.0), (32, 128.0), (32, 600.0), (9, 20.0)])
def test_distance_buckets(rows, far):
    """The table the kernels index by distance: the distance itself below half the rows, logarithmic steps
    that never go back, the last row from ``far`` on."""
    buckets = distance_buckets(rows, far)
    assert len(buckets) == math.ceil(far) + 1
    assert buckets == [plain.distance_bucket(n, rows, far) for n in range(len(buckets))]
    half = rows // 2
    assert buckets[:half] == list(range(half))
    assert all(a <= b for a, b in zip(buckets, buckets[1:]))
    assert buckets[half] == half and buckets[-1] == rows - 1
    assert all(plain.distance_bucket(n, rows, far) == rows - 1 for n in (math.ceil(far), 2 * math.ceil(far), 10 ** 6))


def test_the_oracle_routes_by_groups_and_weights_without_the_correction():
    router = {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([2.0, 0.0, 0.5, 0.4, -3.0, 1.9], dtype=torch.float64)
    none = torch.zeros(6, dtype=torch.float64)
    # group sums of the two members: (0, 1) wins over (2, 3) and (4, 5)
    chosen, weights = plain.route(z, none, router)
    assert chosen == [0, 1]
    s = torch.sigmoid(z)
    assert float(weights[0]) == pytest.approx(float(s[0] / (s[0] + s[1]) * 3.0))
    # a correction moves the choice to the last group, with negative choice scores in the others; the
    # weights are still made of the plain scores
    correction = torch.tensor([-2.0, -2.0, -2.0, -2.0, 0.0, 0.0], dtype=torch.float64)
    chosen, weights = plain.route(z, correction, router)
    assert chosen == [5, 4]
    assert float(sum(weights)) == pytest.approx(3.0)
    assert float(weights[1]) == pytest.approx(float(s[4] / (s[4] + s[5]) * 3.0))
    # all groups kept: the best two of all
    chosen, _ = plain.route(z, none, {**router, "groups": {"count": 3, "keep": 3}})
    assert chosen == [0, 5]
    # experts of groups that are not kept are out even when fewer than ``top`` remain in front of them
    chosen, _ = plain.route(z, torch.tensor([0.0, -5.0, 0, 0, 0, 0], dtype=torch.float64), {**router, "top": 2})
    assert set(chosen) <= {0, 1} or set(chosen) <= {2, 3} or set(chosen) <= {4, 5}


def test_the_oracle_retention_carries_its_state():
    """Tokens in two calls, the second from the first's state and position: the same as one call."""
    g = torch.Generator().manual_seed(3)
    mixer = {"heads": 2, "dim": 6, "vdim": 4, "decay": [0.9, 0.5], "rot": {"dims": 4, "base": 100.0}}
    w = {"m." + n: torch.randn(rows, 10, generator=g, dtype=torch.float64)
         for n, rows in (("q", 12), ("k", 12), ("v", 8), ("g", 8))}
    w["m.o"] = torch.randn(10, 8, generator=g, dtype=torch.float64)
    h = torch.randn(9, 10, generator=g, dtype=torch.float64)
    whole, state = plain.retention(h, w, "m", mixer, 1e-6)
    first, s = plain.retention(h[:4], w, "m", mixer, 1e-6)
    second, s = plain.retention(h[4:], w, "m", mixer, 1e-6, state=s, start=4)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-12)
    assert torch.allclose(s, state, atol=1e-12)


def test_the_oracle_sees_only_its_own_chunk_and_one_more_term():
    seen = plain.chunk_mask(7, 3)
    assert seen.tolist() == [[j <= i and i // 3 == j // 3 for j in range(7)] for i in range(7)]
    assert plain.chunk_mask(4, None).tolist() == [[j <= i for j in range(4)] for i in range(4)]
    scores = torch.zeros(7, 7, dtype=torch.float64)
    weights = plain.softmax_with_one_more(scores, seen)
    # position 3 begins a chunk: itself and the extra term share the denominator
    assert weights[3].tolist() == [0, 0, 0, 0.5, 0, 0, 0]
    assert weights[5, 3:6].tolist() == [0.25, 0.25, 0.25]


@pytest.mark.parametrize("name", sorted(BIMOLIX_CONFIGS))
def test_a_table_takes_its_rows_from_the_checkpoint(name, tmp_path):
    """config.json does not say how many rows a distance table has: a model built from it alone loads
    tables of any number of rows, also where ``bias_max`` lies inside the linear half of the rows that
    random weights would get."""
    from bimolix_configs import write_folder
    from tinyvllm_b200 import read_model_config

    config = BIMOLIX_CONFIGS[name]
    folder = write_folder(tmp_path / name, config, BIMOLIX_SEEDS[name])
    model = Model(read_model_config(folder).to_spec(), device="cpu", dtype=torch.float32).load(folder)
    tensors = tensors_of(config, BIMOLIX_SEEDS[name])
    seen = 0
    for index, layer in enumerate(config.layers):
        if layer.type != "attention" or layer.weights_of is not None:
            continue
        mixer = model.blocks[model.spec.order[index].layer].mixer
        rel = tensors[f"l{index}.mix.rel"].to(torch.bfloat16).float()
        assert mixer.rel.shape == rel.shape
        table = mixer.bias_table
        assert table.shape == (math.ceil(layer.bias_max) + 1, layer.heads)
        for distance in (0, 1, rel.shape[0] // 2, int(layer.bias_max) - 1, math.ceil(layer.bias_max)):
            if 0 <= distance < table.shape[0]:
                assert torch.equal(table[distance], rel[plain.distance_bucket(distance, rel.shape[0], layer.bias_max)])
        seen += 1
    assert seen
