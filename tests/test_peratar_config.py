"""Peratar without a GPU: config.json parsing and its refusals, the spec's tensor names and
shapes, the random-weights folder, the cache's page cost, and the plain implementation's own
mechanisms."""
import copy
import json
import os

import pytest
import torch

import peratar_configs as pc
import plain_peratar as plain
from velox_b200.config.model_config import ConfigError, PeratarConfig
from velox_b200.config.registry import architecture_of, load_model_config


def test_architecture_is_found_by_either_key():
    assert architecture_of({"architecture": "Peratar"}).name == "Peratar"
    assert architecture_of({"architectures": ["Peratar"]}).name == "Peratar"
    with pytest.raises(ConfigError):
        architecture_of({"model": "x"})


@pytest.mark.parametrize("name", list(pc.ALL))
def test_config_round_trip(name):
    cfg = pc.ALL[name]
    typed = PeratarConfig.from_dict(cfg)
    assert typed.vocab_size == cfg["vocab"] and typed.hidden_size == cfg["width"]
    assert typed.num_hidden_layers == len(cfg["layers"])
    assert typed.logit_softcap == cfg["logit_softcap"] and typed.norm_eps == cfg["norm"]["eps"]
    for layer, raw in zip(typed.layers, cfg["layers"]):
        assert layer.ff == (None if raw["mlp"] is None else raw["mlp"]["ff"])
        assert layer.mixer.kv_from == raw["mixer"].get("kv_from")
        assert layer.mixer.rot_dims == raw["mixer"]["rot"]["dims"]
    assert PeratarConfig.from_dict(typed.to_json_dict()) == typed


def test_config_refusals():
    def broken(change):
        cfg = copy.deepcopy(pc.SMALL)
        change(cfg)
        return cfg

    cases = [
        lambda c: c["layers"][0].update(type="convolution"),
        lambda c: c["layers"][0]["mlp"].update(kind="routed"),
        lambda c: c["layers"][0]["mixer"].update(kv_from=0),         # itself
        lambda c: c["layers"][1]["mixer"].update(kv_from=2),         # a later layer
        lambda c: c["layers"][2]["mixer"].update(kv_rank=48),        # not its source's rank
        lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
        lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10),    # more than rot_dim
        lambda c: c["layers"][0]["mixer"].pop("scale"),
        lambda c: c.pop("norm"),
        lambda c: c.update(layers=[]),
        lambda c: c.update(logit_softcap=0.0),
    ]
    for change in cases:
        with pytest.raises(ConfigError):
            PeratarConfig.from_dict(broken(change))
    # a layer may not read a layer that itself reads another
    chained = copy.deepcopy(pc.SMALL)
    chained["layers"].append(copy.deepcopy(chained["layers"][2]))
    chained["layers"][3]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError):
        PeratarConfig.from_dict(chained)


def test_spec_names_shapes_and_schedule():
    arch = architecture_of(pc.ODD)
    spec = arch.build_spec(arch.parse_config(pc.ODD))
    tensors = {name: tuple(src.shape) for name, src in spec.checkpoint_tensors().items()}
    E = 128
    assert tensors["embed"] == (331, E) and tensors["head"] == (331, E) and tensors["final.norm"] == (E,)
    assert tensors["l1.mix.q"] == (5 * (24 + 6), E)
    assert tensors["l1.mix.dkv"] == (33 + 6, E) and tensors["l1.mix.dkv.norm"] == (33,)
    assert tensors["l1.mix.uk"] == (5 * 24, 33) and tensors["l1.mix.uv"] == (5 * 16, 33)
    assert tensors["l1.mix.g"] == (5, E) and tensors["l1.mix.o"] == (E, 5 * 16)
    assert tensors["l1.mlp.up"] == (132, E) and tensors["l1.mlp.down.b"] == (E,) and tensors["l1.mlp.act"] == (2,)
    assert tensors["l3.rg2"] == (E, E) and tensors["l3.rg1.b"] == (E,)
    assert tensors["l0.dwa"] == (2,) and tensors["l4.dwa"] == (6,)
    # a layer on another layer's cache has no down projection; one without feed-forward no second norm
    assert "l2.mix.dkv" not in tensors and "l4.mix.dkv.norm" not in tensors
    assert "l2.mlp.up" not in tensors and "l2.norm2" not in tensors and "l2.rg2" not in tensors
    assert [entry.cache_of for entry in spec.schedule] == [None, None, 1, None, 0]
    mixer = spec.layers[1].mixer
    assert [s.name for s in mixer.weights["in.weight"].sources] == ["l1.rg1", "l1.mix.q", "l1.mix.dkv", "l1.mix.g"]
    assert [s.name for s in spec.layers[2].mixer.weights["in.weight"].sources] == ["l2.rg1", "l2.mix.q", "l2.mix.g"]
    assert spec.lm_head.params["softcap"] == 30.0


def test_random_model_folder_loads_by_name(tmp_path):
    from velox_b200.weights import write_random_model
    from velox_b200.weights.loader import Checkpoint, WeightError, check_checkpoint

    folder = str(tmp_path / "m")
    spec = write_random_model(folder, pc.SMALL, seed=3)
    assert load_model_config(folder) == PeratarConfig.from_dict(pc.SMALL)
    check_checkpoint(Checkpoint(folder), spec)
    with open(os.path.join(folder, "config.json")) as handle:
        assert json.load(handle)["architecture"] == "Peratar"
    # the weights of the depth mix start near an average, so that a random model keeps its scale
    from helpers import read_tensors

    dwa = read_tensors(folder)["l2.dwa"].float()
    assert abs(float(dwa.mean()) - 0.25) < 0.05
    other = architecture_of(pc.ODD)
    with pytest.raises(WeightError):
        check_checkpoint(Checkpoint(folder), other.build_spec(other.parse_config(pc.ODD)))


def test_latent_cache_costs_one_array_per_page():
    from velox_b200.cache.storage import bytes_per_page
    from velox_b200.parts.base import CacheNeeds, PagedCacheSpec

    both = CacheNeeds(paged=PagedCacheSpec(1, 48))
    one = CacheNeeds(paged=PagedCacheSpec(1, 48, None, values_in_keys=True))
    assert bytes_per_page([both], 16, torch.bfloat16) == 2 * bytes_per_page([one], 16, torch.bfloat16)


# ------------------------------------------------------------------ the plain implementation itself
def test_plain_rotation_keeps_lengths_and_relative_angles():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(6, 3, 12, generator=gen, dtype=torch.float64)
    pos = torch.tensor([0, 1, 5, 6, 100, 104])
    y = plain.rotate_pairs(x, pos, 300.0, 8)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1))
    # a product of two rotated vectors depends on the distance of their positions only
    a = torch.randn(1, 1, 8, generator=gen, dtype=torch.float64).expand(6, 1, 8)
    ra = plain.rotate_pairs(a, pos, 300.0, 8)[:, 0]
    assert torch.allclose(ra[1] @ ra[2], ra[4] @ ra[5])


def test_plain_activation_and_norms():
    z = torch.tensor([-1e-9, 0.0, 1e-9], dtype=torch.float64)
    v = plain.xielu(z, 0.3, -0.4)
    assert torch.allclose(v, z / 2, atol=1e-15)  # continuous at 0 with slope 1/2
    big = plain.xielu(torch.tensor([3.0], dtype=torch.float64), 0.3, -0.4)
    assert torch.allclose(big, torch.tensor([plain.softplus(0.3) * 9 + 1.5], dtype=torch.float64))
    x = torch.randn(4, 10, dtype=torch.float64) + 3
    w = torch.ones(10, dtype=torch.float64)
    n = plain.layer_norm(x, w, 0.0)
    assert torch.allclose(n.mean(-1), torch.zeros(4, dtype=torch.float64), atol=1e-12)
    assert torch.allclose((n * n).mean(-1), torch.ones(4, dtype=torch.float64))
    r = plain.rms_norm(x, w, 0.0)
    assert torch.allclose((r * r).mean(-1), torch.ones(4, dtype=torch.float64))


def test_plain_model_is_causal_and_uses_the_shared_cache():
    tensors = pc.make_weights(pc.SMALL, seed=1, sharp=2.0)
    tokens = list(range(3, 40))
    full = plain.forward_logits(tensors, pc.SMALL, tokens)
    part = plain.forward_logits(tensors, pc.SMALL, tokens[:20])
    assert torch.allclose(full[:20], part, atol=1e-9)
    # the last layer reads the first layer's cached latent: changing the first layer's down
    # projection changes the logits even where the first layer's own output gate is shut
    changed = dict(tensors)
    changed["l0.mix.dkv"] = tensors["l0.mix.dkv"] * 1.5
    assert not torch.allclose(plain.forward_logits(changed, pc.SMALL, tokens), full, atol=1e-3)


def test_presets_at_the_qwen_widths_and_other_layer_counts():
    from velox_b200.config.presets import model_size, with_layers

    cfg = model_size("peratar-1.5b")
    twin = model_size("1.5b")
    assert cfg["width"] == twin["hidden_size"] and len(cfg["layers"]) == twin["num_hidden_layers"]
    for count in (1, 2, 5, 40):
        typed = PeratarConfig.from_dict(with_layers(cfg, count))
        assert typed.num_hidden_layers == count
        for index, layer in enumerate(typed.layers):
            assert layer.mixer.kv_from in (None, index - 1)
    assert with_layers(twin, 3)["num_hidden_layers"] == 3
    # a layer's weights are about as many bytes as its twin's
    from velox_b200.cli.roofline import layer_bytes

    mine, _ = layer_bytes(cfg, 1, 1)
    theirs, _ = layer_bytes(twin, 1, 1)
    assert 0.9 < mine / theirs < 1.1
