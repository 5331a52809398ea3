"""CPU tests of the Redalix design: configuration parsing and refusals, the spec's tensor names
and shapes, the random-weights folder, the cache groups with kept first keys, the layout of
attention work whose rows the merge kernel finishes, and the plain implementation's own
mechanisms against closed forms."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_redalix as plain
import redalix_configs as rc
from velox_b200.cache.manager import CacheGroup, CacheManager
from velox_b200.config.model_config import ConfigError, RedalixConfig
from velox_b200.config.registry import architecture_of
from velox_b200.ops import attention_plan as ap


def parse(cfg):
    arch = architecture_of(cfg)
    return arch, arch.parse_config(cfg)


@pytest.mark.parametrize("name", list(rc.ALL))
def test_configuration_round_trip_and_tensor_names(name):
    cfg = rc.ALL[name]
    arch, typed = parse(cfg)
    assert isinstance(typed, RedalixConfig)
    again = typed.to_json_dict()
    assert again["layers"] == cfg["layers"] and again["vocab"] == cfg["vocab"] and again["width"] == cfg["width"]
    assert arch.parse_config(again) == typed
    spec = arch.build_spec(typed)
    tensors = spec.checkpoint_tensors()
    E = cfg["width"]
    assert tensors["embed"].shape == (cfg["vocab"], E) and tensors["head"].shape == (cfg["vocab"], E)
    for index, layer in enumerate(cfg["layers"]):
        p = f"l{index}."
        assert tensors[p + "norm1"].shape == (E,)
        m = layer["mixer"]
        if layer["type"] == "parallel":
            left, right = m["left"], m["right"]
            assert tensors[p + "mix.left.q"].shape == (left["heads"] * left["dim"], E)
            assert tensors[p + "mix.left.v"].shape == (left["kv_heads"] * left["vdim"], E)
            assert tensors[p + "mix.left.o"].shape == (E, left["heads"] * left["vdim"])
            assert tensors[p + "mix.left.sink"].shape == (left["heads"],)
            part = right["width"] // right["blocks"]
            assert tensors[p + "mix.right.ra"].shape == (right["blocks"], part, part)
            assert tensors[p + "mix.right.conv"].shape == (right["width"], right["conv"])
            assert tensors[p + "mix.left.out"].shape == (E,) and tensors[p + "mix.right.out"].shape == (E,)
            assert p + "mix.left.q.b" not in tensors and p + "mix.left.g" not in tensors
        elif layer["type"] == "attention":
            assert tensors[p + "mix.g"].shape == (m["heads"], E)
            assert tensors[p + "mix.k.b"].shape == (m["kv_heads"] * m["dim"],)
            assert p + "mix.sink" not in tensors
        else:
            inner = m["heads"] * m["vdim"]
            assert tensors[p + "mix.in"].shape == (2 * inner + 2 * m["groups"] * m["state"] + m["heads"], E)
            assert tensors[p + "mix.conv"].shape == (inner + 2 * m["groups"] * m["state"], m["conv"])
        mlp = layer["mlp"]
        if mlp is None:
            assert not any(k.startswith(p + "mlp.") for k in tensors)
        elif mlp["kind"] == "moe":
            assert tensors[p + "mlp.table"].shape == (cfg["vocab"], mlp["router"]["top"])
            assert tensors[f"{p}mlp.e{mlp['router']['experts'] - 1}.down"].shape == (E, mlp["expert"]["ff"])
            assert (p + "mlp.shared.sg" in tensors) == ("shared" in mlp)


def test_refusals():
    base = rc.SMALL
    def broken(edit):
        cfg = copy.deepcopy(base)
        edit(cfg)
        return cfg
    cases = [
        lambda c: c["layers"][0].update(type="convolution"),
        lambda c: c["layers"][0]["mixer"]["left"].update(heads=3),               # not a multiple of kv_heads
        lambda c: c["layers"][0]["mixer"]["right"].update(blocks=5),              # does not divide the width
        lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26),                 # more than dim
        lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=2),           # not a key of this mixer
        lambda c: c["layers"][0]["mixer"]["left"].update(rot={"base": 10.0, "dims": 4}),
        lambda c: c["layers"][1]["mlp"]["router"].update(top=9),
        lambda c: c["layers"][1]["mlp"].update(kind="routed"),
        lambda c: c["layers"][2]["mixer"].update(groups=3),
        lambda c: c["layers"][2]["mixer"].update(norm_groups=5),
        lambda c: c.pop("norm"),
        lambda c: c.update(layers=[]),
    ]
    for edit in cases:
        with pytest.raises(ConfigError):
            parse(broken(edit))


def test_random_weights_folder(tmp_path):
    from safetensors.torch import load_file

    from velox_b200.weights import write_random_model

    folder = str(tmp_path / "m")
    spec = write_random_model(folder, rc.SMALL, seed=4, dtype="bfloat16")
    tensors = load_file(folder + "/model.safetensors")
    assert set(tensors) == set(spec.checkpoint_tensors())
    table = tensors["l1.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 5
    assert all(len(set(row.tolist())) == table.shape[1] for row in table)
    assert json.load(open(folder + "/config.json"))["layers"] == rc.SMALL["layers"]
    # the plain model runs on what was written
    weights = {k: (v.numpy() if v.dtype == torch.int32 else v.float().numpy()) for k, v in tensors.items()}
    assert np.isfinite(plain.forward(rc.SMALL, weights, [3, 1, 4, 1, 5, 9, 2, 6])).all()


def test_pages_of_kept_first_keys_are_not_given_back():
    groups = [CacheGroup("all", None), CacheGroup("w", 8, keep_first=5), CacheGroup("plain", 8)]
    cache = CacheManager(groups, num_pages=40, page_size=4, max_num_seqs=2)
    seq = cache.new_sequence("a")
    assert cache.append_slots(seq, 30)
    cache.advance(seq, 30)
    # the next query is at 30 and sees keys 23..; blocks 0..4 hold keys below 20
    assert seq.tables[0].count(0) == 0
    assert [i for i, page in enumerate(seq.tables[2]) if page == 0] == [0, 1, 2, 3, 4]
    assert [i for i, page in enumerate(seq.tables[1]) if page == 0] == [2, 3, 4]      # blocks 0 and 1 hold keys 0..4
    cache.assert_consistent()
    assert cache.append_slots(seq, 9)
    cache.advance(seq, 9)
    assert seq.tables[1][0] != 0 and seq.tables[1][1] != 0
    cache.assert_consistent()
    cache.free(seq)
    assert cache.num_free_pages() == cache.num_total_pages
    for alloc in cache.allocators:
        alloc.assert_consistent()
        assert alloc.num_used == 0


def test_layout_of_rows_the_merge_finishes():
    opt = ap.PlanOptions(num_kv_heads=2, group=2, window=10, use_f32=True, keep_first=4, anchored=True)
    plan = ap.plan_attention([1, 20, 3], [50, 20, 9], opt)
    items, merges = plan.items[ap.KIND_F32], plan.merge_items
    rows = {(int(i[0]), int(i[1])): [] for i in items}
    for i in items:
        rows[(int(i[0]), int(i[1]))].append((int(i[3]), int(i[4]), int(i[7])))
    # the decoded token at position 49: window keys 40..49 and the kept keys 0..3
    assert sorted(rows[(0, 0)]) == [(0, 4, 2), (40, 50, 2)]
    # a portion from the start: its first tile reaches back to key 0, no second range
    assert rows[(1, 0)] == [(0, 8, 1)]
    # a later tile of it (tokens 8..15): the window of its first token starts at 0 as well
    assert rows[(1, 16)] == [(0, 16, 1)]
    assert len(merges) == len(rows)
    for m in merges:
        assert int(m[4]) == len(rows[(int(m[0]), int(m[1]))])
    # partial rows do not overlap
    spans = sorted((int(i[5]), int(i[5]) + opt.num_kv_heads * int(i[2])) for i in items)
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] == plan.partial_rows
    # the fixed shape of padded single-token steps: two items and one merge item per sequence
    kind, padded, padded_merges, partial = ap.plan_single_tokens(np.array([50, 3]), 4, 2, opt)
    assert padded.shape == (8, 8) and padded_merges.shape == (4, 8) and (padded[4:, 0] == -1).all()
    assert sorted((int(i[3]), int(i[4])) for i in padded[:2]) == [(0, 4), (40, 50)]
    assert sorted((int(i[3]), int(i[4])) for i in padded[2:4]) == [(0, 0), (0, 3)]
    assert partial >= 4 * opt.num_kv_heads * 2


def test_plain_mechanisms():
    # the window with kept first keys
    mask = plain.visible(12, 3, 2)
    assert mask[11].tolist() == [True, True] + [False] * 7 + [True] * 3
    assert mask[1].tolist() == [True, True] + [False] * 10
    # stretched pairs: the fastest pairs keep their frequency, the slowest are divided by the factor
    freq, magnitude = plain.yarn_frequencies(16, 100.0, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 0.25})
    plain_freq = np.array([100.0 ** (-2 * i / 16) for i in range(8)])
    assert np.isclose(freq[0], plain_freq[0]) and np.isclose(freq[-1], plain_freq[-1] / 4.0)
    assert np.isclose(magnitude, 0.1 * np.log(4.0) + 1.0)
    # rotation keeps lengths (without the magnitude) and turns pair i by position * f_i
    x = np.random.default_rng(0).normal(size=(5, 2, 8))
    y = plain.rotate_pairs(x, np.arange(5), {"base": 10.0, "dims": 4})
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1))
    assert np.allclose(y[..., 4:], x[..., 4:]) and np.allclose(y[0], x[0])
    # the convolution of an impulse is the taps, newest last
    w = np.array([[1.0, 2.0, 3.0]])
    impulse = np.zeros((5, 1))
    impulse[1] = 1.0
    assert plain.causal_conv(impulse, w, np.zeros(1))[:, 0].tolist() == [0.0, 3.0, 2.0, 1.0, 0.0]
    # constant gates: the recurrence is a geometric sum
    a, steps = 0.5, 6
    S = 0.0
    for _ in range(steps):
        S = a * S + np.sqrt(1 - a * a)
    assert np.isclose(S, np.sqrt(1 - a * a) * (1 - a ** steps) / (1 - a))
    # a sink of minus infinity is the ordinary softmax; a large one takes the weight
    cfg = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 6}}
    rng = np.random.default_rng(1)
    W = {"q": rng.normal(size=(8, 8)), "k": rng.normal(size=(4, 8)), "v": rng.normal(size=(4, 8)), "o": rng.normal(size=(8, 8))}
    h = rng.normal(size=(7, 8))
    none = plain.attention(h, W, "", cfg, np.arange(7))
    low = plain.attention(h, dict(W, sink=np.full(2, -80.0)), "", cfg, np.arange(7))
    high = plain.attention(h, dict(W, sink=np.full(2, 40.0)), "", cfg, np.arange(7))
    assert np.allclose(none, low) and np.abs(high).max() < 1e-3 * np.abs(none).max()
