"""Fikevik without a GPU: configuration, refusals, the spec it builds, cache and state arithmetic of layers that
run another layer's tensors, and the plain implementation's mechanisms on cases small enough to work out by hand."""
import copy
import math

import pytest
import torch

import plain_fikevik as P
from tiny_fikevik import TINY, load_folder, write_tiny

from rosellm_b200.config.base import ConfigError, parse_config, resolve_architecture
from rosellm_b200.config.fikevik import FikevikConfig
from rosellm_b200.models.model import Model, named_params_of_spec
from rosellm_b200.weights.loader import WeightError, match_tensors


def spec_of(raw):
    cfg = parse_config(raw)
    return cfg, resolve_architecture(cfg.to_dict()).build_spec(cfg)


@pytest.mark.parametrize("name", list(TINY))
def test_configuration_round_trip_and_spec(name):
    raw = TINY[name]["raw"]
    cfg, spec = spec_of(raw)
    assert isinstance(cfg, FikevikConfig) and FikevikConfig.from_dict(cfg.to_dict()) == cfg
    owners = [i for i, l in enumerate(raw["layers"]) if l.get("weights_of") is None]
    assert len(spec.layers) == len(owners) and len(spec.run_order) == len(raw["layers"]) and spec.head.kind == "linear"
    for i, (lr, run) in enumerate(zip(raw["layers"], spec.run_order)):
        assert run.own_key == i and run.writes_cache
        assert run.layer == owners.index(cfg.weight_owner(i))
        ls = spec.layers[run.layer]
        names = [n for n, _, _ in ls.parts]
        assert ("mixer" in names) == (lr["type"] == "gla") and ("left" in names) == ("right" in names) == (lr["type"] == "parallel")
        assert (lr["mlp"] is None) == ("feed_forward" not in names)
        if lr["type"] == "parallel":
            left = ls.part("left").params
            assert left["window"] == (lr["mixer"]["left"].get("mask") or {}).get("size")
            assert left["rot_dims"] == (lr["mixer"]["left"].get("rot") or {}).get("dims", 0)


def test_refusals():
    raw = TINY["A"]["raw"]
    for path, value in ((("layers", 0, "type"), "conv"), (("layers", 1, "mixer", "left", "kv_heads"), 4), (("width",), 60),
                        (("layers", 1, "mixer", "left", "rot", "dims"), 7), (("layers", 1, "mixer", "left", "rot", "dims"), 22),
                        (("layers", 1, "mixer", "left", "mask", "size"), 0), (("layers", 0, "mixer", "tau"), 0.0),
                        (("layers", 1, "mixer", "right", "gate_cap"), 0.0), (("norm", "eps"), 0.0), (("layers", 2, "weights_of"), 9),
                        (("layers", 2, "weights_of"), 2), (("layers", 2, "weights_of"), 1), (("layers", 0, "mlp", "kind"), "moe")):
        bad = copy.deepcopy(raw)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(bad)
    loop = copy.deepcopy(raw)
    loop["layers"][0]["weights_of"] = 2  # 0 -> 2 -> 0
    with pytest.raises(ConfigError):
        parse_config(loop)


def test_every_run_keeps_pages_and_state_of_its_own(tmp_path):
    """A layer that runs another's tensors has cache pages and state rows under its own number; the cache rows of
    the windowed attention and the matrix memory's state (the normaliser as one more column, then the maxima)."""
    cfg, spec = spec_of(TINY["A"]["raw"])
    m = Model(spec, torch.float32, "cpu")
    kv, st = m.kv_specs(), m.state_specs()
    assert set(kv) == {(1, "left"), (3, "left")} and all(s.planes == 1 and s.window == 7 for s in kv.values())
    assert kv[(1, "left")].num_kv_heads == 2 and kv[(1, "left")].head_dim == 40   # key 20 -> 24, value 12 -> 36, filled up to 40
    assert set(st) == {0, 2, 4, (1, "right"), (3, "right")}
    assert st[0].shape == st[2].shape == (3, 24, 10) and st[4].shape == (2, 8, 40)
    assert st[(1, "right")].shape == (3 * 8 * 21 + 3,) and st[(1, "right")].dtype == torch.float32
    assert m.layers[spec.run_order[2].layer] is m.layers[spec.run_order[0].layer]
    # a model of linear attention only caches no keys
    _, spec_e = spec_of(TINY["E"]["raw"])
    assert Model(spec_e, torch.float32, "cpu").kv_specs() == {}


def test_tensor_names_and_a_rank_taken_from_the_file(tmp_path):
    folder = write_tiny("A", str(tmp_path))
    raw, tensors = load_folder(folder)
    assert not any(k.startswith(("l2.", "l3.")) for k in tensors)  # layers 2 and 3 have no tensors of their own
    assert {"embed", "head", "final.norm", "l0.mix.a2.b", "l0.rg1.b", "l1.mix.left.q.norm", "l1.mix.left.temp", "l1.mix.right.i.b",
            "l1.mix.right.norm", "l0.mlp.gate", "l4.mix.norm"} <= set(tensors)
    assert tensors["l1.mix.left.temp"].shape == (6,) and tensors["l1.mix.right.norm"].shape == (60,)
    assert tensors["l0.mix.norm"].shape == (10,) and tensors["l1.mix.left.k"].shape == (40, 64)
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
    _, spec2 = spec_of(raw)
    tensors = {k: v.float() for k, v in tensors.items()}
    match_tensors(named_params_of_spec(spec2), tensors, source="test")
    m2 = Model(spec2, torch.float32, "cpu")
    m2.load_tensors(tensors)
    assert m2.layers[0].mixer.rank == 5 and m2.layers[2].mixer.rank == 3
    del tensors["l1.mix.left.temp"]
    with pytest.raises(WeightError):
        match_tensors(named_params_of_spec(spec2), tensors, source="test")


def test_plain_rotation_and_window_by_hand():
    y = torch.tensor([[[1.0, 0.0, 2.0, 0.0, 5.0, 6.0]]], dtype=torch.float64).repeat(3, 1, 1)
    out = P.rotate_pairs(y, torch.arange(3), 4, 100.0)
    for p in range(3):
        a0, a1 = p * 1.0, p * 100.0 ** -0.5
        assert out[p, 0].tolist() == pytest.approx([math.cos(a0), math.sin(a0), 2 * math.cos(a1), 2 * math.sin(a1), 5.0, 6.0])
    # equal scores: a query averages the values of the keys it sees, the last `size` of them
    T = 6
    q, k = torch.zeros(T, 2, 3, dtype=torch.float64), torch.zeros(T, 1, 3, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1)
    o = P.window_softmax(q, k, v, 1.0, torch.ones(2, dtype=torch.float64), 3)
    assert o[:, 1, 0].tolist() == pytest.approx([0.0, 0.5, 1.0, 2.0, 3.0, 4.0])
    assert P.window_softmax(q, k, v, 1.0, torch.ones(2, dtype=torch.float64), 1)[:, 0, 0].tolist() == pytest.approx(list(range(T)))
    assert P.window_softmax(q, k, v, 1.0, torch.ones(2, dtype=torch.float64), None)[:, 0, 0].tolist() == pytest.approx([i / 2 for i in range(T)])
    # a head's temperature multiplies its scores only
    q[5, :, 0], k[4, 0, 0] = 1.0, 2.0
    o = P.window_softmax(q, k, v, 0.5, torch.tensor([1.0, 3.0], dtype=torch.float64), 3)
    for head, temp in ((0, 1.0), (1, 3.0)):
        e = math.exp(temp)
        assert float(o[5, head, 0]) == pytest.approx((3 + 4 * e + 5) / (2 + e))


def test_plain_layer_and_join_by_hand():
    x, y = torch.tensor([[3.0, 4.0]], dtype=torch.float64), torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    w = {"g": torch.zeros(2, 2, dtype=torch.float64), "g.b": torch.tensor([0.0, math.log(3.0)], dtype=torch.float64),
         "n": torch.tensor([2.0, 0.5], dtype=torch.float64)}
    s = [2 * 3 + 0.5 * 1, 2 * 4 + 0.75 * -2]
    r = math.sqrt((s[0] ** 2 + s[1] ** 2) / 2 + 1e-3)
    assert P.sublayer_join(x, y, w, "g", "n", 2.0, 1e-3)[0].tolist() == pytest.approx([s[0] / r * 2, s[1] / r * 0.5])
    assert P.embed(torch.tensor([[1.0], [2.0]], dtype=torch.float64), [1, 0], 12.0)[:, 0].tolist() == [24.0, 12.0]


def test_state_mixers_by_hand():
    """Two tokens, one head, sizes of one: the numbers of the plain recurrences worked out by hand."""
    one = lambda *v: torch.tensor(v, dtype=torch.float64).view(len(v), 1, 1)
    o = P.decay_recurrence(one(1, 2), one(3, 5), one(7, 11), one(0.5, 0.25))
    assert torch.allclose(o.view(-1), torch.tensor([21.0, 2 * (0.25 * 21 + 55)], dtype=torch.float64))
    gi, gf = torch.tensor([[1.0], [-2.0]], dtype=torch.float64), torch.tensor([[-0.5], [-0.25]], dtype=torch.float64)
    o = P.memory_recurrence(one(1, 2), one(3, 5), one(7, 11), gi, gf, floor=0.0)
    # m_1 = max(-0.5 + 0, 1) = 1: S = e^0 * 21, n = 3; o = 21 / max(3, e^-1) = 7
    # m_2 = max(-0.25 + 1, -2) = 0.75: S = 21 + e^-2.75 * 55, n = 3 + e^-2.75 * 5; o = 2 S / max(2 n, e^-0.75)
    w = math.exp(-2.75)
    assert torch.allclose(o.view(-1), torch.tensor([7.0, (21 + w * 55) / (3 + w * 5)], dtype=torch.float64))
    # from nothing, a weak input: the floor e^(-m) with m = 0 bounds the divisor
    o = P.memory_recurrence(one(1), one(0.01), one(5), torch.tensor([[-3.0]], dtype=torch.float64),
                            torch.tensor([[-1.0]], dtype=torch.float64), floor=0.0)
    assert torch.allclose(o.view(-1), torch.tensor([math.exp(-2.0) * 0.05 / math.exp(1.0)], dtype=torch.float64))
