"""Soporax without a GPU: configuration, refusals, the spec it builds (runs of a repeated stretch with pages of
their own, what is added ahead of a pass), tensor names, the frequency scalings, and the plain implementation's
mechanisms on cases small enough to work out by hand."""
import copy
import math

import pytest
import torch

import plain_soporax as P
from tiny_soporax import TINY, WIDE, load_folder, write_tiny

from rosellm_b200.config.base import ConfigError, parse_config, resolve_architecture
from rosellm_b200.config.soporax import SoporaxConfig
from rosellm_b200.models.model import Model, named_params_of_spec
from rosellm_b200.parts.standard import scaled_rotary_frequencies
from rosellm_b200.weights.loader import WeightError, match_tensors


def spec_of(raw):
    cfg = parse_config(raw)
    return cfg, resolve_architecture(cfg.to_dict()).build_spec(cfg)


@pytest.mark.parametrize("name", list(TINY) + ["WIDE"])
def test_configuration_round_trip_and_spec(name):
    raw = WIDE["raw"] if name == "WIDE" else TINY[name]["raw"]
    cfg, spec = spec_of(raw)
    assert isinstance(cfg, SoporaxConfig) and SoporaxConfig.from_dict(cfg.to_dict()) == cfg
    want = P.run_order(raw)
    assert [r.layer for r in spec.run_order] == [i for i, _ in want]
    assert [r.own_key for r in spec.run_order] == list(range(len(want))) and all(r.writes_cache for r in spec.run_order)
    assert len(spec.layers) == len(raw["layers"]) and spec.head.kind == "tied_to_embedding"
    assert spec.final_norm.params["out_scale"] == raw["logit_scale"]
    # what is added ahead of a pass: at the pass's first layer, with the pass's number
    starts = [(pos, t) for pos, (_, t) in enumerate(want) if t is not None and t >= 0]
    assert [(s.before, dict(s.args)["index"]) for s in spec.stream_inputs] == starts
    assert len(spec.stream_parts) == (1 if raw.get("loop") else 0)
    for lr, ls in zip(raw["layers"], spec.layers):
        names = [n for n, _, _ in ls.parts]
        assert (lr["mlp"] is None) == ("feed_forward" not in names) and ls.block.kind == "parallel_sublayers"
        mixer = ls.part("mixer")
        if lr["type"] == "attention":
            assert mixer.kind == "window_attention" and mixer.params["window"] == (lr["mixer"].get("mask") or {}).get("size")
            assert mixer.params["sink"] == "learned" and mixer.params["rot_dims"] == 0 and not mixer.params["qk_norm_weights"]
        elif lr["type"] == "attention_2":
            assert mixer.params["sink"] == 0.0 and mixer.params["gate"] == "head" and mixer.params["bias"]
            assert mixer.params["window"] is None and mixer.params["rot_dims"] == lr["mixer"]["rot"]["dims"]
        else:
            assert mixer.kind == "latent_attention" and mixer.params["gate"] and not mixer.params["sink"]
            assert mixer.params["q_rank"] == lr["mixer"].get("q_rank")
        if lr["mlp"] is not None and lr["mlp"]["kind"] == "moe":
            assert ls.part("feed_forward").params["routing"] == "table"


def test_refusals():
    raw = TINY["A"]["raw"]
    for path, value in ((("layers", 0, "type"), "conv"), (("layers", 1, "mixer", "kv_heads"), 4), (("width",), 60),
                        (("layers", 2, "mixer", "rot", "dims"), 7), (("layers", 2, "mixer", "rot", "dims"), 22),
                        (("layers", 1, "mixer", "mask", "size"), 0), (("norm", "eps"), 0.0), (("loop", "stop"), 5),
                        (("loop", "start"), 3), (("loop", "times"), 0), (("layers", 1, "mlp", "router", "top"), 6),
                        (("layers", 0, "mlp", "kind"), "conv"), (("layers", 0, "mixer", "rot", "scaling", "factor"), 0.0),
                        (("layers", 0, "mixer", "rot_dim"), 5), (("layers", 0, "mixer", "q_rank"), 0),
                        (("layers", 2, "mixer", "rot", "scaling", "high"), 1.5)):
        bad = copy.deepcopy(raw)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_every_run_keeps_pages_of_its_own():
    """A layer of the repeated stretch has pages under the number of each of its runs; windowed layers tell the
    cache their window; a latent layer caches one row a token."""
    cfg, spec = spec_of(TINY["A"]["raw"])
    m = Model(spec, torch.float32, "cpu")
    kv = m.kv_specs()
    # runs: 0 | 1 2 | 1 2 | 1 2 | 3
    assert set(kv) == set(range(8)) and m.state_specs() == {}
    assert kv[0].planes == 1 and kv[0].num_kv_heads == 1 and kv[0].head_dim == 24 and kv[0].window is None
    assert kv[1] == kv[3] == kv[5] and kv[1].window == 7 and kv[1].num_kv_heads == 2 and kv[1].head_dim == 40
    assert kv[2] == kv[4] == kv[6] and kv[2].window is None and kv[2].head_dim == 24
    assert kv[7].window == 40
    assert m.layers[spec.run_order[1].layer] is m.layers[spec.run_order[3].layer]


def test_tensor_names_and_the_table(tmp_path):
    folder = write_tiny("A", str(tmp_path))
    raw, tensors = load_folder(folder)
    assert {"embed", "final.norm", "loop.step", "l0.norm1", "l0.mix.dq", "l0.mix.dq.norm", "l0.mix.uq", "l0.mix.dkv",
            "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l1.mix.sink", "l1.mlp.table",
            "l1.mlp.e4.down", "l2.mix.q.b", "l2.mix.g", "l3.mlp.up"} <= set(tensors)
    assert "head" not in tensors and not any(k.endswith("norm2") for k in tensors)
    assert tensors["loop.step"].shape == (3, 64) and tensors["l2.mix.g"].shape == (4, 64) and tensors["l0.mix.g"].shape == (30, 64)
    assert tensors["l0.mix.uq"].shape == (3 * 18, 20) and tensors["l0.mix.dkv"].shape == (24, 64)
    table = tensors["l1.mlp.table"]
    assert table.dtype == torch.int32 and table.shape == (131, 2) and int(table.min()) >= 0 and int(table.max()) < 5
    assert bool((table[:, 0] != table[:, 1]).all()) and len(set(table[:, 0].tolist())) == 5
    _, spec = spec_of(raw)
    tensors = {k: (v.float() if v.is_floating_point() else v) for k, v in tensors.items()}
    match_tensors(named_params_of_spec(spec), tensors, source="test")
    bad = dict(tensors)
    bad["l1.mlp.table"] = bad["l1.mlp.table"].float()
    with pytest.raises(WeightError):
        match_tensors(named_params_of_spec(spec), bad, source="test")
    del tensors["l1.mix.sink"]
    with pytest.raises(WeightError):
        match_tensors(named_params_of_spec(spec), tensors, source="test")


@pytest.mark.parametrize("dims,base", [(12, 500.0), (64, 20000.0), (2, 9.0), (96, 1.0e6)])
def test_frequency_scalings_against_the_plain_ones(dims, base):
    plain = P.plain_frequencies(dims, base)
    f, mult = scaled_rotary_frequencies(dims, base, None)
    assert mult == 1.0 and f.tolist() == pytest.approx(plain, rel=1e-6)
    for factor, low, high, original in ((3.0, 1.5, 5.0, 16), (8.0, 0.5, 8.0, 2048), (2.0, 2.0, 3.0, 40), (16.0, 1.0, 6.0, 100000)):
        f, mult = scaled_rotary_frequencies(dims, base, dict(kind="wavelength", factor=factor, low=low, high=high, original=original))
        assert mult == 1.0 and f.tolist() == pytest.approx(P.wavelength_scaled(plain, factor, low, high, original), rel=1e-6)
    for factor, original, fast, slow in ((8.0, 32, 16.0, 2.0), (16.0, 300, 24.0, 1.5), (40.0, 48, 8.0, 2.0), (2.0, 20, 4.0, 0.5),
                                         (3.0, 6, 1.0, 1.0)):
        f, mult = scaled_rotary_frequencies(dims, base, dict(kind="ramp", factor=factor, original=original, fast=fast, slow=slow))
        want, want_mult = P.ramp_scaled(plain, dims, base, factor, original, fast, slow)
        assert mult == pytest.approx(want_mult) and f.tolist() == pytest.approx(want, rel=1e-6)
    with pytest.raises(ValueError):
        scaled_rotary_frequencies(dims, base, dict(kind="other", factor=2.0, original=8))


def test_plain_frequency_scalings_by_hand():
    # wavelengths 2 pi, 20 pi, 200 pi against original 100: below 100 / 4 kept, above 100 / 1 slowed, between blended
    f = P.wavelength_scaled([1.0, 0.1, 0.01], 8.0, 1.0, 4.0, 100.0)
    s = (100.0 / (20 * math.pi) - 1.0) / 3.0
    assert f == pytest.approx([1.0, (1 - s) * 0.1 / 8 + s * 0.1, 0.01 / 8])
    # the ramp: pairs below lo keep their frequency, above hi are slowed; between, in proportion
    dims, base = 8, 10000.0
    plain = P.plain_frequencies(dims, base)
    idx = lambda t: dims * math.log(64 / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(idx(4.0)), 0), min(math.ceil(idx(0.25)), dims - 1)
    assert (lo, hi) == (0, 2)
    f, mult = P.ramp_scaled(plain, dims, base, 4.0, 64, 4.0, 0.25)
    assert f == pytest.approx([plain[0], plain[1] * (0.5 / 4 + 0.5), plain[2] / 4, plain[3] / 4])
    assert mult == pytest.approx(0.1 * math.log(4.0) + 1.0)


def test_plain_rotation_sink_and_window_by_hand():
    y = torch.tensor([[[1.0, 0.0, 2.0, 0.0, 5.0, 6.0]]], dtype=torch.float64).repeat(3, 1, 1)
    out = P.rotate_pairs(y, torch.arange(3), [1.0, 0.1], mult=2.0)
    for p in range(3):
        a0, a1 = p * 1.0, p * 0.1
        assert out[p, 0].tolist() == pytest.approx([2 * math.cos(a0), 2 * math.sin(a0), 4 * math.cos(a1), 4 * math.sin(a1), 5.0, 6.0])
    # equal scores of zero: a query averages the values it sees; a sink of score s takes e^s shares of the weight
    T = 6
    q, k = torch.zeros(T, 2, 3, dtype=torch.float64), torch.zeros(T, 1, 3, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1)
    o = P.softmax_attention(q, k, v, 1.0, 3, None)
    assert o[:, 1, 0].tolist() == pytest.approx([0.0, 0.5, 1.0, 2.0, 3.0, 4.0])
    sink = torch.tensor([0.0, math.log(3.0)], dtype=torch.float64)
    o = P.softmax_attention(q, k, v, 1.0, 3, sink)
    assert o[:, 0, 0].tolist() == pytest.approx([0.0, 1 / 3, 3 / 4, 6 / 4, 9 / 4, 12 / 4])
    assert o[:, 1, 0].tolist() == pytest.approx([0.0, 1 / 5, 3 / 6, 6 / 6, 9 / 6, 12 / 6])
    assert P.softmax_attention(q, k, v, 1.0, 1, None)[:, 0, 0].tolist() == pytest.approx(list(range(T)))
    assert P.softmax_attention(q, k, v, 1.0, None, None)[:, 0, 0].tolist() == pytest.approx([i / 2 for i in range(T)])
    # the sink is not scaled: halving the scale leaves its share as it is when all scores are zero
    assert torch.equal(P.softmax_attention(q, k, v, 0.5, 3, sink), o)


def test_plain_feed_forwards_and_passes_by_hand():
    h = torch.tensor([[2.0, -1.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    w = {"m.gate": eye * 3.0, "m.up": eye * 0.25, "m.down": eye}
    # gate 6 -> 1.5 and -3 stays; up 0.5 and -0.25, within the limit
    sg = lambda z: z / (1 + math.exp(-1.702 * z))
    assert P.clamped_dense(h, w, "m.", 1.5)[0].tolist() == pytest.approx([sg(1.5) * 1.5, sg(-3.0) * 0.75])
    assert P.clamped_dense(h, w, "m.", 0.1)[0].tolist() == pytest.approx([sg(0.1) * 1.1, sg(-3.0) * 0.9])
    # two experts, the token's row of the table names both or one
    w = {"m.table": torch.tensor([[0, 1], [1, 0], [1, 1]], dtype=torch.int32)}
    for e, c in ((0, 1.0), (1, 10.0)):
        w.update({f"m.e{e}.gate": eye, f"m.e{e}.up": eye, f"m.e{e}.down": eye * c})
    silu = lambda z: z / (1 + math.exp(-z))
    one = [silu(2.0) * 2.0, silu(-1.0) * -1.0]
    assert P.table_experts(h, [0], w, "m.", 2)[0].tolist() == pytest.approx([5.5 * a for a in one])
    assert P.table_experts(h, [2], w, "m.", 1)[0].tolist() == pytest.approx([10.0 * a for a in one])
    assert P.run_order({"layers": [0] * 4, "loop": {"start": 1, "stop": 3, "times": 2}}) == \
        [(0, None), (1, 0), (2, -1), (1, 1), (2, -1), (3, None)]
    assert P.run_order({"layers": [0] * 2}) == [(0, None), (1, None)]


def test_what_a_pass_adds(tmp_path):
    """A stretch run once differs from no stretch by its row alone; ahead of later passes the token rows come again."""
    folder = write_tiny("E", str(tmp_path))
    cfg, w = load_folder(folder)
    toks = [3, 50, 7, 7, 12]
    streams = []
    P.forward(cfg, w, toks, streams=streams)
    plain = dict(cfg)
    del plain["loop"]
    w2 = dict(w)
    w2["embed"] = w["embed"] + w["loop.step"][0]
    streams2 = []
    P.forward(plain, w2, toks, streams=streams2)
    assert torch.allclose(streams[0], streams2[0], atol=1e-12) and len(streams) == 2
    twice = dict(cfg, loop={"start": 0, "stop": 1, "times": 2})
    w3 = dict(w, **{"loop.step": torch.stack([w["loop.step"][0], w["loop.step"][0] * 3.0])})
    s3 = []
    P.forward(twice, w3, toks, streams=s3)
    x0 = w["embed"][torch.tensor(toks)]
    again = P.layer(s3[0] + x0 + w3["loop.step"][1], toks, w, 0, cfg["layers"][0], cfg["norm"]["eps"])
    assert torch.allclose(s3[1], again, atol=1e-12) and len(s3) == 3
