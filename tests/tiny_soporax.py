"""Small Soporax configurations for the tests, and helpers to write them as model folders.

They differ from one another in every size and constant and in the order of their layers, and avoid
coincidences: key and value sizes differ, one to seven query heads a key/value head, turned entries fewer than
the key size or all of it, odd and large per-head sizes, windows of 1, of a few keys, of more than a page, of more
than any prompt, or none; experts from one to nine with one, some or all of them a token; layers without a
feed-forward; a repeated stretch at the start, in the middle, over the whole stack, run once, or none; both kinds
of frequency scaling with original lengths below the tests' prompts, and none; a query latent or none.
"""
from __future__ import annotations

import json
import os

import torch

from rosellm_b200.config.soporax import SoporaxConfig
from rosellm_b200.weights import write_model_folder


def windowed(heads, kv_heads, dim, vdim, scale, window):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def rotary(heads, kv_heads, dim, vdim, scale, dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                             "rot": rot}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if q_rank is not None:
        m["q_rank"] = q_rank
    return {"type": "latent_attention", "mixer": m}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, eps, logit_scale, loop, layers):
    out = {"architecture": "Soporax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
           "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


RAW_A = model(131, 64, 1e-5, 1.7, (1, 3, 3), [
    (latent(3, 12, 6, 10, 18, 20, 0.21, 10000.0, (8.0, 32, 16.0, 2.0)), dense(100, 0.7)),
    (windowed(6, 2, 20, 12, 0.3, 7), moe(5, 2, 24)),
    (rotary(4, 4, 16, 8, 0.25, 12, 500.0, (3.0, 1.5, 5.0, 16)), None),
    (windowed(3, 3, 8, 24, 0.4, 40), dense(36, 3.0)),
])
RAW_B = model(300, 96, 1e-6, 1.0, None, [
    (rotary(7, 1, 24, 40, 0.2, 24, 77.0), moe(3, 3, 40)),
    (windowed(4, 4, 64, 32, 0.125, None), dense(72, 1.5)),
    (latent(5, 10, 4, 12, 36, None, 0.27, 300.0), moe(9, 1, 16)),
    (rotary(2, 2, 9, 5, 0.35, 2, 1.0e6, (16.0, 0.5, 8.0, 64)), None),
])
RAW_C = model(77, 48, 1e-4, 0.35, (0, 3, 2), [
    (windowed(7, 1, 9, 5, 0.35, 1), moe(1, 1, 20)),
    (latent(1, 40, 8, 9, 24, 7, 0.15, 33.0, (2.0, 20, 4.0, 0.5)), None),
    (windowed(40, 1, 8, 8, 0.4, 1000), dense(24, 0.25)),
])
RAW_D = model(2000, 384, 1e-5, 2.5, (2, 3, 4), [
    (rotary(12, 4, 48, 80, 0.14, 32, 300000.0, (8.0, 1.0, 4.0, 96)), dense(640, 7.0)),
    (latent(6, 64, 32, 96, 200, 136, 0.1, 100000.0, (16.0, 64, 24.0, 1.5)), moe(6, 4, 96)),
    (windowed(2, 1, 136, 130, 0.09, 48), dense(96, 1.0)),
    (latent(4, 24, 16, 24, 72, 48, 0.16, 5000.0, (40.0, 48, 8.0, 2.0)), moe(4, 2, 128)),
])
# the repeated stretch run once; a stack of one kind of mixer each
RAW_E = model(90, 40, 1e-5, 1.0, (0, 1, 1), [
    (windowed(5, 5, 8, 8, 0.3, 16), dense(16, 2.0)),
    (windowed(2, 1, 20, 6, 0.2, 33), None),
])
RAW_F = model(64, 56, 1e-5, 6.0, (1, 2, 2), [
    (latent(7, 10, 6, 6, 12, 9, 0.33, 50.0, (3.0, 24, 6.0, 1.5)), None),
    (rotary(8, 2, 6, 12, 0.4, 6, 9.0, (2.0, 2.0, 3.0, 40)), moe(2, 2, 40)),
])
TINY = {
    "A": dict(raw=RAW_A, seed=61, std=0.2, page_size=16),
    "B": dict(raw=RAW_B, seed=62, std=0.15, page_size=8),
    "C": dict(raw=RAW_C, seed=63, std=0.25, page_size=32),
    "D": dict(raw=RAW_D, seed=64, std=0.07, page_size=16),
    "E": dict(raw=RAW_E, seed=65, std=0.3, page_size=16),
    "F": dict(raw=RAW_F, seed=66, std=0.2, page_size=8),
}
# A wide one: the products' tensor-core paths, windows of many key tiles, a latent of 256.
RAW_WIDE = model(3000, 1024, 1e-5, 0.5, (0, 2, 2), [
    (latent(16, 64, 32, 64, 256, 384, 0.1, 1.0e6, (16.0, 128, 24.0, 2.0)), dense(2048, 7.0)),
    (windowed(16, 4, 64, 64, 0.125, 300), moe(8, 2, 512)),
    (rotary(16, 2, 128, 128, 0.09, 64, 20000.0, (8.0, 2.0, 6.0, 256)), dense(1024, 2.0)),
])
WIDE = dict(raw=RAW_WIDE, seed=71, std=0.03, page_size=16)


def write_tiny(name: str, root: str) -> str:
    """A model folder of random weights.  Sinks are spread over a few units on both sides of zero (so that some
    heads lose much of their weight to the sink and some hardly any), the projections' biases likewise, the rows
    added ahead of a pass are of the stream's own size, and the gates' weights are scaled up so that gates close
    and open."""
    from safetensors.torch import load_file, save_file

    t = WIDE if name == "WIDE" else TINY[name]
    out = os.path.join(root, f"soporax_{name}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_model_folder(SoporaxConfig.from_dict(t["raw"]), t["seed"], out, std=t["std"], norm_affine="random")
        path = os.path.join(out, "model.safetensors")
        tensors = load_file(path)
        g = torch.Generator().manual_seed(t["seed"])
        for key in sorted(tensors):
            old = tensors[key]
            if key.endswith("mix.sink"):
                tensors[key] = (torch.randn(old.shape, generator=g) * 2.0).to(old.dtype)
            elif key.endswith((".q.b", ".k.b", ".v.b")):
                tensors[key] = torch.randn(old.shape, generator=g).to(old.dtype)
            elif key == "loop.step":
                tensors[key] = (torch.randn(old.shape, generator=g) * t["std"] * 2.0).to(old.dtype)
            elif key.endswith("mix.g"):
                tensors[key] = (old.float() * 4.0).to(old.dtype)
        save_file(tensors, path)
    return out


def load_folder(folder: str):
    """The configuration as a dict and the tensors in float64 (integer tables as they are)."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: (v.double() if v.is_floating_point() else v)
                 for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
