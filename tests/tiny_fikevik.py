"""Small Fikevik configurations for the tests, and helpers to write them as model folders.

They differ from one another in every size and constant and in the order of their layers, and avoid
coincidences: key and value sizes differ, heads of the two mixers of a layer differ in number, one to seven
query heads a key/value head, turned entries fewer than the key size or all of it, odd key and value sizes,
windows of 1, of a few keys, of more than a page, of more than any prompt, or none; stream weights and
result weights around and away from 1; layers without a feed-forward; layers that run another layer's
tensors (also through a second such layer) with a cache and state of their own; a model without attention and
one without linear attention.
"""
from __future__ import annotations

import json
import os

import torch

from rosellm_b200.config.fikevik import FikevikConfig
from rosellm_b200.weights import write_model_folder


def gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}}


def side(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def left(heads, kv_heads, dim, vdim, scale, window, rot):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        out["mask"] = {"size": window}
    if rot is not None:
        out["rot"] = {"dims": rot[0], "base": rot[1]}
    return out


def right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def again(j):
    """A layer that runs layer ``j``'s tensors."""
    return ("weights_of", j)


def model(vocab, width, eps, emb_scale, alpha, layers):
    out = []
    for mixer, mlp in layers:
        if isinstance(mixer, tuple) and mixer[0] == "weights_of":
            j = mixer[1]
            out.append(dict(out[j], weights_of=j))
        else:
            out.append(dict(mixer, mlp=mlp))
    return {"architecture": "Fikevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb_scale},
            "postln_alpha": alpha, "layers": out}


RAW_A = model(131, 64, 1e-5, 3.0, 2.25, [
    (gla(3, 24, 10, 4.0, 5), dense(100)),
    (side(left(6, 2, 20, 12, 0.3, 7, (12, 10000.0)), right(3, 8, 20, 5.0), 0.7, 1.3), None),
    (again(0), None),
    (again(1), None),
    (gla(2, 8, 40, 1.0, 3), dense(36)),
])
RAW_B = model(300, 96, 1e-6, 1.0, 1.0, [
    (side(left(4, 4, 64, 32, 0.125, 1000, (64, 500.0)), right(2, 64, 16, 30.0), 1.0, 1.0), dense(72)),
    (side(left(2, 2, 24, 72, 0.2, 1, (2, 77.0)), right(5, 12, 24, 2.0), 2.0, 0.25), None),
    (gla(2, 64, 16, 7.5, 16), None),
    (again(1), None),
    (again(3), None),          # through a layer that itself runs another's tensors
])
RAW_C = model(77, 48, 1e-4, 0.5, 3.0, [
    (side(left(7, 1, 9, 5, 0.35, 33, (8, 33.0)), right(1, 40, 9, 8.0), 0.9, 0.4), dense(20)),
    (gla(1, 16, 40, 2.0, 40), dense(24)),
    (side(left(40, 1, 8, 8, 0.4, 16, None), right(4, 6, 10, 12.0), 1.2, 1.1), None),
    (side(left(3, 3, 16, 24, 0.25, None, (16, 1.0e6)), right(2, 16, 16, 4.0), 0.5, 2.0), dense(16)),
])
RAW_D = model(2000, 384, 1e-5, 20.0, 2.5, [
    (side(left(12, 4, 48, 80, 0.14, 100, (32, 300000.0)), right(6, 32, 96, 15.0), 0.8, 1.2), dense(640)),
    (gla(6, 64, 96, 16.0, 24), dense(512)),
    (again(0), None),
    (gla(3, 96, 136, 32.0, 8), None),
    (again(1), None),
    (side(left(2, 1, 136, 130, 0.09, 48, (136, 10000.0)), right(3, 130, 40, 6.0), 1.5, 0.6), dense(96)),
])
# no attention at all (state slots only, no pages), and no linear attention
RAW_E = model(90, 40, 1e-5, 2.0, 2.0, [
    (gla(5, 8, 8, 3.0, 2), dense(16)),
    (gla(2, 20, 6, 9.0, 6), None),
    (again(0), None),
])
RAW_F = model(64, 56, 1e-5, 6.0, 0.5, [
    (side(left(7, 7, 10, 6, 0.33, 5, (6, 50.0)), right(7, 10, 6, 3.0), 1.0, 0.3), None),
    (side(left(8, 2, 6, 12, 0.4, 64, (6, 9.0)), right(2, 24, 5, 10.0), 0.3, 1.0), dense(40)),
    (again(0), None),
])
TINY = {
    "A": dict(raw=RAW_A, seed=41, std=0.2, page_size=16),
    "B": dict(raw=RAW_B, seed=42, std=0.15, page_size=8),
    "C": dict(raw=RAW_C, seed=43, std=0.25, page_size=32),
    "D": dict(raw=RAW_D, seed=44, std=0.07, page_size=16),
    "E": dict(raw=RAW_E, seed=45, std=0.3, page_size=16),
    "F": dict(raw=RAW_F, seed=46, std=0.2, page_size=8),
}
# A wide one: the products' tensor-core paths, windows of many key tiles, states of 64 and 128 columns.
RAW_WIDE = model(3000, 1024, 1e-5, 30.0, 1.75, [
    (side(left(16, 4, 64, 64, 0.125, 300, (64, 250000.0)), right(8, 64, 128, 15.0), 0.8, 1.25), dense(2048)),
    (gla(8, 64, 128, 12.0, 16), dense(2048)),
    (again(0), None),
    (again(1), None),
])
WIDE = dict(raw=RAW_WIDE, seed=51, std=0.03, page_size=16)


def write_tiny(name: str, root: str) -> str:
    """A model folder of random weights.  The heads' temperatures are spread over (0.5, 2), the decays' and the
    gates' biases over a few units (so that some channels forget fast and some hardly, and the running maximum
    moves), the gates' logits scaled up so that their caps bind now and then."""
    from safetensors.torch import load_file, save_file

    t = WIDE if name == "WIDE" else TINY[name]
    out = os.path.join(root, f"fikevik_{name}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_model_folder(FikevikConfig.from_dict(t["raw"]), t["seed"], out, std=t["std"], norm_affine="random")
        path = os.path.join(out, "model.safetensors")
        tensors = load_file(path)
        g = torch.Generator().manual_seed(t["seed"])
        for key in sorted(tensors):
            old = tensors[key]
            if key.endswith("left.temp"):
                tensors[key] = (0.5 + 1.5 * torch.rand(old.shape, generator=g)).to(old.dtype)
            elif key.endswith("mix.a2.b"):
                tensors[key] = (1.0 + torch.randn(old.shape, generator=g) * 2.0).to(old.dtype)
            elif key.endswith(("right.i.b", "right.f.b")):
                tensors[key] = (torch.randn(old.shape, generator=g) * 2.0 + (2.0 if key.endswith("f.b") else 0.0)).to(old.dtype)
            elif key.endswith(("right.i", "right.f")):
                tensors[key] = (old.float() * 4.0).to(old.dtype)
            elif key.endswith((".rg1.b", ".rg2.b")):
                tensors[key] = torch.randn(old.shape, generator=g).to(old.dtype)
        save_file(tensors, path)
    return out


def load_folder(folder: str):
    """The configuration as a dict and the tensors in float64."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
