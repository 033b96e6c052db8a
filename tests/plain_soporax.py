"""A plain, slow implementation of Soporax: whole sequences, no cache, one function per mechanism.

Written from the design's equations; shares no code with the package.  ``cfg`` is the parsed ``config.json``
(a dict), ``w`` maps tensor names to torch tensors: float64 for the values the tests compare with; given float32
tensors everything is computed in float32, which shows how far rounding alone moves a result.

Notation: ``x`` the stream [tokens, width]; ``unit(y) = y / sqrt(mean(y^2) + eps)`` over the last dimension.
A layer reads ``h = unit(x) * w_1`` once and adds both sublayers' results: ``x <- x + mixer(h) + ff(h)``.
A stretch of layers may run several times in a row (each pass on its own keys); ahead of every pass but the first
the token rows as they entered the stack are added again, and ahead of every pass a learned row of the pass.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

F64 = torch.float64

# Where an engine that keeps activations in 16 bits rounds them (rows that matrix products read, cached keys,
# values and latents, the mixers' results ahead of their output products, inner rows of the feed-forwards): the
# identity, or a function that rounds, to see how far such rounding alone moves the logits of a sequence.
_round = lambda t: t


def to_bfloat16_and_back(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


def unit(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


# ---- rotation ---------------------------------------------------------------------------------------------

def plain_frequencies(dims: int, base: float) -> list[float]:
    return [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]


def wavelength_scaled(freqs: list[float], factor: float, low: float, high: float, original: float) -> list[float]:
    """Short waves stay, long waves are slowed by ``factor``, those between are blended by where
    ``original / wavelength`` lies between ``low`` and ``high``."""
    out = []
    for f in freqs:
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out.append(f)
        elif wave > original / low:
            out.append(f / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def ramp_scaled(freqs: list[float], dims: int, base: float, factor: float, original: float, fast: float,
                slow: float) -> tuple[list[float], float]:
    """A linear ramp over the pairs' indices between the pair that turns ``fast`` times within ``original``
    positions and the one that turns ``slow`` times: pairs below keep their frequency, pairs above are slowed by
    ``factor``.  Also the factor of the cosines and sines, 0.1 ln(factor) + 1."""
    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotation_constants(rot: dict) -> tuple[list[float], float]:
    """(frequency of every pair, factor of cosines and sines) from a mixer's ``rot`` entry."""
    dims, base = rot["dims"], rot["base"]
    freqs, mult = plain_frequencies(dims, base), 1.0
    sc = rot.get("scaling")
    if sc:
        if "fast" in sc or "slow" in sc:
            freqs, mult = ramp_scaled(freqs, dims, base, sc["factor"], sc["original"], sc["fast"], sc["slow"])
        else:
            freqs = wavelength_scaled(freqs, sc["factor"], sc["low"], sc["high"], sc["original"])
    return freqs, mult


def rotate_pairs(y: torch.Tensor, positions: torch.Tensor, freqs: list[float], mult: float = 1.0) -> torch.Tensor:
    """y [tokens, ..., dim]: entries (2i, 2i+1), i < len(freqs), turned by position * freqs[i]; cosines and
    sines times ``mult``."""
    out = y.clone()
    shape = [y.shape[0]] + [1] * (y.dim() - 2)
    for i, f in enumerate(freqs):
        ang = positions.to(y.dtype) * f
        c, s = (torch.cos(ang) * mult).view(shape), (torch.sin(ang) * mult).view(shape)
        a, b = y[..., 2 * i], y[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# ---- softmax attention ---------------------------------------------------------------------------------------

def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, size: int | None,
                      sink: torch.Tensor | None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]: query i sees the keys j with 0 <= i - j < size (``None``: all
    j <= i); query head h uses key/value head h // (H / G); score = q . k * scale.  ``sink`` [H]: one more term
    exp(sink_h) in the softmax's denominator, with no value."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (i - j >= 0) if size is None else (i - j >= 0) & (i - j < size)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = ((q[:, hd] @ k[:, g].T) * scale).masked_fill(~seen, -math.inf)
        if sink is None:
            p = torch.softmax(s, -1)
        else:
            top = torch.maximum(s.max(-1, keepdim=True).values, sink[hd].to(s.dtype))
            e = torch.exp(s - top)
            p = e / (e.sum(-1, keepdim=True) + torch.exp(sink[hd].to(s.dtype) - top))
        out[:, hd] = p @ v[:, g]
    return out


def window_sink_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """``attention``: no positions; queries and keys of unit root mean square per head; the latest ``mask.size``
    keys; a learned sink per head."""
    T, h = h.shape[0], _round(h)
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit((h @ w[p + "q"].T).view(T, H, dk), eps)
    k = unit((h @ w[p + "k"].T).view(T, G, dk), eps)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    size = m["mask"]["size"] if m.get("mask") else None
    out = softmax_attention(q, _round(k), _round(v), m["scale"], size, w[p + "sink"])
    return _round(out.reshape(T, H * dv)) @ w[p + "o"].T


def rotary_gated_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """``attention_2``: projections with biases, the first ``rot.dims`` entries of every head of q and k turned,
    all earlier keys, a sink of score 0, and a gate per head on the heads' results."""
    T, h = h.shape[0], _round(h)
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    pos = torch.arange(T)
    if m.get("rot"):
        freqs, mult = rotation_constants(m["rot"])
        q, k = rotate_pairs(q, pos, freqs, mult), rotate_pairs(k, pos, freqs, mult)
    out = softmax_attention(q, _round(k), _round(v), m["scale"], None, torch.zeros(H, dtype=h.dtype))
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, H]
    out = out * gate[:, :, None]
    return _round(out.reshape(T, H * dv)) @ w[p + "o"].T


def latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Queries through a normed latent; one normed key/value latent and one turned key part a token, shared by
    the heads; per head a plain key part and a value projected from the latent; a plain softmax over all earlier
    keys; an element-wise gate on the merged heads."""
    T, h = h.shape[0], _round(h)
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    if m.get("q_rank") is None:  # a model may leave the queries' latent out
        q = (h @ w[p + "q"].T).view(T, H, dn + dr)
    else:
        cq = _round(unit(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"])
        q = (cq @ w[p + "uq"].T).view(T, H, dn + dr)
    dkv = h @ w[p + "dkv"].T
    c = _round(unit(dkv[:, :rank], eps) * w[p + "dkv.norm"])
    k_rot = dkv[:, rank:]
    pos = torch.arange(T)
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    rot = dict(m["rot"], dims=dr) if m.get("rot") else None
    if rot:
        freqs, mult = rotation_constants(rot)
        q_rot = rotate_pairs(q_rot, pos, freqs, mult)
        k_rot = rotate_pairs(k_rot, pos, freqs, mult)
    k_rot = _round(k_rot)
    k_plain = (c @ w[p + "uk"].T).view(T, H, dn)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out[:, hd] = torch.softmax(s.masked_fill(j > i, -math.inf), -1) @ v[:, hd]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return _round(out) @ w[p + "o"].T


MIXERS = {"attention": window_sink_attention, "attention_2": rotary_gated_attention,
          "latent_attention": latent_attention}


# ---- feed-forwards ---------------------------------------------------------------------------------------------

def clamped_dense(h: torch.Tensor, w: dict, p: str, limit: float) -> torch.Tensor:
    h = _round(h)
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return _round(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def silu_expert(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    g = h @ w[p + "gate"].T
    return _round(g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def table_experts(h: torch.Tensor, tokens, w: dict, p: str, top: int) -> torch.Tensor:
    """Every token's experts come from a table by its id; each counts 1 / top."""
    h = _round(h)
    out = torch.zeros_like(h)
    table = w[p + "table"]
    for t, tok in enumerate(tokens):
        for c in range(top):
            e = int(table[int(tok), c])
            out[t] += silu_expert(h[t:t + 1], w, f"{p}e{e}.")[0] / top
    return out


def feed_forward(h: torch.Tensor, tokens, w: dict, p: str, mlp: dict | None) -> torch.Tensor:
    if mlp is None:
        return torch.zeros_like(h)
    if mlp["kind"] == "dense":
        return clamped_dense(h, w, p, mlp["limit"])
    return table_experts(h, tokens, w, p, mlp["router"]["top"])


# ---- the model --------------------------------------------------------------------------------------------------

def layer(x: torch.Tensor, tokens, w: dict, i: int, lc: dict, eps: float) -> torch.Tensor:
    h = unit(x, eps) * w[f"l{i}.norm1"]
    return x + (MIXERS[lc["type"]](h, w, f"l{i}.mix.", lc["mixer"], eps) + feed_forward(h, tokens, w, f"l{i}.mlp.", lc.get("mlp")))


def run_order(cfg: dict) -> list[tuple[int, int | None]]:
    """(layer, pass) in the order they run; pass ``None`` outside the repeated stretch, else the pass's number
    at its first layer and -1 at its others."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t if i == loop["start"] else -1) for i in range(loop["start"], loop["stop"])]
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, w: dict, tokens, rounding=None, streams: list | None = None) -> torch.Tensor:
    """Logits [tokens, vocab] of one sequence.  ``streams`` (a list) receives the stream after every run of a
    layer."""
    global _round
    keep, _round = _round, (rounding or (lambda t: t))
    try:
        eps = cfg["norm"]["eps"]
        x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        x = x0.clone()
        for i, t in run_order(cfg):
            if t is not None and t >= 0:
                if t > 0:
                    x = x + x0
                x = x + w["loop.step"][t]
            x = layer(x, tokens, w, i, cfg["layers"][i], eps)
            if streams is not None:
                streams.append(x.clone())
        h = _round(unit(x, eps) * w["final.norm"])
        return (h @ w["embed"].T) * cfg.get("logit_scale", 1.0)
    finally:
        _round = keep


# ---- model folders ------------------------------------------------------------------------------------------------

_DTYPES = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "I32": (torch.int32, 4),
           "I64": (torch.int64, 8)}


def read_safetensors(path: str) -> dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        dt, _ = _DTYPES[m["dtype"]]
        a, b = m["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=dt).reshape(m["shape"]).clone()
    return out


def load_folder(folder: str, dtype: torch.dtype = F64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in
         read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w
