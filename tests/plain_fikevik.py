"""A plain, slow implementation of Fikevik: whole sequences, no cache, float64, one function per mechanism.

Written from the design's equations; shares no code with the package.  ``cfg`` is the parsed ``config.json``
(a dict), ``w`` maps tensor names to float64 torch tensors.

Notation: ``x`` the stream [tokens, width]; ``unit(y) = y / sqrt(mean(y^2) + eps)`` over the last dimension.
A layer: ``x <- unit(alpha x + sigmoid(W_rg1 x + b_rg1) * mixer(x)) * w_1`` and, where it has a feed-forward,
``x <- unit(alpha x + sigmoid(W_rg2 x + b_rg2) * ff(x)) * w_2``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def embed(table: torch.Tensor, tokens, scale: float) -> torch.Tensor:
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def rotate_pairs(y: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """y [tokens, heads, dim]: entries (2i, 2i+1), i < dims/2, turned by position * base^(-2i/dims)."""
    out = y.clone()
    for i in range(dims // 2):
        ang = positions.to(F64) * float(base) ** (-2.0 * i / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = y[..., 2 * i], y[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def windowed_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Softmax attention over the last ``mask.size`` positions, grouped key/value heads, normed and
    rotated queries and keys, unit values, a temperature per head."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, G, dk)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q = unit(q, eps) * w[p + "q.norm"]
    k = unit(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    q = rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"])
    v = unit(v, eps)
    out = torch.zeros(T, H, dv, dtype=F64)
    size = m["mask"]["size"]
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] * w[p + "temp"][hd]
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        seen = (i - j >= 0) & (i - j < size)
        s = s.masked_fill(~seen, -math.inf)
        out[:, hd] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def matrix_memory(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """A matrix memory with exponential input gate and a running maximum that starts at zero."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    S = torch.zeros(H, dk, dv, dtype=F64)
    n = torch.zeros(H, dk, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        keep = torch.exp(gf[t] + mx - m_new)
        take = torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    o = unit(out, eps).reshape(T, H * dv) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def decayed_linear_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """S_t = diag(a_t) S_(t-1) + k_t v_t^T with a_t = sigmoid(z_t)^(1/tau) per key channel; o_t = S_t^T q_t."""
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = ((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]).view(T, H, dk)
    a = torch.sigmoid(z) ** (1.0 / tau)
    S = torch.zeros(H, dk, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = (unit(out, eps) * w[p + "norm"]).reshape(T, H * dv)
    g = h @ w[p + "g"].T
    return (o * g * torch.sigmoid(g)) @ w[p + "o"].T


def side_by_side(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    left = windowed_attention(h, w, p + "left.", m["left"], eps)
    right = matrix_memory(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def gated_feed_forward(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def sublayer_join(x: torch.Tensor, y: torch.Tensor, w: dict, gate: str, norm: str, alpha: float, eps: float) -> torch.Tensor:
    """unit(alpha x + sigmoid(W x + b) * y) * w_norm: the gate reads what the sublayer read."""
    g = torch.sigmoid(x @ w[gate].T + w[gate + ".b"])
    return unit(alpha * x + g * y, eps) * w[norm]


MIXERS = {"gla": decayed_linear_attention, "parallel": side_by_side}


def layer(x: torch.Tensor, w: dict, cfg: dict, i: int) -> torch.Tensor:
    lc = cfg["layers"][i]
    p = f"l{lc.get('weights_of', i)}."
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    y = MIXERS[lc["type"]](x, w, p + "mix.", lc["mixer"], eps)
    x = sublayer_join(x, y, w, p + "rg1", p + "norm1", alpha, eps)
    if lc.get("mlp") is not None:
        y = gated_feed_forward(x, w, p + "mlp.")
        x = sublayer_join(x, y, w, p + "rg2", p + "norm2", alpha, eps)
    return x


def forward(cfg: dict, w: dict, tokens, streams: list | None = None) -> torch.Tensor:
    """Logits [tokens, vocab] of one sequence; ``streams`` (a list) receives the stream after every layer."""
    x = embed(w["embed"], tokens, cfg["embedding"]["scale"])
    for i in range(len(cfg["layers"])):
        x = layer(x, w, cfg, i)
        if streams is not None:
            streams.append(x.clone())
    x = unit(x, cfg["norm"]["eps"]) * w["final.norm"]
    return x @ w["head"].T
