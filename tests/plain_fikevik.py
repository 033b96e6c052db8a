"""A plain, slow implementation of Fikevik: whole sequences, no cache, one function per mechanism.

Written from the design's equations; shares no code with the package.  ``cfg`` is the parsed ``config.json``
(a dict), ``w`` maps tensor names to torch tensors: float64 for the values the tests compare with; given float32
tensors everything is computed in float32, which shows how far rounding alone moves a result.

Notation: ``x`` the stream [tokens, width]; ``unit(y) = y / sqrt(mean(y^2) + eps)`` over the last dimension.
A layer: ``x <- unit(alpha x + sigmoid(W_rg1 x + b_rg1) * mixer(x)) * w_1`` and, where it has a feed-forward,
``x <- unit(alpha x + sigmoid(W_rg2 x + b_rg2) * ff(x)) * w_2``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64

# Where an engine that keeps activations in 16 bits rounds them (the rows that matrix products read, cached keys
# and values, the mixers' results ahead of their output products, the feed-forward's inner rows): the identity,
# or a function that rounds, to see how far such rounding alone moves the logits of a sequence.
_round = lambda t: t


def to_bfloat16_and_back(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


def unit(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def embed(table: torch.Tensor, tokens, scale: float) -> torch.Tensor:
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def rotate_pairs(y: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """y [tokens, heads, dim]: entries (2i, 2i+1), i < dims/2, turned by position * base^(-2i/dims)."""
    out = y.clone()
    for i in range(dims // 2):
        ang = positions.to(y.dtype) * float(base) ** (-2.0 * i / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = y[..., 2 * i], y[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def window_softmax(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, temp: torch.Tensor,
                   size: int | None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]: query i sees the keys j with 0 <= i - j < size (``None``: all
    j <= i); query head h uses key/value head h // (H / G); score = q . k * scale * temp[h]."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (i - j >= 0) if size is None else (i - j >= 0) & (i - j < size)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale * temp[hd]
        out[:, hd] = torch.softmax(s.masked_fill(~seen, -math.inf), -1) @ v[:, g]
    return out


def windowed_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Softmax attention over the last ``mask.size`` positions, grouped key/value heads, normed and
    rotated queries and keys, unit values, a temperature per head."""
    T, h = h.shape[0], _round(h)
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, G, dk)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q = unit(q, eps) * w[p + "q.norm"]
    k = unit(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    if m.get("rot"):
        q = rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"])
    out = window_softmax(q, _round(k), _round(unit(v, eps)), m["scale"], w[p + "temp"], m["mask"]["size"] if m.get("mask") else None)
    return _round(out.reshape(T, H * dv)) @ w[p + "o"].T


def capped_log_gates(zi: torch.Tensor, zf: torch.Tensor, cap: float):
    """The logarithms of the input and forget gates from their logits: cap * tanh(z / cap), the forget gate's
    through a log-sigmoid."""
    return cap * torch.tanh(zi / cap), torch.nn.functional.logsigmoid(cap * torch.tanh(zf / cap))


def memory_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gi: torch.Tensor, gf: torch.Tensor,
                      floor: float = 1e-6) -> torch.Tensor:
    """q, k [T, H, dk], v [T, H, dv], log gates gi, gf [T, H].  S, n and the running maximum m start at zero:
    m_t = max(gf + m, gi); S_t = e^(gf + m - m_t) S + e^(gi - m_t) k v^T; n_t likewise with k;
    o_t = S_t^T q / (max(|n_t . q|, e^(-m_t)) + floor)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    n = torch.zeros(H, dk, dtype=q.dtype)
    mx = torch.zeros(H, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        keep = torch.exp(gf[t] + mx - m_new)
        take = torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + floor
        out[t] = num / den[:, None]
    return out


def decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """q, k, a [T, H, dk], v [T, H, dv]: S_t = diag(a_t) S_(t-1) + k_t v_t^T from S = 0; o_t = S_t^T q_t."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def matrix_memory(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """A matrix memory with exponential input gate and a running maximum that starts at zero."""
    T, h = h.shape[0], _round(h)
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    gi, gf = capped_log_gates(h @ w[p + "i"].T + w[p + "i.b"], h @ w[p + "f"].T + w[p + "f.b"], cap)
    out = memory_recurrence(q, k, v, gi, gf)
    o = unit(out, eps).reshape(T, H * dv) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return _round(o) @ w[p + "o"].T


def decayed_linear_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention whose state forgets per key channel: a_t = sigmoid(z_t)^(1/tau), z through a low rank."""
    T, h = h.shape[0], _round(h)
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = ((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]).view(T, H, dk)
    out = decay_recurrence(q, k, v, torch.sigmoid(z) ** (1.0 / tau))
    o = (unit(out, eps) * w[p + "norm"]).reshape(T, H * dv)
    g = h @ w[p + "g"].T
    return _round(o * g * torch.sigmoid(g)) @ w[p + "o"].T


def side_by_side(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    left = windowed_attention(h, w, p + "left.", m["left"], eps)
    right = matrix_memory(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def gated_feed_forward(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    h = _round(h)
    g = h @ w[p + "gate"].T
    return _round(g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def sublayer_join(x: torch.Tensor, y: torch.Tensor, w: dict, gate: str, norm: str, alpha: float, eps: float) -> torch.Tensor:
    """unit(alpha x + sigmoid(W x + b) * y) * w_norm: the gate reads what the sublayer read."""
    g = torch.sigmoid(_round(x) @ w[gate].T + w[gate + ".b"])
    return unit(alpha * x + g * y, eps) * w[norm]


MIXERS = {"gla": decayed_linear_attention, "parallel": side_by_side}


def layer(x: torch.Tensor, w: dict, cfg: dict, i: int) -> torch.Tensor:
    lc, owner = cfg["layers"][i], i
    while cfg["layers"][owner].get("weights_of") is not None:  # a layer that runs another layer's tensors
        owner = cfg["layers"][owner]["weights_of"]
    p = f"l{owner}."
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    y = MIXERS[lc["type"]](x, w, p + "mix.", lc["mixer"], eps)
    x = sublayer_join(x, y, w, p + "rg1", p + "norm1", alpha, eps)
    if lc.get("mlp") is not None:
        y = gated_feed_forward(x, w, p + "mlp.")
        x = sublayer_join(x, y, w, p + "rg2", p + "norm2", alpha, eps)
    return x


def forward(cfg: dict, w: dict, tokens, streams: list | None = None, rounding=None) -> torch.Tensor:
    """Logits [tokens, vocab] of one sequence; ``streams`` (a list) receives the stream after every layer.
    ``rounding`` (``to_bfloat16_and_back``): applied where a 16-bit engine stores activations."""
    global _round
    keep, _round = _round, rounding or (lambda t: t)
    try:
        x = embed(w["embed"], tokens, cfg["embedding"]["scale"])
        for i in range(len(cfg["layers"])):
            x = layer(x, w, cfg, i)
            if streams is not None:
                streams.append(x.clone())
        x = unit(x, cfg["norm"]["eps"]) * w["final.norm"]
        return _round(x) @ w["head"].T
    finally:
        _round = keep
