"""Mixers that keep a matrix-valued state per request and head instead of a cache of keys.

Both forms run one recurrence, ``S_t = diag(w_t) S_(t-1) [- (a_t * u_t)(u_t^T S_(t-1))] + k_t v_t^T`` and
``o_t = S_t^T r_t``, on the kernels of csrc/recurrent.cu: the state is float32 ``[heads, key size, value
size]`` in the request's state slot (zero when the slot is taken), a step continues it for however many
tokens the request brings, and everything between the projections and the output product is float32.

All projections of the layer's input are one product: the weights are packed at bind time (each
tensor's rows filled up to a multiple of 8) and the product writes float32, so the recurrence reads
unrounded projections in both precisions.
"""
from __future__ import annotations

import math

import torch

from ..ops import kernels as K
from .base import ParamSpec, Part, StateSpec, register_part


def pack_rows(tensors: list[torch.Tensor]) -> tuple[torch.Tensor, list[int]]:
    """The tensors stacked along dimension 0, each starting at a multiple of 8 rows (rows of zeros in
    between), and every tensor's first row."""
    parts, offsets, at = [], [], 0
    for t in tensors:
        offsets.append(at)
        parts.append(t)
        fill = -t.shape[0] % 8
        if fill:
            parts.append(t.new_zeros((fill, t.shape[1])))
        at += t.shape[0] + fill
    return torch.cat(parts).contiguous(), offsets


class _StateMixer(Part):
    graph_safe = True
    launches_replayable = True

    def _project(self, ctx, h, proj=None):
        """The packed projections of the layer's input, float32 [tokens, rows of ``proj_weight``]: computed here,
        or (``proj``) handed in by a block that multiplies several parts' packed weights in one product."""
        if proj is not None:
            return proj
        proj = ctx.workspace.get("mixer_proj", (ctx.n_tokens, self.proj_weight.shape[0]), torch.float32)
        K.linear(h, self.proj_weight, None, proj)
        return proj

    def _out_buffer(self, ctx):
        """The recurrence's output in the activation dtype, its rows filled up to a multiple of 8 entries
        for the output product (the fill stays zero: the buffer is zeroed when made, is named by its
        widths, and no kernel writes the fill)."""
        real, padded = self.out_width, self.out_padded
        if real == padded:
            return ctx.workspace.get("state_mixer_out", (ctx.n_tokens, padded), ctx.act_dtype), None
        buf = ctx.workspace.get_zeroed(f"state_mixer_out_{real}_{padded}", (ctx.n_tokens, padded), ctx.act_dtype)
        return buf, buf[:, :real]

    def _scratch(self, ctx, mode: int, dk: int, dv: int):
        n = ctx.n_tokens
        prep = ctx.workspace.get("state_mixer_prep", (self.num_heads * n * K.recurrence_record(mode, dk, dv),), torch.float32)
        oraw = ctx.workspace.get("state_mixer_raw", (n, self.num_heads * dv), torch.float32)
        return prep, oraw

    def _pad_out_weight(self) -> None:
        self.out_padded = -(-self.out_width // 8) * 8
        if self.out_padded != self.out_width:
            self.out_weight = torch.nn.functional.pad(self.out_weight, (0, self.out_padded - self.out_width)).contiguous()


@register_part("mixer", "delta_rule")
class DeltaRuleMixer(_StateMixer):
    """The generalized delta rule.  ``r, k, v = W_r h, W_k h, W_v h`` (heads x dim each); per head and key
    channel a decay ``w = exp(-decay_scale * sigmoid(w0 + W_w2 tanh(W_w1 h)))`` and a removal rate
    ``a = sigmoid(W_a h + a_bias)``; with the unit key ``u = k / sqrt(sum k^2 + unit_eps)``:
    ``S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T`` (decay and removal both act on ``S_(t-1)``) and
    ``o_t = S_t^T r``.  Each head's ``o`` is divided by its root mean square (``norm_eps``), multiplied by
    ``out_norm`` (one entry per head and column) and by ``sigmoid(W_g h)``, then ``W_o``.
    ``low_rank``: the inner size of the decay's projection; ``None`` takes it from the bound tensors."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, norm_eps: float, low_rank: int | None = None,
                 decay_scale: float = math.exp(-0.5), unit_eps: float = 1e-6) -> None:
        if head_dim > 256:
            raise ValueError(f"delta rule: head size {head_dim}: the state kernel takes up to 256")
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.norm_eps, self.low_rank = float(norm_eps), low_rank
        self.decay_scale, self.unit_eps = float(decay_scale), float(unit_eps)
        self.width = self.out_width = num_heads * head_dim
        self.out_padded = -(-self.out_width // 8) * 8
        self.proj_weight = self.out_weight = None

    def param_specs(self):
        w, hid, rank = self.width, self.hidden_size, -1 if self.low_rank is None else self.low_rank
        return [ParamSpec("r_weight", (w, hid)), ParamSpec("k_weight", (w, hid)), ParamSpec("v_weight", (w, hid)),
                ParamSpec("a_weight", (w, hid)), ParamSpec("g_weight", (w, hid)), ParamSpec("w1_weight", (rank, hid)),
                ParamSpec("w2_weight", (w, rank), kind="vector"), ParamSpec("a_bias", (w,), kind="vector", init="zeros"),
                ParamSpec("w0", (w,), kind="vector", init="zeros"), ParamSpec("out_norm", (w,), kind="vector", init="ones"),
                ParamSpec("out_weight", (hid, w))]

    def state_spec(self):
        return StateSpec((self.num_heads, self.head_dim, self.head_dim), torch.float32)

    def bind(self, tensors) -> None:
        t = dict(tensors)
        rank = t["w1_weight"].shape[0]
        if t["w2_weight"].shape[1] != rank or (self.low_rank is not None and rank != self.low_rank):
            raise ValueError(f"delta rule: the decay's two matrices disagree on their inner size "
                             f"({t['w1_weight'].shape[0]} and {t['w2_weight'].shape[1]})")
        self.rank = rank
        names = ("r", "k", "v", "a", "g", "w")
        self.proj_weight, offs = pack_rows([t[n + "_weight"] for n in ("r", "k", "v", "a", "g", "w1")])
        self.offsets = dict(zip(names, offs))
        self.w2t_weight = t["w2_weight"].t().contiguous()  # [rank, channels]: the kernel's threads walk the channels
        self.a_bias, self.w0, self.out_norm = t["a_bias"], t["w0"], t["out_norm"]
        self.out_weight = t["out_weight"]
        self._pad_out_weight()

    def forward(self, ctx, run, h, x, add: bool = True) -> None:
        proj = self._project(ctx, h)
        buf, view = self._out_buffer(ctx)
        mode = K.RECURRENCES["delta"]
        prep, oraw = self._scratch(ctx, mode, self.head_dim, self.head_dim)
        K.recurrence(mode, proj, self.offsets, ctx.state(run.state_key), buf if view is None else view,
                     ctx.q_start, ctx.slots, prep, oraw, n_reqs=ctx.n_reqs, n_heads=self.num_heads, dk=self.head_dim,
                     dv=self.head_dim, eps=self.norm_eps, a_bias=self.a_bias, w0=self.w0, out_weight=self.out_norm,
                     w2t=self.w2t_weight, rank=self.rank, decay_scale=self.decay_scale, unit_eps=self.unit_eps)
        K.linear(buf, self.out_weight, None, x, residual=add)


@register_part("mixer", "gated_recurrence")
class GatedRecurrenceMixer(_StateMixer):
    """A linear recurrence with one gate for forgetting and writing: what a channel does not keep, it takes from the value.  ``q = silu(W_q h)`` (heads x
    key_dim), ``v = W_v h`` (heads x value_dim), ``f = l + (1 - l) * sigmoid(W_f h + f_bias)`` with the lower
    bound ``l`` per head and key channel; ``S_t = diag(f) S_(t-1) + (1 - f) v^T``, ``o_t = S_t^T q``.  Each
    head's ``o`` is RMS-normed over value_dim with a weight the heads share (``norm_eps``), then ``W_o``."""

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, norm_eps: float) -> None:
        if key_dim > 256 or value_dim > 256:
            raise ValueError(f"gated recurrence: sizes {key_dim} / {value_dim}: the state kernel takes up to 256")
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = hidden_size, num_heads, key_dim, value_dim
        self.norm_eps = float(norm_eps)
        self.key_width, self.out_width = num_heads * key_dim, num_heads * value_dim
        self.out_padded = -(-self.out_width // 8) * 8
        self.proj_weight = self.out_weight = None

    def param_specs(self):
        kw, vw, hid = self.key_width, self.out_width, self.hidden_size
        return [ParamSpec("q_weight", (kw, hid)), ParamSpec("f_weight", (kw, hid)), ParamSpec("v_weight", (vw, hid)),
                ParamSpec("f_bias", (kw,), kind="vector", init="zeros"), ParamSpec("lower", (kw,), kind="vector", init="zeros"),
                ParamSpec("out_norm", (self.value_dim,), kind="vector", init="ones"), ParamSpec("out_weight", (hid, vw))]

    def state_spec(self):
        return StateSpec((self.num_heads, self.key_dim, self.value_dim), torch.float32)

    def bind(self, tensors) -> None:
        t = dict(tensors)
        self.proj_weight, offs = pack_rows([t["q_weight"], t["f_weight"], t["v_weight"]])
        self.offsets = dict(zip(("r", "a", "v"), offs))
        self.f_bias, self.lower, self.out_norm, self.out_weight = t["f_bias"], t["lower"], t["out_norm"], t["out_weight"]
        self._pad_out_weight()

    def forward(self, ctx, run, h, x, add: bool = True) -> None:
        proj = self._project(ctx, h)
        buf, view = self._out_buffer(ctx)
        mode = K.RECURRENCES["gated"]
        prep, oraw = self._scratch(ctx, mode, self.key_dim, self.value_dim)
        K.recurrence(mode, proj, self.offsets, ctx.state(run.state_key), buf if view is None else view,
                     ctx.q_start, ctx.slots, prep, oraw, n_reqs=ctx.n_reqs, n_heads=self.num_heads, dk=self.key_dim,
                     dv=self.value_dim, eps=self.norm_eps, a_bias=self.f_bias, w0=self.lower, out_weight=self.out_norm)
        K.linear(buf, self.out_weight, None, x, residual=add)


@register_part("mixer", "decayed_linear_attention")
class DecayedLinearAttention(_StateMixer):
    """Linear attention whose state forgets per key channel.  ``q = W_q h * query_scale`` (``None``:
    key_dim^(-1/2)), ``k = W_k h`` (heads x key_dim), ``v = W_v h`` (heads x value_dim); a decay per head and key
    channel ``a = sigmoid(z)^(1/tau)`` with ``z = W_a2 (W_a1 h) + a_bias``, a projection through a low rank with
    no function in between; ``S_t = diag(a_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``.  Each head's ``o`` is
    RMS-normed over value_dim with a weight the heads share (``norm_eps``), the merged heads are multiplied by
    ``silu(W_g h)``, then ``W_o``.  ``low_rank``: the inner size of the decay's projection; ``None`` takes it
    from the bound tensors.  The decay is evaluated as ``exp(logsigmoid(z) / tau)`` in float32."""

    takes_projection = True  # forward(.., proj=): the input times ``proj_weight``, made by the caller

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, tau: float, norm_eps: float,
                 low_rank: int | None = None, query_scale: float | None = None) -> None:
        if key_dim > 256 or value_dim > 256:
            raise ValueError(f"decayed linear attention: sizes {key_dim} / {value_dim}: the state kernel takes up to 256")
        if tau <= 0:
            raise ValueError("decayed linear attention: tau must be positive")
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = hidden_size, num_heads, key_dim, value_dim
        self.tau, self.norm_eps, self.low_rank = float(tau), float(norm_eps), low_rank
        self.query_scale = float(key_dim) ** -0.5 if query_scale is None else float(query_scale)
        self.key_width, self.out_width = num_heads * key_dim, num_heads * value_dim
        self.out_padded = -(-self.out_width // 8) * 8
        self.proj_weight = self.out_weight = None

    def param_specs(self):
        kw, vw, hid, rank = self.key_width, self.out_width, self.hidden_size, -1 if self.low_rank is None else self.low_rank
        return [ParamSpec("q_weight", (kw, hid)), ParamSpec("k_weight", (kw, hid)), ParamSpec("v_weight", (vw, hid)),
                ParamSpec("g_weight", (vw, hid)), ParamSpec("a1_weight", (rank, hid)),
                ParamSpec("a2_weight", (kw, rank), kind="vector"), ParamSpec("a_bias", (kw,), kind="vector", init="zeros"),
                ParamSpec("out_norm", (self.value_dim,), kind="vector", init="ones"), ParamSpec("out_weight", (hid, vw))]

    def state_spec(self):
        return StateSpec((self.num_heads, self.key_dim, self.value_dim), torch.float32)

    def bind(self, tensors) -> None:
        t = dict(tensors)
        rank = t["a1_weight"].shape[0]
        if t["a2_weight"].shape[1] != rank or (self.low_rank is not None and rank != self.low_rank):
            raise ValueError(f"decayed linear attention: the decay's two matrices disagree on their inner size "
                             f"({t['a1_weight'].shape[0]} and {t['a2_weight'].shape[1]})")
        self.rank = rank
        self.proj_weight, offs = pack_rows([t[n + "_weight"] for n in ("q", "k", "v", "g", "a1")])
        self.offsets = dict(zip(("r", "k", "v", "g", "w"), offs))
        self.a2t_weight = t["a2_weight"].t().contiguous()  # [rank, channels]: the kernel's threads walk the channels
        self.a_bias, self.out_norm, self.out_weight = t["a_bias"], t["out_norm"], t["out_weight"]
        self._pad_out_weight()

    def forward(self, ctx, run, h, x, add: bool = True, proj=None) -> None:
        proj = self._project(ctx, h, proj)
        buf, view = self._out_buffer(ctx)
        mode = K.RECURRENCES["decayed_keys"]
        prep, oraw = self._scratch(ctx, mode, self.key_dim, self.value_dim)
        K.recurrence(mode, proj, self.offsets, ctx.state(run.state_key), buf if view is None else view,
                     ctx.q_start, ctx.slots, prep, oraw, n_reqs=ctx.n_reqs, n_heads=self.num_heads, dk=self.key_dim,
                     dv=self.value_dim, eps=self.norm_eps, a_bias=self.a_bias, w0=self.a_bias, out_weight=self.out_norm,
                     w2t=self.a2t_weight, rank=self.rank, tau=self.tau, qscale=self.query_scale)
        K.linear(buf, self.out_weight, None, x, residual=add)


@register_part("mixer", "matrix_memory")
class MatrixMemory(_StateMixer):
    """A matrix memory with an exponential input gate, kept in range by a running maximum.  ``q = W_q h *
    query_scale`` (``None``: key_dim^(-1/2)), ``k = W_k h`` (heads x key_dim), ``v = W_v h`` (heads x value_dim);
    per head the log gates ``i = cap * tanh((W_i h + i_bias) / cap)`` and ``f = logsigmoid(cap * tanh((W_f h +
    f_bias) / cap))`` (``gate_cap``).  With ``m_0 = 0``, ``S_0 = 0``, ``n_0 = 0``:

        m_t = max(f + m_(t-1), i);  S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T;  n_t likewise with k alone
        o_t = S_t^T q / (max(|n_t . q|, e^(-m_t)) + floor_eps)

    Each head's ``o`` is divided by its root mean square (``norm_eps``); the merged heads are multiplied by
    ``out_norm`` (one entry per head and column) and by ``sigmoid(W_g h)``, then ``W_o``.

    The state slot holds, per head, the matrix with the normaliser as one more column ([key_dim, value_dim +
    1]: n obeys S's recurrence with a value of 1), and behind all matrices the heads' running maxima."""

    takes_projection = True  # forward(.., proj=): the input times ``proj_weight``, made by the caller

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, gate_cap: float, norm_eps: float,
                 floor_eps: float = 1e-6, query_scale: float | None = None) -> None:
        if key_dim > 256 or value_dim > 256:
            raise ValueError(f"matrix memory: sizes {key_dim} / {value_dim}: the state kernel takes up to 256")
        if gate_cap <= 0:
            raise ValueError("matrix memory: the gates' cap must be positive")
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = hidden_size, num_heads, key_dim, value_dim
        self.gate_cap, self.norm_eps, self.floor_eps = float(gate_cap), float(norm_eps), float(floor_eps)
        self.query_scale = float(key_dim) ** -0.5 if query_scale is None else float(query_scale)
        self.key_width, self.out_width = num_heads * key_dim, num_heads * value_dim
        self.out_padded = -(-self.out_width // 8) * 8
        self.proj_weight = self.out_weight = None

    def param_specs(self):
        kw, vw, hid, H = self.key_width, self.out_width, self.hidden_size, self.num_heads
        return [ParamSpec("q_weight", (kw, hid)), ParamSpec("k_weight", (kw, hid)), ParamSpec("v_weight", (vw, hid)),
                ParamSpec("g_weight", (vw, hid)), ParamSpec("i_weight", (H, hid)), ParamSpec("f_weight", (H, hid)),
                ParamSpec("i_bias", (H,), kind="vector", init="zeros"), ParamSpec("f_bias", (H,), kind="vector", init="zeros"),
                ParamSpec("out_norm", (vw,), kind="vector", init="ones"), ParamSpec("out_weight", (hid, vw))]

    def state_spec(self):
        return StateSpec((self.num_heads * self.key_dim * (self.value_dim + 1) + self.num_heads,), torch.float32)

    def bind(self, tensors) -> None:
        t = dict(tensors)
        self.proj_weight, offs = pack_rows([t[n + "_weight"] for n in ("q", "k", "v", "g", "i", "f")])
        self.offsets = dict(zip(("r", "k", "v", "g", "a", "w"), offs))
        self.i_bias, self.f_bias, self.out_norm, self.out_weight = t["i_bias"], t["f_bias"], t["out_norm"], t["out_weight"]
        self._pad_out_weight()

    def forward(self, ctx, run, h, x, add: bool = True, proj=None) -> None:
        proj = self._project(ctx, h, proj)
        buf, view = self._out_buffer(ctx)
        mode = K.RECURRENCES["matrix_memory"]
        prep, oraw = self._scratch(ctx, mode, self.key_dim, self.value_dim + 1)
        gates = ctx.workspace.get("state_mixer_gates", (ctx.n_tokens * self.num_heads * 4,), torch.float32)
        K.recurrence(mode, proj, self.offsets, ctx.state(run.state_key), buf if view is None else view,
                     ctx.q_start, ctx.slots, prep, oraw, n_reqs=ctx.n_reqs, n_heads=self.num_heads, dk=self.key_dim,
                     dv=self.value_dim, eps=self.norm_eps, a_bias=self.i_bias, w0=self.f_bias, out_weight=self.out_norm,
                     cap=self.gate_cap, floor_eps=self.floor_eps, qscale=self.query_scale, gates=gates)
        K.linear(buf, self.out_weight, None, x, residual=add)
