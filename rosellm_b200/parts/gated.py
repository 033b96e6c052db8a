"""Gated feed-forward layers: dense, a mixture of experts, and a token-gated input.

All three end in a product whose result goes to the residual stream or (``add=False``) to a
buffer that the block normalises first.  The gate functions are those of csrc/gated_act.cuh:
``relu``, ``silu``, ``gelu_tanh`` (f(g) * u) and ``clamped_swish``
(g' = min(g, limit), u' = clamp(u, -limit, limit): g' * sigmoid(alpha * g') * (u' + 1)).
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import ParamSpec, Part, register_part


def _gate(name: str) -> int:
    if name not in K.GATES:
        raise ValueError(f"gate function {name!r}; one of {sorted(K.GATES)}")
    return K.GATES[name]


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """``W_down f(W_gate h, W_up h)``, no biases.  The file may hold gate and up apart (a
    ``Concat`` in the model's spec joins them, gate rows first)."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, hidden_size: int, inner_size: int, gate: str = "silu", alpha: float = 1.0,
                 limit: float = 0.0) -> None:
        if hidden_size % 8:
            raise ValueError(f"gated MLP: the width {hidden_size} must be a multiple of 8")
        self.hidden_size, self.inner_size = hidden_size, inner_size
        self.gate, self.alpha, self.limit = _gate(gate), float(alpha), float(limit)
        self.inner_padded = -(-inner_size // 8) * 8
        self.gate_up_weight = self.down_weight = None

    def param_specs(self):
        return [ParamSpec("gate_up_weight", (2 * self.inner_size, self.hidden_size)),
                ParamSpec("down_weight", (self.hidden_size, self.inner_size))]

    def bind(self, tensors) -> None:
        """An inner size that is no multiple of 8 is filled up with units of zero weight: every
        gate function maps (0, 0) to 0, and their columns of W_down are zero."""
        super().bind(tensors)
        pad = self.inner_padded - self.inner_size
        if pad:
            f = self.inner_size
            g, u = self.gate_up_weight[:f], self.gate_up_weight[f:]
            fill = torch.nn.functional.pad
            self.gate_up_weight = torch.cat([fill(g, (0, 0, 0, pad)), fill(u, (0, 0, 0, pad))]).contiguous()
            self.down_weight = fill(self.down_weight, (0, pad)).contiguous()

    def forward(self, ctx, h, x, add: bool = True) -> None:
        n, f = ctx.n_tokens, self.inner_padded
        gu = ctx.workspace.get("gated_gate_up", (n, 2 * f), ctx.act_dtype)
        K.linear(h, self.gate_up_weight, None, gu)
        a = ctx.workspace.get("gated_inner", (n, f), ctx.act_dtype)
        K.gated_act(gu, a, width=f, up_at=f, gate=self.gate, alpha=self.alpha, limit=self.limit)
        K.linear(a, self.down_weight, None, x, residual=add)


@register_part("feed_forward", "moe")
class MixtureOfExperts(Part):
    """``num_experts`` gated feed-forward layers of which a token uses ``top``.

    Router logits ``z = W_router h`` with float32 accumulation and output; scores
    ``s = softmax(z)`` over all experts, or (``score="sigmoid"``) each expert's ``sigmoid(z)``; the choice is made on ``s + correction`` (where the
    model has one), restricted, with groups, to the experts of the ``group_keep`` groups (of
    ``group_count`` equal groups of neighbours) whose best choice score is largest; the chosen
    experts' outputs are summed with their scores ``s`` as weights (not renormalised); with
    ``weight_input`` the weight multiplies the expert's input instead: the sum of ``expert(s * h)``.
    ``routing="table"``: no router; row ``token id`` of an integer table ``[vocab_size, top]`` (tensor ``table``; the
    entries of a row differ) names the token's experts, each with weight ``1 / top``.
    Routing, the experts' layout and their products all run on the device
    (csrc/moe.cu): a step's launches follow from its token count alone.
    Experts' tensors: ``gate_up_weight`` [experts * 2 * inner, hidden] (per expert the gate rows,
    then the up rows), ``down_weight`` [experts * hidden, inner]; the model's spec joins the
    file's per-expert tensors with ``Concat``."""

    graph_safe = True
    launches_replayable = True
    _made = 0

    def __init__(self, hidden_size: int, inner_size: int, num_experts: int, top: int, group_count: int = 1,
                 group_keep: int = 1, gate: str = "silu", alpha: float = 1.0, limit: float = 0.0,
                 correction: bool = False, score: str = "softmax", weight_input: bool = False,
                 routing: str = "router", vocab_size: int = 0) -> None:
        if routing not in ("router", "table"):
            raise ValueError(f"mixture of experts: routing {routing!r}; 'router' or 'table'")
        if routing == "table" and (vocab_size <= 0 or correction or group_count != 1):
            raise ValueError("mixture of experts: a routing table needs the vocabulary's size and takes no "
                             "correction and no groups")
        if routing == "table" and weight_input:
            raise ValueError("mixture of experts: a routing table weights the experts' outputs")
        self.routing, self.vocab_size = routing, int(vocab_size)
        MixtureOfExperts._made += 1
        self._tag = MixtureOfExperts._made  # names this part's own routing buffers in a step's workspace
        if score not in K.MOE_SCORES:
            raise ValueError(f"mixture of experts: score {score!r}; one of {sorted(K.MOE_SCORES)}")
        self.score, self.weight_input = K.MOE_SCORES[score], bool(weight_input)
        if hidden_size % 8:
            raise ValueError(f"mixture of experts: the width {hidden_size} must be a multiple of 8")
        if not 0 < top <= num_experts or num_experts > 2048:
            raise ValueError(f"mixture of experts: top {top} of {num_experts} experts (at most 2048)")
        if group_count < 1 or num_experts % group_count or not 1 <= group_keep <= group_count:
            raise ValueError(f"mixture of experts: {num_experts} experts do not form {group_count} equal groups, "
                             f"or {group_keep} of them cannot be kept")
        if top > group_keep * (num_experts // group_count):
            raise ValueError(f"mixture of experts: top {top} exceeds the experts of {group_keep} groups")
        self.hidden_size, self.inner_size = hidden_size, inner_size
        self.num_experts, self.top = num_experts, top
        self.group_count, self.group_keep = group_count, group_keep
        self.gate, self.alpha, self.limit = _gate(gate), float(alpha), float(limit)
        self.has_correction = bool(correction)
        self.router_weight = self.correction = self.gate_up_weight = self.down_weight = self.table = None

    def param_specs(self):
        E, f, hid = self.num_experts, self.inner_size, self.hidden_size
        specs = [ParamSpec("gate_up_weight", (E * 2 * f, hid)),
                 ParamSpec("down_weight", (E * hid, f))]
        if self.routing == "table":
            specs.append(ParamSpec("table", (self.vocab_size, self.top), kind="int_table", below=E))
        else:
            specs.insert(0, ParamSpec("router_weight", (E, hid)))
        if self.has_correction:
            specs.append(ParamSpec("correction", (E,), kind="vector"))
        return specs

    def _table_route(self, ctx):
        """Routing by the table and its layout.  Both depend on the step's token ids alone, so a part that runs
        several times in a step (a stretch of layers run in passes) routes once: the buffers are this part's own
        (named by ``_tag``) and are found again in ``ctx.extras``."""
        routes = ctx.extras.setdefault("moe_table_routes", {})
        got = routes.get(id(self))
        if got is not None:
            return got
        n, E, top = ctx.n_tokens, self.num_experts, self.top
        ws, i32, tag = ctx.workspace, torch.int32, self._tag
        ids = ws.get(f"moe_ids@{tag}", (n * top,), i32)
        weights = ws.get(f"moe_weights@{tag}", (n * top,), torch.float32)
        offsets = ws.get(f"moe_offsets@{tag}", (E + 1,), i32)
        tiles = ws.get(f"moe_tiles@{tag}", (K.moe_max_tiles(n * top, E) * 3,), i32)
        meta = ws.get(f"moe_meta@{tag}", (4,), i32)
        row_token = ws.get(f"moe_row_token@{tag}", (n * top,), i32)
        place_of = ws.get(f"moe_place_of@{tag}", (n * top,), i32)
        feedback = ctx.extras.get("token_feedback")
        if n * top <= K.MOE_TABLE_ROUTE_MAX_PAIRS:
            K.moe_table_route(ctx.token_ids, self.table, n_experts=E, weight=1.0 / top, ids=ids, weights=weights,
                              offsets=offsets, tiles=tiles, meta=meta, row_token=row_token, place_of=place_of,
                              feedback=feedback)
        else:
            counts = ws.get_zeroed("moe_counts", (E,), i32)
            fill = ws.get_zeroed("moe_fill", (E,), i32)
            K.moe_table_select(ctx.token_ids, self.table, n_experts=E, weight=1.0 / top, ids=ids, weights=weights,
                               counts=counts, feedback=feedback)
            K.moe_plan(ids, counts, fill, offsets, tiles, meta, row_token, place_of, n_tokens=n, n_experts=E, top=top)
        got = routes[id(self)] = (weights, tiles, meta, row_token, place_of)
        return got

    def forward(self, ctx, h, x, add: bool = True) -> None:
        n, E, top, f, hid = ctx.n_tokens, self.num_experts, self.top, self.inner_size, self.hidden_size
        ws, i32 = ctx.workspace, torch.int32
        by_place = None
        if self.routing == "table":
            weights, tiles, meta, row_token, place_of = self._table_route(ctx)
        else:
            ids = ws.get("moe_ids", (n * top,), i32)
            weights = ws.get("moe_weights", (n * top,), torch.float32)
            counts = ws.get_zeroed("moe_counts", (E,), i32)
            fill = ws.get_zeroed("moe_fill", (E,), i32)
            z = ws.get("moe_logits", (n, E), torch.float32)
            K.linear(h, self.router_weight, None, z)
            K.moe_select(z, self.correction, top=top, group_count=self.group_count, group_keep=self.group_keep, ids=ids,
                         weights=weights, counts=counts, score=self.score)
            offsets = ws.get("moe_offsets", (E + 1,), i32)
            tiles = ws.get("moe_tiles", (K.moe_max_tiles(n * top, E) * 3,), i32)
            meta = ws.get("moe_meta", (4,), i32)
            row_token = ws.get("moe_row_token", (n * top,), i32)
            place_of = ws.get("moe_place_of", (n * top,), i32)
            by_place = ws.get("moe_place_weight", (n * top,), torch.float32) if self.weight_input else None
            K.moe_plan(ids, counts, fill, offsets, tiles, meta, row_token, place_of, n_tokens=n, n_experts=E, top=top,
                       weights=weights if self.weight_input else None, place_weight=by_place)
        act = ws.get("moe_inner", (n * top, f), ctx.act_dtype)
        eo = ws.get("moe_expert_out", (n * top, hid), torch.float32)
        K.moe_experts(h, self.gate_up_weight, self.down_weight, tiles, meta, row_token, place_of,
                      None if self.weight_input else weights, act, eo, x, n_experts=E, top=top, ff=f, gate=self.gate,
                      alpha=self.alpha, limit=self.limit, add=add, place_weight=by_place)


@register_part("feed_forward", "token_gated_input")
class TokenGatedInput(Part):
    """A per-layer input that depends on the token itself: ``W_proj (gelu_tanh(W_gate h) * e)``
    with ``e`` the entries ``[column, column + dim)`` of the token's row in a second embedding
    table, which all layers share (each names the same file tensor and takes its own columns;
    the table lies on the device once)."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, hidden_size: int, dim: int, vocab_size: int, table_width: int, column: int) -> None:
        if hidden_size % 8:
            raise ValueError(f"token-gated input: the width {hidden_size} must be a multiple of 8")
        if dim <= 0 or column < 0 or column + dim > table_width:
            raise ValueError(f"token-gated input: columns [{column}, {column + dim}) of a table {table_width} wide")
        self.hidden_size, self.dim, self.vocab_size = hidden_size, dim, vocab_size
        self.table_width, self.column = table_width, column
        self.dim_padded = -(-dim // 8) * 8
        self.table = self.gate_weight = self.proj_weight = None

    def param_specs(self):
        return [ParamSpec("table", (self.vocab_size, self.table_width)),
                ParamSpec("gate_weight", (self.dim, self.hidden_size)),
                ParamSpec("proj_weight", (self.hidden_size, self.dim))]

    def bind(self, tensors) -> None:
        super().bind(tensors)
        pad = self.dim_padded - self.dim
        if pad:  # the second product reads rows in 16-byte pieces
            self.gate_weight = torch.nn.functional.pad(self.gate_weight, (0, 0, 0, pad)).contiguous()
            self.proj_weight = torch.nn.functional.pad(self.proj_weight, (0, pad)).contiguous()

    def forward(self, ctx, h, x, add: bool = True) -> None:
        n, d = ctx.n_tokens, self.dim_padded
        s = ctx.workspace.get("token_gate_in", (n, d), ctx.act_dtype)
        K.linear(h, self.gate_weight, None, s)
        g = ctx.workspace.get("token_gate_out", (n, d), ctx.act_dtype)
        K.token_gate(s, ctx.token_ids, self.table, self.column, self.dim, g, ctx.extras.get("token_feedback"))
        K.linear(g, self.proj_weight, None, x, residual=add)
