"""Layers that normalise the stream itself, after each sublayer's result has been added to it.

``x <- norm(alpha * x + gate * sublayer(x))``: the sublayers read the stream, their result passes a gate
computed from the same input, and the norm is taken of the sum, so the stream that the next sublayer reads is
always a normalised one.  The join (gate, weighted sum, norm) is one kernel (csrc/rms_norm.cu:
``gated_join_norm_kernel``), which also leaves the bfloat16 copy of the new rows that the next products read.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import ParamSpec, Part, register_part
from .recurrent import pack_rows
from .standard import NormedSublayersBlock


@register_part("norm", "gated_join_norm")
class GatedJoinNorm(Part):
    """The norm after the sum, with a gated sublayer result: for a sublayer that read ``h`` and gave ``y``,

        x <- (alpha * x + sigmoid(W_gate h + b_gate) * y) / sqrt(mean(.^2) + eps) * weight

    all in float32 but the gate's product, which takes ``h`` as the other products do (``gate`` off: no gate).  ``y`` may be the sum of
    several results with a weight each (mixers side by side).  ``forward`` is the plain RMS norm with the same
    weight, for a consumer that wants normalised rows."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, hidden_size: int, eps: float, alpha: float = 1.0, gate: bool = True) -> None:
        if eps <= 0:
            raise ValueError("the norm's eps must be positive")
        self.hidden_size, self.eps, self.alpha, self.has_gate = hidden_size, float(eps), float(alpha), bool(gate)
        self.weight = self.gate_weight = self.gate_bias = None

    def param_specs(self):
        specs = [ParamSpec("weight", (self.hidden_size,), kind="vector", init="ones")]
        if self.has_gate:
            specs += [ParamSpec("gate_weight", (self.hidden_size, self.hidden_size)),
                      ParamSpec("gate_bias", (self.hidden_size,), kind="vector", init="zeros")]
        return specs

    def forward(self, ctx, x, rows=None, n_rows=None, name="normed", defer: bool = False):
        n = x.shape[0] if rows is None else int(n_rows)
        out = ctx.workspace.get(name, (n, self.hidden_size), ctx.act_dtype)
        K.rmsnorm(x, self.weight, self.eps, out, rows)
        return out

    def join(self, ctx, h, x, results, copy=None, logits=None) -> None:
        """``results``: one or two (float32 [tokens, hidden], weight) pairs of the sublayer that read ``h``;
        ``copy``: where the new rows go in bfloat16 (``None`` in the 32-bit mode); ``logits``: the gate's product
        ``h W_gate^T`` without its bias (float32, a view with a row stride will do), where the caller has
        multiplied ``gate_weight`` together with other weights that read ``h``."""
        if not 1 <= len(results) <= 2:
            raise ValueError("gated_join_norm: one or two results are joined at a time")
        z = bias = None
        if self.has_gate:
            if logits is not None:
                z, bias = logits, self.gate_bias
            else:
                z = ctx.workspace.get("join_gate", tuple(x.shape), torch.float32)
                K.linear(h, self.gate_weight, self.gate_bias, z)
        (y0, s0), (y1, s1) = results[0], results[1] if len(results) == 2 else (None, 0.0)
        K.gated_join_norm(y0, s0, y1, s1, z, self.weight, self.eps, self.alpha, x, copy, z_bias=bias)


@register_part("block", "post_norm_gated")
class PostNormGatedBlock(Part):
    """``x <- join_mixer(x, sum_m scale_m * mixer_m(x))``, then (where the layer has one) ``x <-
    join_feed_forward(x, feed_forward(x))``, the joins being ``gated_join_norm`` parts.  ``mixers``: (name of the
    layer's sub-part, weight of its result) for every mixer that reads the same input, one or two; each keeps
    pages and state of its own under its name.  A mixer with ``takes_projection`` (it has a packed ``proj_weight``
    and its ``forward`` takes ``proj``, the product of the input with that weight) gets its projections from one
    product a layer, which also makes the logits of the join's gate."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, mixers=(("mixer", 1.0),), feed_forward: bool = True) -> None:
        self.mixers = tuple((str(n), float(s)) for n, s in mixers)
        if not 1 <= len(self.mixers) <= 2:
            raise ValueError("post_norm_gated: one or two mixers a layer")
        self.has_feed_forward = bool(feed_forward)
        self._packed = None  # (the sublayer's weights that read the layer's input as one, each part's rows) once bound
        self.uses = {name: "mixer" for name, _ in self.mixers}
        self.uses["join_mixer"] = "norm"
        if feed_forward:
            self.uses.update(feed_forward="feed_forward", join_feed_forward="norm")

    def _pack(self, layer):
        """Everything of the mixer sublayer that multiplies the layer's input (the mixers' packed projections
        and the join's gate) as one weight, so that one product serves them all; the parts keep views of their
        rows, not copies.  Parts without a ``proj_weight`` (a mixer that projects otherwise) stay on their own."""
        takers = [getattr(layer, name) for name, _ in self.mixers]
        takers = [m for m in takers if getattr(m, "takes_projection", False) and getattr(m, "proj_weight", None) is not None]
        gate = layer.join_mixer if layer.join_mixer.has_gate else None
        weights = [m.proj_weight for m in takers] + ([gate.gate_weight] if gate is not None else [])
        if len(weights) < 2 or len({(w.dtype, w.shape[1]) for w in weights}) != 1:
            self._packed = (None, {})
            return
        packed, offsets = pack_rows(weights)
        spans = {}
        for part, w, o in zip(takers + ([gate] if gate is not None else []), weights, offsets):
            spans[id(part)] = (o, o + w.shape[0])
            if part is gate:
                part.gate_weight = packed[o:o + w.shape[0]]
            else:
                part.proj_weight = packed[o:o + w.shape[0]]
        self._packed = (packed, spans)

    def forward(self, ctx, run, layer, x) -> None:
        h, copy = NormedSublayersBlock._stream_input(ctx, x)
        if self._packed is None:
            self._pack(layer)
        packed, spans = self._packed
        proj = None
        if packed is not None:
            proj = ctx.workspace.get("layer_proj", (ctx.n_tokens, packed.shape[0]), torch.float32)
            K.linear(h, packed, None, proj)

        def part_of(part):
            span = spans.get(id(part))
            return None if span is None else proj[:, span[0]:span[1]]

        results = []
        for i, (name, scale) in enumerate(self.mixers):
            y = ctx.workspace.get(f"sublayer_out_{i}", tuple(x.shape), torch.float32)
            mixer, view = getattr(layer, name), part_of(getattr(layer, name))
            if view is None:
                mixer.forward(ctx, run.for_part(name), h, y, add=False)
            else:
                mixer.forward(ctx, run.for_part(name), h, y, add=False, proj=view)
            results.append((y, scale))
        layer.join_mixer.join(ctx, h, x, results, copy, logits=part_of(layer.join_mixer))
        if self.has_feed_forward:
            y = ctx.workspace.get("sublayer_out_0", tuple(x.shape), torch.float32)
            layer.feed_forward.forward(ctx, h, y, add=False)
            layer.join_feed_forward.join(ctx, h, x, [(y, 1.0)], copy)
