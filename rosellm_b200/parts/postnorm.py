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

    def join(self, ctx, h, x, results, copy=None) -> None:
        """``results``: one or two (float32 [tokens, hidden], weight) pairs of the sublayer that read ``h``;
        ``copy``: where the new rows go in bfloat16 (``None`` in the 32-bit mode)."""
        if not 1 <= len(results) <= 2:
            raise ValueError("gated_join_norm: one or two results are joined at a time")
        z = None
        if self.has_gate:
            z = ctx.workspace.get("join_gate", tuple(x.shape), torch.float32)
            K.linear(h, self.gate_weight, self.gate_bias, z)
        (y0, s0), (y1, s1) = results[0], results[1] if len(results) == 2 else (None, 0.0)
        K.gated_join_norm(y0, s0, y1, s1, z, self.weight, self.eps, self.alpha, x, copy)


@register_part("block", "post_norm_gated")
class PostNormGatedBlock(Part):
    """``x <- join_mixer(x, sum_m scale_m * mixer_m(x))``, then (where the layer has one) ``x <-
    join_feed_forward(x, feed_forward(x))``, the joins being ``gated_join_norm`` parts.  ``mixers``: (name of the
    layer's sub-part, weight of its result) for every mixer that reads the same input, one or two; each keeps
    pages and state of its own under its name."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, mixers=(("mixer", 1.0),), feed_forward: bool = True) -> None:
        self.mixers = tuple((str(n), float(s)) for n, s in mixers)
        if not 1 <= len(self.mixers) <= 2:
            raise ValueError("post_norm_gated: one or two mixers a layer")
        self.has_feed_forward = bool(feed_forward)
        self.uses = {name: "mixer" for name, _ in self.mixers}
        self.uses["join_mixer"] = "norm"
        if feed_forward:
            self.uses.update(feed_forward="feed_forward", join_feed_forward="norm")

    def forward(self, ctx, run, layer, x) -> None:
        h, copy = NormedSublayersBlock._stream_input(ctx, x)
        results = []
        for i, (name, scale) in enumerate(self.mixers):
            y = ctx.workspace.get(f"sublayer_out_{i}", tuple(x.shape), torch.float32)
            getattr(layer, name).forward(ctx, run.for_part(name), h, y, add=False)
            results.append((y, scale))
        layer.join_mixer.join(ctx, h, x, results, copy)
        if self.has_feed_forward:
            y = ctx.workspace.get("sublayer_out_0", tuple(x.shape), torch.float32)
            layer.feed_forward.forward(ctx, h, y, add=False)
            layer.join_feed_forward.join(ctx, h, x, [(y, 1.0)], copy)
