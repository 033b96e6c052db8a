"""What a stack adds to the stream between two runs of its layers.

``pass_input`` serves stacks that run a stretch of their layers several times in a row: ahead of every pass a
learned row of the pass is added to every token's row of the stream, and ahead of every pass but the first also
the embedding's output as it entered the stack.  One kernel an occurrence (csrc/stream_ops.cu), float32.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import ParamSpec, Part, register_part
from .standard import RMSNorm


@register_part("stream_input", "pass_input")
class PassInput(Part):
    """``x <- x + table[index]`` and, for ``index > 0`` (``readd_embedding``), ``+ x_0``, the embedding's output.
    ``table`` float32 [passes, hidden].  The embedding's output is kept in a buffer of the step: by the
    occurrence that comes first in the run (it reads the stream before anything was added), else by
    ``keep_embedding``."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, hidden_size: int, passes: int, readd_embedding: bool = True) -> None:
        if passes <= 0:
            raise ValueError("pass input: at least one pass")
        self.hidden_size, self.passes, self.readd_embedding = int(hidden_size), int(passes), bool(readd_embedding)
        self.table = None

    def param_specs(self):
        return [ParamSpec("table", (self.passes, self.hidden_size), kind="vector", init="zeros")]

    def _kept(self, ctx, x):
        return ctx.workspace.get("stream_first", tuple(x.shape), torch.float32)

    @property
    def wants_embedding(self) -> bool:
        return self.readd_embedding and self.passes > 1

    def keep_embedding(self, ctx, x) -> None:
        if self.wants_embedding:
            K.stream_inject(x, keep=self._kept(ctx, x))

    def forward(self, ctx, x, first: bool = False, layer=None, index: int = 0) -> None:
        if not 0 <= index < self.passes:
            raise ValueError(f"pass input: pass {index} of {self.passes}")
        keep = self._kept(ctx, x) if first and self.wants_embedding else None
        again = self._kept(ctx, x) if index > 0 and self.readd_embedding else None
        # where the layer that runs next begins with an RMS norm of the stream and takes it ready-made, the same
        # launch leaves it (fused: no kernel of its own normalises the rows this one has just written)
        name = getattr(getattr(layer, "block", None), "takes_normed_ahead", None)
        norm = getattr(layer, name, None) if name else None
        if isinstance(norm, RMSNorm):
            out = ctx.workspace.get("normed", tuple(x.shape), ctx.act_dtype)
            K.stream_inject(x, vec=self.table[index], again=again, keep=keep, norm=(norm.weight, norm.eps, out))
            ctx.extras["normed_ahead"] = out
        else:
            K.stream_inject(x, vec=self.table[index], again=again, keep=keep)
