"""Causal attention whose positions enter through the scores alone: a distance bias per head and a query
temperature that grows with the position; no rotation.  Keys and values have sizes of their own, query
heads share key/value heads in groups, values may be mixed with those of an earlier layer, and the merged
heads pass an output gate.  Kernels: csrc/bias_attention.cu.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import KVCacheSpec, ParamSpec, Part, register_part, step_decode_plan
from .recurrent import pack_rows


def distance_slopes(num_heads: int, log2_span: float) -> torch.Tensor:
    """slope_h = 2^(-log2_span * (h + 1) / num_heads) for h = 0 .. num_heads - 1, evaluated in float64 and
    kept in float32."""
    h = torch.arange(1, num_heads + 1, dtype=torch.float64)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), -float(log2_span) * h / num_heads).to(torch.float32)


@register_part("mixer", "biased_attention")
class BiasedAttention(Part):
    """``q, k, v = W_q h, W_k h, W_v h`` without biases; query head ``h`` uses key/value head
    ``h // (num_heads / num_kv_heads)``.  For a query at position ``i`` and a key at ``j <= i``:

        score = (q . k) * scale * (1 + temp_coef * ln(floor((i + 1) / temp_every) + 1)) - slope_h * (i - j)

    with ``slope_h = 2^(-slope_log2_span * (h + 1) / num_heads)`` (``slope_log2_span = 0``: no bias;
    ``temp_every = 0``: no temperature), a plain softmax over the keys a query may see, and the merged heads
    multiplied by ``sigmoid(W_g h)`` (``gate``) ahead of ``W_o``.

    ``value_mix``: ``"source"`` leaves the step's values for later layers; ``"mix"`` replaces its own by
    ``(1 - lambda) v + lambda v_source`` (``lambda``: the scalar ``mix_weight``) before they are cached, so
    the cache holds the mixed values and nothing of the source has to be kept beyond the step.

    The cache keeps one row a token and key/value head: the key's ``key_dim`` entries, then (from a
    multiple of 8 on) the value's ``value_dim``.  All four projections are one product writing float32;
    scores, softmax and the weighted sums are float32 in both precisions (in bfloat16 mode the prompt
    portions' two products take bfloat16 operands on the tensor cores and accumulate in float32)."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 slope_log2_span: float = 8.0, temp_coef: float = 0.0, temp_every: int = 0,
                 value_mix: str | None = None, gate: bool = True) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} key/value heads")
        if key_dim > 256 or value_dim > 256:
            raise ValueError(f"biased attention: sizes {key_dim} / {value_dim}: the kernel takes up to 256")
        if value_mix not in (None, "source", "mix"):
            raise ValueError(f"value_mix {value_mix!r}; None, 'source' or 'mix'")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim, self.scale = key_dim, value_dim, float(scale)
        self.slope_log2_span, self.temp_coef, self.temp_every = float(slope_log2_span), float(temp_coef), int(temp_every)
        self.value_mix, self.has_gate = value_mix, bool(gate)
        self.v_at = -(-key_dim // 8) * 8
        self.row = -(-(self.v_at + value_dim) // 8) * 8
        self.q_width, self.k_width = num_heads * key_dim, num_kv_heads * key_dim
        self.v_width, self.out_width = num_kv_heads * value_dim, num_heads * value_dim
        self.out_padded = -(-self.out_width // 8) * 8
        self.proj_weight = self.out_weight = self.mix_weight = self.slopes = None
        self._shape = None

    def decode_plan_for(self, n_decode: int, span: int, act_dtype=None) -> tuple[int, bool]:
        """(parts, False): into how many parts the keys of a decoded request are cut when ``n_decode`` requests
        attend over about ``span`` keys each.  A block walks its keys 32 at a time, one tile after the other,
        and a tile is a chain of dependent steps, so what hides its latency is other blocks on the same SM
        (they are small: eight fit): the keys are spread until there are about eight blocks an SM, each
        keeping at least two tiles; the parts are merged in their order by a second kernel."""
        if n_decode <= 0:
            return 1, False
        blocks = n_decode * self.num_kv_heads * -(-(self.num_heads // self.num_kv_heads) // 32)
        tiles = max(1, -(-span // 32))
        return max(1, min(8 * K.sm_count() // blocks, tiles // 2, 32)), False

    def launch_key(self, ctx) -> tuple:
        return (step_decode_plan(self, ctx),) if ctx.n_decode else ()

    def param_specs(self):
        hid = self.hidden_size
        specs = [ParamSpec("q_weight", (self.q_width, hid)), ParamSpec("k_weight", (self.k_width, hid)),
                 ParamSpec("v_weight", (self.v_width, hid)), ParamSpec("out_weight", (hid, self.out_width))]
        if self.has_gate:
            specs.append(ParamSpec("gate_weight", (self.out_width, hid)))
        if self.value_mix is not None:
            specs.append(ParamSpec("mix_weight", (), kind="vector", init="zeros"))
        return specs

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.row, None, planes=1)

    def bind(self, tensors) -> None:
        t = dict(tensors)
        parts = [t["q_weight"], t["k_weight"], t["v_weight"]] + ([t["gate_weight"]] if self.has_gate else [])
        self.proj_weight, offs = pack_rows(parts)
        self.offsets = dict(zip(("q", "k", "v", "g"), offs))
        self.out_weight = t["out_weight"]
        if self.out_padded != self.out_width:
            self.out_weight = torch.nn.functional.pad(self.out_weight, (0, self.out_padded - self.out_width)).contiguous()
        self.mix_weight = t.get("mix_weight")
        if self.mix_weight is not None:
            self.mix_weight = self.mix_weight.reshape(1).contiguous()
        self.slopes = None
        if self.slope_log2_span != 0.0:
            self.slopes = distance_slopes(self.num_heads, self.slope_log2_span).to(self.out_weight.device)

    def forward(self, ctx, run, h, x, add: bool = True) -> None:
        n, ws = ctx.n_tokens, ctx.workspace
        proj = ws.get("mixer_proj", (n, self.proj_weight.shape[0]), torch.float32)
        K.linear(h, self.proj_weight, None, proj)
        o = self.offsets
        q = proj[:, o["q"]:o["q"] + self.q_width]
        gate = proj[:, o["g"]:o["g"] + self.out_width] if self.has_gate else None
        pool, table = ctx.kv_pool(run.cache_key), ctx.block_table(run.cache_key)
        if run.writes_cache:
            mix, src = 0, None
            if self.value_mix == "source":
                mix, src = 1, ws.get("value_source", (n, self.v_width), torch.float32)
                ctx.extras["value_source"] = src
            elif self.value_mix == "mix":
                mix, src = 2, ctx.extras.get("value_source")
                if src is None or tuple(src.shape) != (n, self.v_width):
                    raise ValueError("biased attention: a layer that mixes values runs after the layer that is their "
                                     "source, whose values have the same size")
            K.bias_kv_store(proj[:, o["k"]:o["k"] + self.k_width], proj[:, o["v"]:o["v"] + self.v_width], pool, table,
                            ctx.positions, ctx.req_of_token, ctx.slots, v_at=self.v_at, max_pos=ctx.cache.max_seq_len,
                            mix=mix, v_src=src, lam=self.mix_weight if mix == 2 else None)
        if self.out_padded == self.out_width:
            buf = ws.get("biased_attn_out", (n, self.out_padded), ctx.act_dtype)
            out = buf
        else:  # the fill stays zero: see the state mixers' output buffer
            buf = ws.get_zeroed(f"biased_attn_out_{self.out_width}_{self.out_padded}", (n, self.out_padded), ctx.act_dtype)
            out = buf[:, :self.out_width]
        mma = K.bias_attention_tensor_cores(ctx.act_dtype, self.key_dim, self.value_dim)
        if self._shape is None or self._shape[0] != mma:
            self._shape = (mma, K.bias_attention_shape(self.num_heads // self.num_kv_heads, mma)[1])
        wide = self._shape[1] > 16  # the tokens a block takes must divide the tiles the step is cut into
        splits = step_decode_plan(self, ctx)[0]
        part_o = part_ml = None
        if splits > 1:
            rows = ctx.n_decode * self.num_heads * splits
            part_o = ws.get("biased_attn_part_o", (rows, self.value_dim), torch.float32)
            part_ml = ws.get("biased_attn_part_ml", (rows, 2), torch.float32)
        K.bias_attention(q, gate, pool, table, ctx.q_start, ctx.kv_len, ctx.slots, out, n_heads=self.num_heads,
                         dk=self.key_dim, dv=self.value_dim, v_at=self.v_at, scale=self.scale, slopes=self.slopes,
                         temp_coef=self.temp_coef, temp_every=self.temp_every,
                         tiles=ctx.tiles_wide if wide else ctx.tiles, n_tiles=ctx.n_tiles_wide if wide else ctx.n_tiles,
                         tile_tokens=64 if wide else 16, decode_reqs=ctx.decode_reqs, n_decode=ctx.n_decode,
                         max_pos=ctx.cache.max_seq_len, n_splits=splits, part_o=part_o, part_ml=part_ml, tensor_cores=mma)
        K.linear(buf, self.out_weight, None, x, residual=add)
