"""Softmax attention over the latest keys only, with normalised and rotated queries and keys, values of unit
root mean square and a temperature per head; optionally biases in the projections, a softmax sink (learned per
head, or a constant) and an output gate (a logit per head, or per value column).

It runs on the kernels of the distance-biased attention (csrc/bias_attention.cu: rows of [key | value] in the
cache, key and value sizes of their own, grouped key/value heads), which take a window and a per-head factor
of the scores; what happens to queries, keys and values between the projections and the cache is one kernel
of its own (``K.qkv_norm_rotate``).
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import KVCacheSpec, ParamSpec, register_part, step_decode_plan
from .biased import BiasedAttention
from .recurrent import pack_rows
from .standard import RotaryPositions


@register_part("mixer", "window_attention")
class WindowAttention(BiasedAttention):
    """``q, k, v = W_q h, W_k h, W_v h`` without biases; query head ``h`` uses key/value head
    ``h // (num_heads / num_kv_heads)``.  With ``qk_norm`` every head of q and k is divided by its root mean
    square over ``key_dim`` (``norm_eps`` inside the root) and multiplied by a weight the heads share
    (``q_norm`` / ``k_norm``); then the first ``rot_dims`` entries of every head of q and k are turned in
    neighbouring pairs (2i, 2i + 1) by the angle position * ``rot_base``^(-2i / rot_dims); with ``unit_values``
    every head of v is divided by its root mean square over ``value_dim`` (no weight) and cached so.

        score = (q . k) * scale * head_temp[h]        for 0 <= i - j < window   (``window`` None: j <= i)

    (``head_temperature`` off: no per-head factor), a plain softmax over the keys a query sees, the merged
    heads through ``W_o``.  The cache gives pages back once the window has passed them.  Norms, angles,
    rotation, scores, softmax and the weighted sums are float32 in both precisions.

    Further switches, each off by default: ``qk_norm_weights=False`` (with ``qk_norm``): queries and keys are
    divided by their root mean square and get no weight; ``bias``: q, k and v have biases, added by the
    projection; ``rot_scaling``: the rotation's frequencies are stretched (``RotaryPositions``); ``sink``:
    ``"learned"`` (a tensor with one entry a head) or a number: one more term exp(sink) in the softmax's
    denominator, which has no key and no value and is not scaled; ``gate``: ``"head"`` (``W_g`` [heads, hidden]:
    head h's result times sigmoid((W_g h)_h)) or ``"element"`` (``W_g`` [heads * value_dim, hidden]: the merged
    heads times sigmoid(W_g h) element by element), read from the same input as the projections and packed
    with them into one product."""

    takes_projection = True  # forward(.., proj=): the input times ``proj_weight``, made by the caller

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 norm_eps: float, window: int | None = None, rot_dims: int = 0, rot_base: float = 10000.0,
                 qk_norm: bool = True, unit_values: bool = True, head_temperature: bool = True,
                 qk_norm_weights: bool = True, bias: bool = False, rot_scaling: dict | None = None,
                 sink: "str | float | None" = None, gate: str | None = None) -> None:
        super().__init__(hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, slope_log2_span=0.0,
                         value_mix=None, gate=False)
        if gate not in (None, "head", "element"):
            raise ValueError(f"window attention: gate {gate!r}; None, 'head' or 'element'")
        if sink is not None and sink != "learned" and not isinstance(sink, (int, float)):
            raise ValueError(f"window attention: sink {sink!r}; None, 'learned' or a number")
        self.gate_kind, self.has_bias, self.sink_kind = gate, bool(bias), sink
        self.has_gate = gate is not None
        self.gate_width = 0 if gate is None else (num_heads if gate == "head" else self.out_width)
        self.qk_norm_weights = bool(qk_norm_weights)
        if window is not None and window <= 0:
            raise ValueError(f"window attention: a window of {window} keys")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > key_dim:
            raise ValueError(f"window attention: {rot_dims} turned entries of {key_dim}: an even count within the key size")
        self.window = None if window is None else int(window)
        self.norm_eps = float(norm_eps)
        self.rot_dims = int(rot_dims)
        self.rotary = RotaryPositions(dims=self.rot_dims, base=rot_base, scaling=rot_scaling) if rot_dims else None
        self.qk_norm, self.unit_values, self.head_temperature = bool(qk_norm), bool(unit_values), bool(head_temperature)
        self.q_norm = self.k_norm = self.head_temp = self.sink = self.proj_bias = None

    def decode_plan_for(self, n_decode: int, span: int, act_dtype=None) -> tuple[int, bool]:
        return super().decode_plan_for(n_decode, span if self.window is None else min(span, self.window), act_dtype)

    def param_specs(self):
        hid = self.hidden_size
        specs = [ParamSpec("q_weight", (self.q_width, hid)), ParamSpec("k_weight", (self.k_width, hid)),
                 ParamSpec("v_weight", (self.v_width, hid)), ParamSpec("out_weight", (hid, self.out_width))]
        if self.qk_norm and self.qk_norm_weights:
            specs += [ParamSpec("q_norm", (self.key_dim,), kind="vector", init="ones"),
                      ParamSpec("k_norm", (self.key_dim,), kind="vector", init="ones")]
        if self.head_temperature:
            specs.append(ParamSpec("head_temp", (self.num_heads,), kind="vector", init="ones"))
        if self.has_bias:
            specs += [ParamSpec("q_bias", (self.q_width,), kind="vector", init="zeros"),
                      ParamSpec("k_bias", (self.k_width,), kind="vector", init="zeros"),
                      ParamSpec("v_bias", (self.v_width,), kind="vector", init="zeros")]
        if self.sink_kind == "learned":
            specs.append(ParamSpec("sink", (self.num_heads,), kind="vector", init="zeros"))
        if self.has_gate:
            specs.append(ParamSpec("gate_weight", (self.gate_width, hid)))
        return specs

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.row, self.window, planes=1)

    def bind(self, tensors) -> None:
        t = dict(tensors)
        parts = [t["q_weight"], t["k_weight"], t["v_weight"]] + ([t["gate_weight"]] if self.has_gate else [])
        self.proj_weight, offs = pack_rows(parts)
        self.offsets = dict(zip(("q", "k", "v", "g"), offs))
        self.proj_bias = None
        if self.has_bias:  # the packed product's bias: the three biases at their rows, zero elsewhere
            self.proj_bias = torch.zeros(self.proj_weight.shape[0], dtype=torch.float32, device=self.proj_weight.device)
            for name, role in (("q", "q_bias"), ("k", "k_bias"), ("v", "v_bias")):
                self.proj_bias[self.offsets[name]:self.offsets[name] + t[role].numel()] = t[role]
        self.sink = t.get("sink")
        if self.sink_kind is not None and self.sink_kind != "learned":
            self.sink = torch.full((self.num_heads,), float(self.sink_kind), dtype=torch.float32,
                                   device=self.proj_weight.device)
        self.out_weight = t["out_weight"]
        if self.out_padded != self.out_width:
            self.out_weight = torch.nn.functional.pad(self.out_weight, (0, self.out_padded - self.out_width)).contiguous()
        self.q_norm, self.k_norm, self.head_temp = t.get("q_norm"), t.get("k_norm"), t.get("head_temp")
        self.slopes = self.mix_weight = None

    def forward(self, ctx, run, h, x, add: bool = True, proj=None) -> None:
        n, ws = ctx.n_tokens, ctx.workspace
        if proj is None:  # else: a block has multiplied this part's packed weight together with others'
            proj = ws.get("mixer_proj", (n, self.proj_weight.shape[0]), torch.float32)
            K.linear(h, self.proj_weight, self.proj_bias, proj)
        elif self.has_bias:
            raise ValueError("window attention: a projection made by the block carries no biases")
        o = self.offsets
        q = proj[:, o["q"]:o["q"] + self.q_width]
        k = proj[:, o["k"]:o["k"] + self.k_width]
        v = proj[:, o["v"]:o["v"] + self.v_width]
        gate = proj[:, o["g"]:o["g"] + self.gate_width] if self.has_gate else None
        pool, table = ctx.kv_pool(run.cache_key), ctx.block_table(run.cache_key)
        stored = False
        if self.qk_norm or self.rot_dims or self.unit_values:
            # the same pass puts the step's keys and values into their pages (fused: no store kernel behind it)
            stored = run.writes_cache
            target = K.QkvCache(pool, table, ctx.req_of_token, ctx.slots, self.v_at, ctx.cache.max_seq_len) if stored else None
            K.qkv_norm_rotate(q, k, v, ctx.positions, n_heads=self.num_heads, n_kv=self.num_kv_heads, dk=self.key_dim,
                              dv=self.value_dim, eps=self.norm_eps, q_norm=self.q_norm, k_norm=self.k_norm,
                              freq=self.rotary.frequencies(ctx.device) if self.rotary is not None else None,
                              rot_dims=self.rot_dims, unit_values=self.unit_values,
                              unit_qk=self.qk_norm and not self.qk_norm_weights, cache=target)
        if run.writes_cache and not stored:
            K.bias_kv_store(k, v, pool, table, ctx.positions, ctx.req_of_token, ctx.slots, v_at=self.v_at,
                            max_pos=ctx.cache.max_seq_len)
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
                         dk=self.key_dim, dv=self.value_dim, v_at=self.v_at, scale=self.scale,
                         tiles=ctx.tiles_wide if wide else ctx.tiles, n_tiles=ctx.n_tiles_wide if wide else ctx.n_tiles,
                         tile_tokens=64 if wide else 16, decode_reqs=ctx.decode_reqs, n_decode=ctx.n_decode,
                         max_pos=ctx.cache.max_seq_len, n_splits=splits, part_o=part_o, part_ml=part_ml, tensor_cores=mma,
                         window=self.window or 0, head_scale=self.head_temp, sink=self.sink,
                         gate_per_head=self.gate_kind == "head")
        K.linear(buf, self.out_weight, None, x, residual=add)
