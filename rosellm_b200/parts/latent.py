"""Attention that caches a latent instead of keys and values.

``LatentAttention`` projects a token to per-head queries (``plain_dim`` entries that meet the
keys' up-projection and ``rot_dim`` rotated ones), and to one row ``[c, k_r]`` shared by all
heads: ``c`` (``kv_rank`` entries, RMS-normalised) and a rotated key part ``k_r``.  Head h's key
is ``[W_uk,h c, k_r]`` and its value ``W_uv,h c``; only the row is cached.  Because keys and
values are linear in ``c``, the engine never expands them: the query takes ``W_uk`` over
(``q_c = W_uk,h^T q_plain``), attention runs over the cached rows with ``c`` as the value
(csrc/latent_attention.cu), and ``W_uv`` is applied to the weighted sum of latents.  The cost of
a decoded token is then one pass over ``kv_rank + rot_dim`` numbers per cached token for all
heads together.  A softmax sink per head is optional; so are a latent for the queries (``q_rank``: ``c_q =
norm(W_dq h)``, ``q = W_uq c_q``), an element-wise output gate on the merged heads (``gate``: times ``sigmoid(W_g
h)``) and stretched rotation frequencies (``rot_scaling``).  Everything that multiplies the layer's input but
feeds float32 arithmetic (the key/value latent, the query latent, the gate) is one product with float32 output.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import KVCacheSpec, ParamSpec, Part, register_part, step_decode_plan
from .recurrent import pack_rows
from .standard import RotaryPositions


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    graph_safe = True
    launches_replayable = True

    def __init__(self, hidden_size: int, num_heads: int, plain_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 scale: float, rot_dims: int, rot_base: float, norm_eps: float, sink: bool = True,
                 q_rank: int | None = None, gate: bool = False, rot_scaling: dict | None = None) -> None:
        if min(hidden_size, num_heads, plain_dim, value_dim, kv_rank) <= 0 or rot_dim < 0:
            raise ValueError("latent attention: sizes must be positive")
        if hidden_size % 8:
            raise ValueError(f"latent attention: the width {hidden_size} must be a multiple of 8 (the products read "
                             "rows in 16-byte pieces)")
        if not 0 <= rot_dims <= rot_dim:
            raise ValueError(f"latent attention: {rot_dims} rotated entries of a rotated part of {rot_dim}")
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.plain_dim, self.rot_dim, self.value_dim, self.kv_rank = plain_dim, rot_dim, value_dim, kv_rank
        self.head_in = plain_dim + rot_dim
        self.scale, self.norm_eps, self.has_sink = float(scale), float(norm_eps), bool(sink)
        self.rotary = RotaryPositions(dims=rot_dims, base=rot_base, scaling=rot_scaling)
        if q_rank is not None and q_rank <= 0:
            raise ValueError("latent attention: the queries' latent must have a positive size")
        self.q_rank, self.has_gate = q_rank, bool(gate)
        self.q_rank_padded = 0 if q_rank is None else -(-q_rank // 8) * 8
        # a cached row: the latent, the rotated part, zeros up to a multiple of 8 entries
        self.row_width = -(-(kv_rank + rot_dim) // 8) * 8
        self.heads_width = num_heads * value_dim
        self.heads_padded = -(-self.heads_width // 8) * 8
        if not K_fits(num_heads, kv_rank, self.row_width):
            raise ValueError(f"latent attention: a latent of {kv_rank} with a rotated part of {rot_dim} is beyond "
                             "the attention kernels (latents up to 512, rows that fit shared memory)")
        self.q_weight = self.dkv_weight = self.dkv_norm = self.uk_weight = self.uv_weight = self.o_weight = None
        self.sink = self.dq_norm = self.proj_weight = None

    def param_specs(self):
        H, hid = self.num_heads, self.hidden_size
        specs = [ParamSpec("q_weight", (H * self.head_in, hid if self.q_rank is None else self.q_rank)),
                 ParamSpec("dkv_weight", (self.kv_rank + self.rot_dim, hid)),
                 ParamSpec("dkv_norm", (self.kv_rank,), kind="vector", init="ones"),
                 ParamSpec("uk_weight", (H * self.plain_dim, self.kv_rank)),
                 ParamSpec("uv_weight", (H * self.value_dim, self.kv_rank)),
                 ParamSpec("o_weight", (hid, self.heads_width))]
        if self.has_sink:
            specs.append(ParamSpec("sink", (H,), kind="vector"))
        if self.q_rank is not None:
            specs += [ParamSpec("dq_weight", (self.q_rank, hid)),
                      ParamSpec("dq_norm", (self.q_rank,), kind="vector", init="ones")]
        if self.has_gate:
            specs.append(ParamSpec("gate_weight", (self.heads_width, hid)))
        return specs

    def bind(self, tensors) -> None:
        t = dict(tensors)
        dq, gate = t.pop("dq_weight", None), t.pop("gate_weight", None)
        super().bind(t)
        # one product for all that multiplies the layer's input and is wanted in float32
        names = (["dq"] if dq is not None else []) + ["dkv"] + (["g"] if gate is not None else [])
        self.proj_weight, offs = pack_rows([{"dq": dq, "dkv": self.dkv_weight, "g": gate}[k] for k in names])
        self.offsets = dict(zip(names, offs))
        self.dkv_weight = None  # it lives in the packed weight
        if self.q_rank is not None and self.q_rank_padded != self.q_rank:  # the product with W_uq reads 16-byte pieces
            self.q_weight = torch.nn.functional.pad(self.q_weight, (0, self.q_rank_padded - self.q_rank)).contiguous()
        # W_uk per head as [latent, plain]: the query's product with it then reads both operands
        # along their inner index, like every other product
        self.uk_weight = self.uk_weight.view(self.num_heads, self.plain_dim, self.kv_rank).transpose(1, 2).contiguous()
        pad = self.heads_padded - self.heads_width
        if pad:  # the output product reads rows in 16-byte pieces: zero columns fill the last one
            self.o_weight = torch.nn.functional.pad(self.o_weight, (0, pad)).contiguous()

    def cache_spec(self):
        return KVCacheSpec(1, self.row_width, None, planes=1)

    # ---- how decoded requests are spread over blocks --------------------------------------------
    def decode_plan_for(self, n_decode: int, span: int, act_dtype: torch.dtype = torch.bfloat16) -> tuple[int, bool]:
        """(splits, False): into how many parts the keys of a decoded request are cut, each part a
        block that serves all heads.  Enough parts to give every SM a block, none shorter than
        64 keys."""
        if n_decode == 0 or not K.latent_decode_fits(self.num_heads, self.kv_rank, self.row_width):
            return 1, False
        sms = K.sm_count()
        return max(1, min(span // 64, -(-sms // n_decode), 64)), False

    def decode_plan(self, ctx) -> tuple[int, bool]:
        return self.decode_plan_for(ctx.n_decode, ctx.max_kv_len, ctx.act_dtype)

    def launch_key(self, ctx) -> tuple:
        return (step_decode_plan(self, ctx) if ctx.n_decode else None,)

    def forward(self, ctx, run, h, x, add: bool = True) -> None:
        n, H, W, rank = ctx.n_tokens, self.num_heads, self.row_width, self.kv_rank
        ws, act = ctx.workspace, ctx.act_dtype
        freq = self.rotary.frequencies(ctx.device)
        pool = ctx.kv_pool(run.cache_key)
        table = ctx.block_table(run.cache_key)
        q = ws.get("latent_q", (n, H * self.head_in), act)
        off, proj = self.offsets, None
        if run.writes_cache or len(off) > 1:
            proj = ws.get("latent_proj", (n, self.proj_weight.shape[0]), torch.float32)
            K.linear(h, self.proj_weight, None, proj)
        if self.q_rank is None:
            K.linear(h, self.q_weight, None, q)
        else:  # the queries' latent: normalised in float32, rounded once for the product with W_uq
            if self.q_rank_padded != self.q_rank:
                cq_buf = ws.get_zeroed(f"latent_cq_{self.q_rank}", (n, self.q_rank_padded), act)
            else:
                cq_buf = ws.get("latent_cq", (n, self.q_rank_padded), act)
            K.rmsnorm(proj[:, off["dq"]:off["dq"] + self.q_rank], self.dq_norm, self.norm_eps, cq_buf[:, :self.q_rank])
            K.linear(cq_buf, self.q_weight, None, q)
        if run.writes_cache:
            dkv = proj[:, off["dkv"]:off["dkv"] + rank + self.rot_dim]
            K.latent_kv_write(dkv, self.dkv_norm, self.norm_eps, freq, self.rotary.dims, pool, table, ctx.positions,
                              ctx.req_of_token, ctx.slots, rank=rank, rot_dim=self.rot_dim,
                              max_pos=ctx.cache.max_seq_len, rot_mult=self.rotary.mult)
        # the query rows [q_plain W_uk | rotated part] of every head
        rows = ws.get("latent_q_rows", (n, H * W), act)
        K.head_linear(q, self.uk_weight, rows, n_tokens=n, n_heads=H, k=self.plain_dim, n=rank,
                      in_strides=(q.stride(0), self.head_in), w_strides=(self.plain_dim * rank, 1, self.plain_dim),
                      out_strides=(H * W, W))
        K.latent_q_rope(q, rows, freq, ctx.positions, n_heads=H, head_in=self.head_in, plain=self.plain_dim,
                        rank=rank, rot_dim=self.rot_dim, rot_dims=self.rotary.dims, row_width=W,
                        rot_mult=self.rotary.mult)
        o_lat = ws.get("latent_o", (n, H * rank), act)
        by_request = ctx.n_decode > 0 and K.latent_decode_fits(H, rank, W)
        splits = step_decode_plan(self, ctx)[0] if by_request else 1
        part_o = part_ml = None
        if splits > 1:
            parts = ctx.n_decode * H * splits
            part_o = ws.get("latent_part_o", (parts, rank), torch.float32)
            part_ml = ws.get("latent_part_ml", (parts, 2), torch.float32)
        K.latent_attention(rows, pool, table, ctx.q_start, ctx.kv_len, ctx.slots, o_lat, sink=self.sink, n_heads=H,
                           rank=rank, scale=self.scale, tiles=ctx.tiles, n_tiles=ctx.n_tiles,
                           decode_reqs=ctx.decode_reqs, n_decode=ctx.n_decode, decode_by_request=by_request,
                           n_splits=splits, part_o=part_o, part_ml=part_ml)
        # the heads' values: (sum of probabilities x latents) W_uv,h^T, then the output product
        if self.heads_padded != self.heads_width:
            o = ws.get_zeroed(f"latent_heads_{self.heads_width}", (n, self.heads_padded), act)
        else:
            o = ws.get("latent_heads", (n, self.heads_padded), act)
        gate, gate_strides = None, (0, 0)
        if self.has_gate:  # the merged heads' gate rides on the product that makes them
            gate, gate_strides = proj[:, off["g"]:off["g"] + self.heads_width], (proj.stride(0), self.value_dim)
        K.head_linear(o_lat, self.uv_weight, o, n_tokens=n, n_heads=H, k=rank, n=self.value_dim,
                      in_strides=(H * rank, rank), w_strides=(self.value_dim * rank, 1, rank),
                      out_strides=(self.heads_padded, self.value_dim), gate=gate, gate_strides=gate_strides)
        K.linear(o, self.o_weight, None, x, residual=add)


def K_fits(n_heads: int, rank: int, row_width: int) -> bool:
    """The kernels' size limits, as plain arithmetic (no device is asked): latents up to 512
    entries, and a tile of 16 query rows and 32 cached rows in 200 KB of shared memory."""
    if rank > 512 or row_width < rank or row_width % 8:
        return False
    return (16 * row_width + 32 * (row_width + 1)) * 4 <= 200 * 1024
