"""The parts this package ships: what GPT-2 is assembled from.

Each part takes its sizes and constants as constructor parameters and calls
the sm_100a kernels through ``rosellm_b200.ops.kernels``.  The residual
stream ``x`` is float32 ``[tokens, hidden]`` in both precisions; activations
between a norm and a matrix product are in the compute dtype.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import KVCacheSpec, ParamSpec, Part, StateSpec, register_part


@register_part("position", "none")
class NoPositions(Part):
    """No position information is added anywhere."""

    graph_safe = True
    launches_replayable = True
    rotates = False  # rotate() changes nothing: keys may go to the cache straight from the qkv product

    def table(self):
        return None

    def rotate(self, ctx, q, k) -> None:
        return None


@register_part("position", "learned_absolute")
class LearnedAbsolutePositions(Part):
    """A learned table added to the token embedding: ``x = wte[id] + wpe[pos]``
    (rosellm/rosetrainer/model.py:543-562)."""

    graph_safe = True
    launches_replayable = True
    rotates = False

    def __init__(self, max_positions: int, hidden_size: int) -> None:
        self.max_positions = max_positions
        self.hidden_size = hidden_size
        self.weight = None

    def param_specs(self):
        return [ParamSpec("weight", (self.max_positions, self.hidden_size))]

    def table(self):
        return self.weight

    def rotate(self, ctx, q, k) -> None:
        return None


def rotary_frequencies(dims: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i/dims) for the pairs i = 0 .. dims/2 - 1, evaluated in float64 and kept
    in float32 (the kernels form the angle position * f_i in float32)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(torch.float32)


ROTARY_SCALINGS = ("wavelength", "ramp")


def scaled_rotary_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[torch.Tensor, float]:
    """(frequencies, factor of the cosines and sines) of a rotation whose frequencies are stretched for
    sequences longer than ``scaling["original"]`` positions; float64 arithmetic, float32 result.

    ``kind`` ``"wavelength"`` (``factor``, ``low``, ``high``, ``original``): a pair whose wavelength l = 2 pi / f
    is below original / high keeps f; above original / low it turns ``factor`` times slower; between, with
    s = (original / l - low) / (high - low), it gets (1 - s) f / factor + s f.

    ``kind`` ``"ramp"`` (``factor``, ``original``, ``fast``, ``slow``): with index(t) = dims ln(original / (2 pi t)) /
    (2 ln base), lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), dims - 1) and r_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1), pair i gets r_i f_i / factor + (1 - r_i) f_i; cosines and sines are multiplied by
    0.1 ln(factor) + 1."""
    import math

    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return torch.tensor(f, dtype=torch.float64).to(torch.float32), 1.0
    kind = scaling.get("kind")
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if factor <= 0 or original <= 0:
        raise ValueError("rotary scaling: factor and original must be positive")
    mult = 1.0
    if kind == "wavelength":
        low, high = float(scaling["low"]), float(scaling["high"])
        if high == low:
            raise ValueError("rotary scaling: low and high must differ")
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < original / high:
                out.append(fi)
            elif wave > original / low:
                out.append(fi / factor)
            else:
                s = (original / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    elif kind == "ramp":
        fast, slow = float(scaling["fast"]), float(scaling["slow"])
        if fast <= 0 or slow <= 0 or base == 1.0:
            raise ValueError("rotary scaling: fast and slow must be positive and the base not 1")

        def index_of(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(index_of(fast)), 0)
        hi = min(math.ceil(index_of(slow)), dims - 1)
        ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(len(f))]
        f = [fi / factor * r + fi * (1.0 - r) for fi, r in zip(f, ramp)]
        mult = 0.1 * math.log(factor) + 1.0
    else:
        raise ValueError(f"rotary scaling kind {kind!r}; one of {ROTARY_SCALINGS}")
    return torch.tensor(f, dtype=torch.float64).to(torch.float32), mult


@register_part("position", "rotary")
class RotaryPositions(Part):
    """Rotation of queries and keys by their positions: of every head's ``head_dim`` entries the
    first ``dims`` are turned, entry 2i with entry 2i+1 (the interleaved layout) by the angle
    position * base^(-2i/dims); the rest pass unchanged.  Angles and rotation in float32.
    ``scaling`` (a dict with ``kind`` and the kind's constants: ``scaled_rotary_frequencies``) stretches the
    frequencies; ``mult`` is then the factor of the cosines and sines that the kind asks for (1 otherwise).

    A mixer whose rotation has constants of its own builds one for itself (``RotaryPositions(
    dims=..., base=...)``) and asks it for ``frequencies(device)``; as a model's ``position``
    part it has no table for the embedding to add."""

    graph_safe = True
    launches_replayable = True
    rotates = True

    def __init__(self, dims: int, base: float, scaling: dict | None = None) -> None:
        if dims < 0 or dims % 2:
            raise ValueError(f"rotary dims {dims}: pairs are turned, the count must be even")
        if base <= 0:
            raise ValueError(f"rotary base {base} must be positive")
        self.dims, self.base = int(dims), float(base)
        self.scaling = dict(scaling) if scaling else None
        self._host, self.mult = None, 1.0
        if self.scaling is not None:
            self._host, self.mult = scaled_rotary_frequencies(max(self.dims, 2), self.base, self.scaling)
        self._freq: dict = {}

    def table(self):
        return None

    def frequencies(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._freq:
            host = self._host if self._host is not None else rotary_frequencies(max(self.dims, 2), self.base)
            self._freq[key] = host.to(device)
        return self._freq[key]


@register_part("embedding", "token_table")
class TokenEmbedding(Part):
    graph_safe = True
    launches_replayable = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0) -> None:
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.scale = float(scale)  # the token's row is multiplied by it (in float32, on its way into the stream)
        self.weight = None

    def param_specs(self):
        return [ParamSpec("weight", (self.vocab_size, self.hidden_size))]

    def forward(self, ctx, position) -> torch.Tensor:
        x = ctx.workspace.get("residual", (ctx.n_tokens, self.hidden_size), torch.float32)
        K.embed(ctx.token_ids, ctx.positions, self.weight, position.table(), x, ctx.extras.get("token_feedback"),
                scale=self.scale)
        return x


@register_part("embedding", "token_pair_table")
class TokenPairEmbedding(Part):
    """``x = table[token] + pair_table[(previous token * mul_prev + token * mul_cur) mod buckets]`` (+ the
    position table's row): a second, hashed table indexed by the pair of neighbouring tokens; a
    sequence's first token has no pair and takes row ``buckets``, which the table holds beyond its buckets.

    The previous token of a portion's first token is the request's own state (one int32 in its
    state slot, kept up to date by the kernel), so a prompt may be cut anywhere."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int) -> None:
        if buckets <= 0:
            raise ValueError("token pair table: buckets must be positive")
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.weight = self.pair_weight = None

    def param_specs(self):
        return [ParamSpec("weight", (self.vocab_size, self.hidden_size)),
                ParamSpec("pair_weight", (self.buckets + 1, self.hidden_size))]

    def state_spec(self):
        return StateSpec((1,), torch.int32)

    def forward(self, ctx, position) -> torch.Tensor:
        x = ctx.workspace.get("residual", (ctx.n_tokens, self.hidden_size), torch.float32)
        K.embed_pair(ctx.token_ids, ctx.positions, ctx.req_of_token, ctx.q_start, ctx.slots, self.weight,
                     position.table(), self.pair_weight, x, ctx.state("embedding"), buckets=self.buckets,
                     mul_prev=self.mul_prev, mul_cur=self.mul_cur, feedback=ctx.extras.get("token_feedback"))
        return x


@register_part("norm", "layer_norm")
class LayerNorm(Part):
    """``(x - mean) * rsqrt(var + eps) * weight + bias`` over the last dimension
    (rosellm/rosetrainer/fused_layernorm.py:99-120)."""

    graph_safe = True
    launches_replayable = True
    can_defer = True  # forward(..., defer=True) may hand the consumer a K.NormInput to fuse

    def __init__(self, hidden_size: int, eps: float, bias: bool = True) -> None:
        self.hidden_size = hidden_size
        self.eps = eps
        self.has_bias = bias
        self.weight = None
        self.bias = None

    def param_specs(self):
        specs = [ParamSpec("weight", (self.hidden_size,), kind="vector", init="ones")]
        if self.has_bias:
            specs.append(ParamSpec("bias", (self.hidden_size,), kind="vector", init="zeros"))
        return specs

    def forward(self, ctx, x, rows=None, n_rows=None, name="normed", defer: bool = False):
        """Normalised rows in the activation dtype.  With ``defer`` (the consumer has declared
        ``takes_norm_input``) and few, short rows in bfloat16, a ``K.NormInput`` instead: the
        consumer's first product normalises inside its own kernel and no kernel runs here."""
        if defer and rows is None and K.NormInput.possible(x.shape[0], self.hidden_size, ctx.act_dtype):
            return K.NormInput(x, self.weight, self.bias, self.eps)
        n = x.shape[0] if rows is None else int(n_rows)
        out = ctx.workspace.get(name, (n, self.hidden_size), ctx.act_dtype)
        K.layernorm(x, self.weight, self.bias, self.eps, out, rows)
        return out


@register_part("norm", "rms_norm")
class RMSNorm(Part):
    """``x / sqrt(mean(x^2) + eps) * (weight_offset + weight)`` over the last dimension, in float32
    (``weight_offset`` 1 for scales kept as offsets from one; the sum is formed once, when the
    weights are bound).  ``out_scale``: a constant that the normalised rows are multiplied by on their way
    out (a model whose logits are its head's product times a constant gives it to its final norm: the head is
    linear); it too goes into the weight once, in float32.

    ``forward`` normalises rows of the stream for a consumer (a head, a pre-norm block).
    ``add_to`` serves blocks that normalise a sublayer's output instead of its input:
    ``stream += mult * norm(y)``, leaving (bfloat16 mode) the rounded new rows in ``copy`` for the
    next sublayer's products."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, hidden_size: int, eps: float, weight_offset: float = 0.0, out_scale: float = 1.0) -> None:
        if eps <= 0:
            raise ValueError("the norm's eps must be positive")
        self.hidden_size = hidden_size
        self.eps = float(eps)
        self.weight_offset = float(weight_offset)
        self.out_scale = float(out_scale)
        self.weight = None

    def param_specs(self):
        return [ParamSpec("weight", (self.hidden_size,), kind="vector", init="zeros" if self.weight_offset else "ones")]

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.weight_offset:
            self.weight = self.weight + self.weight_offset
        if self.out_scale != 1.0:
            self.weight = self.weight * self.out_scale

    def forward(self, ctx, x, rows=None, n_rows=None, name="normed", defer: bool = False):
        n = x.shape[0] if rows is None else int(n_rows)
        out = ctx.workspace.get(name, (n, self.hidden_size), ctx.act_dtype)
        K.rmsnorm(x, self.weight, self.eps, out, rows)
        return out

    def add_to(self, ctx, y, x, mult: float, copy=None) -> None:
        K.rmsnorm_add(y, self.weight, self.eps, x, mult, copy)

    def add_then_norm(self, ctx, y, x, following: "RMSNorm", name: str = "normed"):
        """``x += norm(y)`` and, in the same pass, the new rows normalised by ``following`` (the norm
        ahead of the next sublayer) in the activation dtype."""
        out = ctx.workspace.get(name, tuple(x.shape), ctx.act_dtype)
        if self.hidden_size > K.RMSNORM_ADD_NORM_MAX_WIDTH:
            K.rmsnorm_add(y, self.weight, self.eps, x, 1.0, None)
            K.rmsnorm(x, following.weight, following.eps, out)
        else:
            K.rmsnorm_add_norm(y, self.weight, self.eps, x, following.weight, following.eps, out)
        return out


_NARROW_PARTS: dict[tuple, int] = {}  # (request-head pairs, keys, bytes a key, blocks at once) -> parts, as computed before


def narrow_decode_blocks_at_once(head_dim: int, element_bytes: int, percent: int = 50) -> int:
    """How many four-warp blocks of the decode attention run at once on the device: each holds
    a ring of two tiles of keys and values per warp in shared memory (csrc/attention_kernels.cuh,
    ``DecodeTile``: 4 warps x 2 stages x 2 x the tile's words), and every small kernel of the
    library asks for half of an SM's memory as shared memory.  ``percent``: the denser forms of
    the kernel ask for 80 % or all of it (taken when the blocks would not run at once otherwise)."""
    words = head_dim // 8 * element_bytes // 4
    sub = 4 if words <= 4 else (2 if words <= 8 else 1)
    block = 4 * 2 * 2 * sub * 32 * words * 4 + 1024  # the ring, and what the driver keeps per block
    sms, shared = K.device_facts()
    return sms * max(1, min(16, (shared * percent // 100) // block))


# The forms of the narrow kernel: (share of an SM's memory as shared memory, what a key costs a
# block against the common form; less L1 is left beside the shared memory).  Measured at 40, 48
# and 64 requests of 512 keys: 13.6, 14.0 us (80 %: five blocks an SM) and 18.2 us (all of it:
# six) in one round against 18.4, 19.7 and 20.6 us in two rounds of the common form; 48 requests
# of 1024 keys: 29.7 us whole, 35.5 in two parts, 32.1 in three.
NARROW_FORMS = ((50, 1.0), (80, 1.15), (100, 1.3))


# Longest context of a step from which prompt portions go to the tcgen05 attention kernel
# (measured on B200, 12 heads of 64: 48 against 56 TFLOP/s at 256 tokens, 101 against 86 at
# 1024, 131 against 96 at 2048).
TC_ATTENTION_MIN_CONTEXT = 512


@register_part("mixer", "causal_self_attention")
class CausalSelfAttention(Part):
    """Multi-head causal attention over the paged cache.

    ``qkv = h W_qkv + b``, columns split into queries, keys and values in that
    order, head ``j // head_dim`` owning column ``j`` of each
    (rosellm/rosetrainer/model.py:95-98, 248-255); the step's keys and values
    are written to the cache, then every query attends over the cached keys
    up to its own position (csrc/attention.cu); heads are merged and
    ``x += o W_out + b`` (model.py:218-221, 412-413).
    """

    graph_safe = True
    launches_replayable = True
    takes_norm_input = True  # h may be a K.NormInput: the qkv product then normalises its own input

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, num_kv_heads: int | None = None,
                 window: int | None = None, scale: float | None = None, bias: bool = True,
                 weights_in_out: bool = False) -> None:
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        self.head_dim = head_dim
        self.window = window
        self.scale = scale if scale is not None else head_dim ** -0.5
        self._split = (None, None, None, None)  # the packed qkv buffer last seen and its three views
        self.has_bias = bias
        self.weights_in_out = weights_in_out
        if head_dim % 16 != 0 or head_dim > 256:
            raise ValueError(f"head size {head_dim}: the attention kernels take multiples of 16 up to 256")
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{num_heads} heads are not a multiple of {self.num_kv_heads} key/value heads")
        self.q_width = self.num_heads * head_dim
        self.kv_width = self.num_kv_heads * head_dim
        self.qkv_weight = self.qkv_bias = self.out_weight = self.out_bias = None
        self._out_weight_packed = None

    def _matrix(self, role, n_out, n_in):
        shape = (n_in, n_out) if self.weights_in_out else (n_out, n_in)
        return ParamSpec(role, shape, transpose=self.weights_in_out)

    def param_specs(self):
        qkv = self.q_width + 2 * self.kv_width
        specs = [self._matrix("qkv_weight", qkv, self.hidden_size),
                 self._matrix("out_weight", self.hidden_size, self.q_width)]
        if self.has_bias:
            specs += [ParamSpec("qkv_bias", (qkv,), kind="vector"),
                      ParamSpec("out_bias", (self.hidden_size,), kind="vector")]
        return specs

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def decode_plan_for(self, n_decode: int, span: int, act_dtype: torch.dtype = torch.bfloat16) -> tuple[int, bool]:
        """(splits, wide): over how many blocks the keys of one decoded request are split when
        ``n_decode`` requests attend over about ``span`` keys each, and whether the blocks have
        sixteen warps instead of four.  With few requests wide blocks take 256 keys a round, so
        that a request's keys need no split and no merge; with many, narrow blocks fill the SMs."""
        if n_decode == 0:
            return 1, False
        if self.window is not None:
            span = min(span, self.window)
        units = n_decode * self.num_heads
        sms = K.sm_count()
        if units <= 2 * sms:
            return max(1, min(span // 1024, 2 * sms // units, 32)), True   # up to four rounds a block
        # Narrow blocks: a few fit on an SM (shared memory); where they do not all run at once the
        # kernel takes its dense form (twice as many an SM, each slower), and what is still left
        # waits for a second round.
        # Measured on B200 with 12 heads of 64 in bfloat16 (three blocks an SM, 256 bytes a key):
        # a round costs about 0.8 us + 0.0152 us a key, and a split adds the merge kernel,
        # 6 us + 1 us a part (32 x 512: 10.3 us whole against 15.7 us in two parts).  Other head
        # sizes and the 32-bit cache scale the cost of a key by the bytes it takes, and change
        # how many blocks fit.
        element_bytes = 2 if act_dtype == torch.bfloat16 else 4
        key_bytes = 2 * self.head_dim * element_bytes
        at_once = narrow_decode_blocks_at_once(self.head_dim, element_bytes)
        span = -(-span // 64) * 64  # in steps of 64 keys: every layer of a step, and most steps, ask the same
        best = _NARROW_PARTS.get((units, span, key_bytes, at_once))
        if best is None:
            best_cost, best = None, 1
            per_key = 0.0152 * key_bytes / 256.0
            forms = [(narrow_decode_blocks_at_once(self.head_dim, element_bytes, pc), f) for pc, f in NARROW_FORMS]
            for parts in range(1, min(span // 64, 32) + 1):
                # the form the kernel takes (csrc/attention_kernels.cuh: launch_decode): the
                # first that holds all blocks at once, else the densest
                room, factor = next(((r, f) for r, f in forms if units * parts <= r), forms[-1])
                rounds, key_cost = -(-units * parts // room), per_key * factor
                cost = rounds * (0.8 + key_cost * span / parts) + (6.0 + 1.0 * parts if parts > 1 else 0.0)
                if best_cost is None or cost < best_cost - 1e-9:
                    best_cost, best = cost, parts
            if len(_NARROW_PARTS) > 4096:
                _NARROW_PARTS.clear()
            _NARROW_PARTS[(units, span, key_bytes, at_once)] = best
        return best, False

    def decode_plan(self, ctx) -> tuple[int, bool]:
        return self.decode_plan_for(ctx.n_decode, ctx.max_kv_len, ctx.act_dtype)

    @staticmethod
    def _tc_prompt_attention(ctx) -> bool:
        """Whether the step's prompt portions go to the tcgen05 kernel: decided by the longest
        context among the requests that bring portions (decoded requests beside them have
        nothing to do with it)."""
        return ctx.max_tile_kv_len >= TC_ATTENTION_MIN_CONTEXT

    def launch_key(self, ctx) -> tuple:
        """The longest context decides how decoded requests are split over blocks and which
        kernel takes the prompt portions."""
        return (ctx.extras.get("decode_plan") or self.decode_plan(ctx) if ctx.n_decode else None,
                self._tc_prompt_attention(ctx) if ctx.n_tiles else None)

    def bind(self, tensors) -> None:
        super().bind(tensors)
        # the fused kernel of a decode step reads W_out slice by slice: laid out for it once, here
        self._out_weight_packed = None
        w = self.out_weight
        if (w is not None and w.is_cuda and self.window is None and self.num_kv_heads == self.num_heads
                and self.q_width == self.hidden_size):
            cluster = K.attn_block_fused_cluster(self.hidden_size, self.num_heads, self.head_dim, w.dtype)
            if cluster:
                self._out_weight_packed = K.attn_pack_out_weight(w, self.num_heads, self.head_dim, cluster)

    def _fused_decode(self, ctx, run, h, x) -> bool:
        """A step of few decoded requests and nothing else: the whole of this part (its norm
        included) in one kernel, where the sizes fit."""
        n = ctx.n_tokens
        return (self._out_weight_packed is not None and K.FUSED_ROWS and n <= 16
                and isinstance(h, K.NormInput) and h.x is x and n == ctx.n_decode == ctx.n_reqs and run.writes_cache
                and not getattr(ctx.position, "rotates", True))

    def forward(self, ctx, run, h, x, add: bool = True) -> None:
        if add and self._fused_decode(ctx, run, h, x):
            K.attn_block_fused(x, h, self.qkv_weight, self.qkv_bias, self._out_weight_packed, self.out_bias,
                               ctx.kv_pool(run.cache_key), ctx.block_table(run.cache_key), ctx.positions, ctx.slots,
                               n_heads=self.num_heads, scale=self.scale, max_pos=ctx.cache.max_seq_len)
            return
        n = ctx.n_tokens
        qkv_w = self.q_width + 2 * self.kv_width
        qkv = ctx.workspace.get("qkv", (n, qkv_w), ctx.act_dtype)
        pool = ctx.kv_pool(run.cache_key)
        table = ctx.block_table(run.cache_key)
        # keys and values can go to their pages straight from the product when nothing has to
        # touch them in between (no rotation) and the product runs the row kernel
        fuse_write = (run.writes_cache and not getattr(ctx.position, "rotates", True)
                      and K.product_writes_cache(n, ctx.act_dtype, qkv_w, self.hidden_size))
        target = None
        if fuse_write:
            target = K.KvTarget(pool, table, ctx.positions, ctx.req_of_token, ctx.slots, self.q_width,
                                ctx.cache.max_seq_len)
        K.linear(h, self.qkv_weight, self.qkv_bias, qkv, kv=target)
        if self._split[0] is not qkv:  # the workspace hands out one tensor object per size
            self._split = (qkv, qkv[:, : self.q_width], qkv[:, self.q_width: self.q_width + self.kv_width],
                           qkv[:, self.q_width + self.kv_width:])
        _, q, k, v = self._split
        if not fuse_write:
            ctx.position.rotate(ctx, q, k)
            if run.writes_cache:
                K.kv_write(k, v, pool, table, ctx.positions, ctx.req_of_token, ctx.slots, ctx.cache.max_seq_len)
        o = ctx.workspace.get("attn_out", (n, self.q_width), ctx.act_dtype)
        splits, wide = ctx.extras.get("decode_plan") or self.decode_plan(ctx)
        part_o = part_ml = None
        if splits > 1:
            rows = ctx.n_decode * self.num_heads * splits
            part_o = ctx.workspace.get("attn_part_o", (rows, self.head_dim), torch.float32)
            part_ml = ctx.workspace.get("attn_part_ml", (rows, 2), torch.float32)
        K.attention(q, pool, table, ctx.q_start, ctx.kv_len, ctx.slots, o, n_heads=self.num_heads,
                    scale=self.scale, window=self.window, tiles=ctx.tiles, n_tiles=ctx.n_tiles,
                    decode_reqs=ctx.decode_reqs, n_decode=ctx.n_decode, n_splits=splits,
                    part_o=part_o, part_ml=part_ml, tiles_wide=ctx.tiles_wide, n_tiles_wide=ctx.n_tiles_wide,
                    decode_wide=wide,
                    # what decoded requests read of the cache beside their newest key is of earlier
                    # steps, and a step begins with a copy to the device that separates it from them
                    old_keys_settled=True,
                    # prompt portions: the tcgen05 kernel (where its sizes fit) wins once a block
                    # walks several tiles of keys; short contexts are faster on mma.sync
                    prefill_path=None if self._tc_prompt_attention(ctx) else "mma")
        K.linear(o, self.out_weight, self.out_bias, x, residual=add)


@register_part("feed_forward", "dense_mlp")
class DenseMLP(Part):
    """``x += act(h W_in + b_in) W_out + b_out`` (rosellm/rosetrainer/model.py:331-349);
    ``activation`` is ``gelu_tanh`` (model.py:274-277) or ``gelu_erf`` (``F.gelu``)."""

    graph_safe = True
    launches_replayable = True
    takes_norm_input = True

    def __init__(self, hidden_size: int, inner_size: int, activation: str, bias: bool = True,
                 weights_in_out: bool = False) -> None:
        if activation not in K.ACTIVATIONS or activation == "none":
            raise ValueError(f"activation {activation!r}; one of gelu_tanh, gelu_erf")
        self.hidden_size = hidden_size
        self.inner_size = inner_size
        self.activation = K.ACTIVATIONS[activation]
        self.has_bias = bias
        self.weights_in_out = weights_in_out
        self.in_weight = self.in_bias = self.out_weight = self.out_bias = None
        self._fused_slice, self._out_weight_packed = 0, None

    def _matrix(self, role, n_out, n_in):
        shape = (n_in, n_out) if self.weights_in_out else (n_out, n_in)
        return ParamSpec(role, shape, transpose=self.weights_in_out)

    def param_specs(self):
        specs = [self._matrix("in_weight", self.inner_size, self.hidden_size),
                 self._matrix("out_weight", self.hidden_size, self.inner_size)]
        if self.has_bias:
            specs += [ParamSpec("in_bias", (self.inner_size,), kind="vector"),
                      ParamSpec("out_bias", (self.hidden_size,), kind="vector")]
        return specs

    def bind(self, tensors) -> None:
        """The products read rows in 16-byte pieces, so an inner size that is no multiple of 8
        is filled up with units whose weights and bias are zero: their activation is 0 (both
        GELU forms map 0 to 0) and they add nothing to the output."""
        super().bind(tensors)
        pad = -self.inner_size % 8
        self.inner_padded = self.inner_size + pad
        if pad:
            self.in_weight = torch.nn.functional.pad(self.in_weight, (0, 0, 0, pad)).contiguous()
            self.out_weight = torch.nn.functional.pad(self.out_weight, (0, pad)).contiguous()
            if self.in_bias is not None:
                self.in_bias = torch.nn.functional.pad(self.in_bias, (0, pad)).contiguous()
        # the fused kernel of few rows reads W_out slice by slice: laid out for it once, here
        self._fused_slice, self._out_weight_packed = 0, None
        if self.out_weight.is_cuda:
            self._fused_slice = K.mlp_fused_slice(1, self.hidden_size, self.inner_padded, True, self.out_weight.dtype)
            if self._fused_slice:
                self._out_weight_packed = K.mlp_pack_out_weight(self.out_weight, self._fused_slice)

    def forward(self, ctx, h, x, add: bool = True) -> None:
        # few rows: both products in one kernel, the inner activations never leave the SM
        width = self._fused_slice if add and ctx.n_tokens <= 16 and K.FUSED_ROWS else 0
        if width:
            K.mlp_fused(x, h, self.in_weight, self.in_bias, self._out_weight_packed, self.out_bias, act=self.activation,
                        slice_width=width)
            return
        u = ctx.workspace.get("mlp_inner", (ctx.n_tokens, self.inner_padded), ctx.act_dtype)
        K.linear(h, self.in_weight, self.in_bias, u, act=self.activation)
        K.linear(u, self.out_weight, self.out_bias, x, residual=add)


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))`` (rosellm/rosetrainer/model.py:372-428)."""

    graph_safe = True
    launches_replayable = True
    # the sub-parts of a layer this block arranges, by name and category
    uses = {"norm_mixer": "norm", "mixer": "mixer", "norm_feed_forward": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, run, layer, x) -> None:
        h = self._normed(ctx, layer.norm_mixer, x, layer.mixer)
        layer.mixer.forward(ctx, run, h, x)
        h = self._normed(ctx, layer.norm_feed_forward, x, layer.feed_forward)
        layer.feed_forward.forward(ctx, h, x)

    @staticmethod
    def _normed(ctx, norm, x, consumer):
        """The norm's output; between a norm that can defer and a consumer that takes it, the
        norm is handed over unevaluated for the consumer to fuse into its first product."""
        if getattr(norm, "can_defer", False) and getattr(consumer, "takes_norm_input", False):
            return norm.forward(ctx, x, defer=True)
        return norm.forward(ctx, x)


@register_part("block", "parallel_sublayers")
class ParallelSublayersBlock(Part):
    """One norm, both sublayers on its output: with ``h = norm(x)``, ``x += mixer(h) + feed_forward(h)`` (a layer
    may have no feed-forward).  Both sublayers end in a product that adds into the float32 stream, so the layer
    is the norm's kernel and the sublayers' own; nothing reads the stream between the two additions."""

    graph_safe = True
    launches_replayable = True

    # the sub-part whose output ``ctx.extras["normed_ahead"]`` stands for, when whatever wrote the stream last has
    # normalised its rows in the same launch
    takes_normed_ahead = "norm_input"

    def __init__(self, feed_forward: bool = True) -> None:
        self.has_feed_forward = bool(feed_forward)
        self.uses = {"norm_input": "norm", "mixer": "mixer"}
        if feed_forward:
            self.uses["feed_forward"] = "feed_forward"

    def forward(self, ctx, run, layer, x) -> None:
        h = ctx.extras.pop("normed_ahead", None)
        if h is None:
            h = layer.norm_input.forward(ctx, x)
        layer.mixer.forward(ctx, run, h, x)
        if self.has_feed_forward:
            layer.feed_forward.forward(ctx, h, x)


@register_part("block", "normed_sublayers")
class NormedSublayersBlock(Part):
    """Sublayers that read the stream itself and are normalised on the way back:
    ``x += mult * norm(sublayer(x))`` for the mixer, then (where the layer has them) for the
    feed-forward and for a token-gated input, each with a norm of its own.

    The sublayers' products read the stream in the activation dtype: the stream itself in the
    32-bit mode; in bfloat16 a rounded copy that the norm's kernel refreshes whenever it has
    added to the stream (``ctx.extras["stream_copy"]``; the first layer of a step makes it)."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, residual_mult: float = 1.0, feed_forward: bool = True, token_input: bool = False) -> None:
        self.mult = float(residual_mult)
        self.uses = {"mixer": "mixer", "norm_mixer": "norm"}
        if feed_forward:
            self.uses.update(feed_forward="feed_forward", norm_feed_forward="norm")
        if token_input:
            self.uses.update(token_input="feed_forward", norm_token_input="norm")
        self.has_feed_forward, self.has_token_input = feed_forward, token_input

    @staticmethod
    def _stream_input(ctx, x):
        if ctx.act_dtype == torch.float32:
            return x, None
        h = ctx.extras.get("stream_copy")
        if h is None:
            h = ctx.extras["stream_copy"] = ctx.workspace.get("stream_copy", tuple(x.shape), ctx.act_dtype)
            K.cast_rows(x, h)
        return h, h

    def forward(self, ctx, run, layer, x) -> None:
        h, copy = self._stream_input(ctx, x)
        y = ctx.workspace.get("sublayer_out", tuple(x.shape), torch.float32)
        layer.mixer.forward(ctx, run, h, y, add=False)
        layer.norm_mixer.add_to(ctx, y, x, self.mult, copy)
        if self.has_feed_forward:
            layer.feed_forward.forward(ctx, h, y, add=False)
            layer.norm_feed_forward.add_to(ctx, y, x, self.mult, copy)
        if self.has_token_input:
            layer.token_input.forward(ctx, h, y, add=False)
            layer.norm_token_input.add_to(ctx, y, x, self.mult, copy)


@register_part("block", "pre_post_norm")
class PrePostNormBlock(Part):
    """Norms on both sides of every sublayer: ``x += norm_out(mixer(norm(x)))``, then (where the layer has
    a feed-forward) ``x += norm_out(feed_forward(norm(x)))``, four norms of their own.  A norm behind a
    sublayer and the norm ahead of the next one (the feed-forward's, or the first norm of the layer that
    runs next) are one kernel: a layer launches two norm kernels, the model's first layer three."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, feed_forward: bool = True) -> None:
        self.has_feed_forward = bool(feed_forward)
        self.uses = {"norm_mixer": "norm", "mixer": "mixer", "norm_mixer_out": "norm"}
        if feed_forward:
            self.uses.update(norm_feed_forward="norm", feed_forward="feed_forward", norm_feed_forward_out="norm")

    def forward(self, ctx, run, layer, x) -> None:
        h = ctx.extras.pop("normed_ahead", None)  # left by the layer before, with its last addition to the stream
        if h is None:
            h = layer.norm_mixer.forward(ctx, x)
        y = ctx.workspace.get("sublayer_out", tuple(x.shape), torch.float32)
        layer.mixer.forward(ctx, run, h, y, add=False)
        last = layer.norm_mixer_out
        if self.has_feed_forward:
            fused = getattr(last, "add_then_norm", None)
            if fused is not None and isinstance(layer.norm_feed_forward, RMSNorm):
                h = fused(ctx, y, x, layer.norm_feed_forward)
            else:
                last.add_to(ctx, y, x, 1.0)
                h = layer.norm_feed_forward.forward(ctx, x)
            layer.feed_forward.forward(ctx, h, y, add=False)
            last = layer.norm_feed_forward_out
        # the layer's last addition to the stream, in one kernel with the first norm of the layer that runs next
        # where that layer is arranged the same way
        nxt = ctx.extras.get("next_layer")
        follow = getattr(nxt, "norm_mixer", None) if nxt is not None and isinstance(nxt.block, PrePostNormBlock) else None
        if isinstance(follow, RMSNorm) and hasattr(last, "add_then_norm"):
            ctx.extras["normed_ahead"] = last.add_then_norm(ctx, y, x, follow)
        else:
            last.add_to(ctx, y, x, 1.0)


@register_part("head", "tied_to_embedding")
class TiedHead(Part):
    """``logits = h wte^T`` with the embedding's own table, no bias
    (rosellm/rosetrainer/model.py:503-504, 639-641)."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, vocab_size: int, hidden_size: int) -> None:
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight = None  # set by the model to the embedding's table

    tied = True
    takes_norm_input = True  # h may be a K.NormInput: the product then normalises its own input

    def forward(self, ctx, h) -> torch.Tensor:
        n_rows = h.x.shape[0] if isinstance(h, K.NormInput) else h.shape[0]
        logits = ctx.workspace.get("logits", (n_rows, self.vocab_size), torch.float32)
        K.linear(h, self.weight, None, logits)
        return logits

    def can_sample(self, n_rows: int, dtype: torch.dtype, with_temperature: bool = False) -> bool:
        """Whether ``forward_sample`` should be given this many rows (some of them with a
        temperature, or all taking the arg-max): a head that can choose the next tokens inside
        its product writes no logits for them."""
        return K.sampling_product_possible(n_rows, self.vocab_size, self.hidden_size, dtype, with_temperature)

    def forward_sample(self, ctx, h, into: "K.SampleInto") -> None:
        """The next token of every row of ``h`` into ``into.out_ids`` (arg-max, or by the rows'
        temperatures), chosen in the product's epilogue: what the sampling kernel would choose
        from ``forward``'s logits."""
        K.linear_sample(h, self.weight, None, into)


@register_part("head", "linear")
class LinearHead(TiedHead):
    """``logits = h W^T`` with a table of its own."""

    tied = False

    def param_specs(self):
        return [ParamSpec("weight", (self.vocab_size, self.hidden_size))]
