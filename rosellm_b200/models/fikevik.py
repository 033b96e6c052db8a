"""Fikevik as a list of parts.

A decoder-only model whose layers normalise the stream itself: ``x <- norm(alpha x + gate * sublayer(x))`` for
the mixer and then for the feed-forward, the gate a sigmoid of a product of the sublayer's input.  The mixer is
either linear attention with a decay per key channel (``gla``), or two mixers side by side on the same input
whose results are summed with a weight each (``parallel``): softmax attention over the latest keys (normed and
rotated queries and keys, unit values, a temperature per head) and a matrix memory with exponential gates.  A
layer may use another layer's tensors with a cache and state of its own.  The token rows are scaled on their way
into the stream; a final RMS norm and a head of its own.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.rg1``,
``l<i>.rg1.b``, ``l<i>.rg2``, ``l<i>.rg2.b``, ``l<i>.mlp.{gate,up,down}``, and ``l<i>.mix.*`` (gla: ``q, k, v, g,
o, norm, a1, a2, a2.b``; parallel: ``left.{q, k, v, o, q.norm, k.norm, temp}`` and ``right.{q, k, v, g, o, norm,
i, i.b, f, f.b}``).  Linear weights are stored [out, in].
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.fikevik import FikevikConfig
from ..parts.spec import Concat, LayerSpec, ModelSpec, PartSpec, RunEntry

MEMORY_FLOOR_EPS = 1e-6  # matrix memory: added to the output's divisor


def build_fikevik_spec(cfg: FikevikConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps

    def join(norm: str, gate: str) -> PartSpec:
        return PartSpec("gated_join_norm", dict(hidden_size=width, eps=eps, alpha=cfg.postln_alpha, gate=True),
                        {"weight": norm, "gate_weight": gate, "gate_bias": gate + ".b"})

    layers, index_of = [], {}
    for i, lc in enumerate(cfg.layers):
        if lc.weights_of is not None:
            continue
        index_of[i] = len(layers)
        p, mx = f"l{i}.", lc.mixer
        if lc.type == "gla":
            m = p + "mix."
            named = dict(mixer=("mixer", PartSpec(
                "decayed_linear_attention",
                dict(hidden_size=width, num_heads=mx.heads, key_dim=mx.dim, value_dim=mx.vdim, tau=mx.tau, norm_eps=eps,
                     low_rank=mx.decay_rank),
                {"q_weight": m + "q", "k_weight": m + "k", "v_weight": m + "v", "g_weight": m + "g", "a1_weight": m + "a1",
                 "a2_weight": m + "a2", "a_bias": m + "a2.b", "out_norm": m + "norm", "out_weight": m + "o"})))
            mixers = (("mixer", 1.0),)
        else:  # parallel
            l, r = p + "mix.left.", p + "mix.right."
            named = dict(
                left=("mixer", PartSpec(
                    "window_attention",
                    dict(hidden_size=width, num_heads=mx.left.heads, num_kv_heads=mx.left.kv_heads, key_dim=mx.left.dim,
                         value_dim=mx.left.vdim, scale=mx.left.scale, norm_eps=eps, window=mx.left.window,
                         rot_dims=mx.left.rot_dims, rot_base=mx.left.rot_base, qk_norm=True, unit_values=True,
                         head_temperature=True),
                    {"q_weight": l + "q", "k_weight": l + "k", "v_weight": l + "v", "out_weight": l + "o",
                     "q_norm": l + "q.norm", "k_norm": l + "k.norm", "head_temp": l + "temp"})),
                right=("mixer", PartSpec(
                    "matrix_memory",
                    dict(hidden_size=width, num_heads=mx.right.heads, key_dim=mx.right.dim, value_dim=mx.right.vdim,
                         gate_cap=mx.right.gate_cap, norm_eps=eps, floor_eps=MEMORY_FLOOR_EPS),
                    {"q_weight": r + "q", "k_weight": r + "k", "v_weight": r + "v", "g_weight": r + "g",
                     "i_weight": r + "i", "f_weight": r + "f", "i_bias": r + "i.b", "f_bias": r + "f.b",
                     "out_norm": r + "norm", "out_weight": r + "o"})))
            mixers = (("left", mx.left_scale), ("right", mx.right_scale))
        named["join_mixer"] = ("norm", join(p + "norm1", p + "rg1"))
        if lc.ff is not None:
            named["feed_forward"] = ("feed_forward", PartSpec(
                "gated_mlp", dict(hidden_size=width, inner_size=lc.ff, gate="silu"),
                {"gate_up_weight": Concat((p + "mlp.gate", p + "mlp.up"), dim=0), "down_weight": p + "mlp.down"}))
            named["join_feed_forward"] = ("norm", join(p + "norm2", p + "rg2"))
        layers.append(LayerSpec.of(PartSpec("post_norm_gated", dict(mixers=mixers, feed_forward=lc.ff is not None)), **named))
    # every layer of the configuration is one run under its own number: of its own parts, or of the parts of the
    # layer whose tensors it uses
    run_order = tuple(RunEntry(index_of[cfg.weight_owner(i)], instance=i) for i in range(len(cfg.layers)))
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, hidden_size=width, scale=cfg.embedding_scale),
                           {"weight": "embed"}),
        position=PartSpec("none"),
        layers=tuple(layers),
        run_order=run_order,
        final_norm=PartSpec("rms_norm", dict(hidden_size=width, eps=eps), {"weight": "final.norm"}),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=width), {"weight": "head"}),
        eos_token_id=cfg.eos_token_id,
    )


register_architecture("Fikevik", FikevikConfig, build_fikevik_spec, model_types=("fikevik",), replace=True)
