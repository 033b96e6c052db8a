"""Soporax as a list of parts.

A decoder-only model whose layers read one RMS norm of the stream with both sublayers and add both results:
``h = norm(x); x += mixer(h) + ff(h)``.  Three mixers, in whatever order the configuration lists them: softmax
attention over the latest keys with unit-size queries and keys, no positions and a learned sink per head
(``attention``); rotary attention over all earlier keys with biased projections, stretched frequencies, a sink of
score zero and a gate per head (``attention_2``); and latent attention with a query latent, a ramp-scaled rotation
and an element-wise output gate (``latent_attention``).  Feed-forwards: dense with a clamped swish gate, or experts
chosen by a table indexed by the token's id; a layer may have none.  A stretch of layers may run several times in
a row on the same tensors, each pass on a cache of its own; ahead of every pass a row of ``loop.step`` is added to
the stream, and ahead of every pass but the first the embedding's output as well.  Final RMS norm; the logits are
the embedding table's product times ``logit_scale``.

Tensor names: ``embed``, ``final.norm``, ``loop.step``; layer i: ``l<i>.norm1``, ``l<i>.mix.*`` (attention: ``q, k, v,
sink, o``; attention_2: ``q, q.b, k, k.b, v, v.b, g, o``; latent_attention: ``dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g,
o``), ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.table`` with ``l<i>.mlp.e<j>.{gate,up,down}``.  Linear weights are
stored [out, in].
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.soporax import SoporaxConfig
from ..parts.spec import Concat, LayerSpec, ModelSpec, PartSpec, RunEntry, StreamInput

SWISH_ALPHA = 1.702  # the dense feed-forward's gate: g * sigmoid(1.702 g)
ZERO_SINK = 0.0      # attention_2: the softmax's denominator holds one more exp(0)


def _mixer_spec(kind: str, mx, m: str, width: int, eps: float) -> PartSpec:
    if kind == "latent_attention":
        rot = mx.rot
        tensors = {"q_weight": m + ("uq" if mx.q_rank is not None else "q"), "dkv_weight": m + "dkv",
                   "dkv_norm": m + "dkv.norm", "uk_weight": m + "uk", "uv_weight": m + "uv", "o_weight": m + "o",
                   "gate_weight": m + "g"}
        if mx.q_rank is not None:
            tensors.update(dq_weight=m + "dq", dq_norm=m + "dq.norm")
        return PartSpec(
            "latent_attention",
            dict(hidden_size=width, num_heads=mx.heads, plain_dim=mx.dim, rot_dim=mx.rot_dim, value_dim=mx.vdim,
                 kv_rank=mx.kv_rank, scale=mx.scale, rot_dims=0 if rot is None else rot.dims,
                 rot_base=10000.0 if rot is None else rot.base, norm_eps=eps, sink=False, q_rank=mx.q_rank, gate=True,
                 rot_scaling=None if rot is None else rot.scaling_params()),
            tensors)
    common = dict(hidden_size=width, num_heads=mx.heads, num_kv_heads=mx.kv_heads, key_dim=mx.dim, value_dim=mx.vdim,
                  scale=mx.scale, norm_eps=eps, window=mx.window, unit_values=False, head_temperature=False)
    tensors = {"q_weight": m + "q", "k_weight": m + "k", "v_weight": m + "v", "out_weight": m + "o"}
    if kind == "attention":  # unit-size queries and keys without a weight, no positions, a learned sink
        tensors["sink"] = m + "sink"
        return PartSpec("window_attention", dict(common, qk_norm=True, qk_norm_weights=False, rot_dims=0, sink="learned"),
                        tensors)
    # attention_2: biases, rotation, a sink of score zero, a gate per head
    rot = mx.rot
    tensors.update(q_bias=m + "q.b", k_bias=m + "k.b", v_bias=m + "v.b", gate_weight=m + "g")
    return PartSpec(
        "window_attention",
        dict(common, qk_norm=False, bias=True, rot_dims=0 if rot is None else rot.dims,
             rot_base=10000.0 if rot is None else rot.base, rot_scaling=None if rot is None else rot.scaling_params(),
             sink=ZERO_SINK, gate="head"),
        tensors)


def _feed_forward_spec(mlp, p: str, width: int, vocab: int) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", dict(hidden_size=width, inner_size=mlp.ff, gate="clamped_swish", alpha=SWISH_ALPHA,
                                          limit=mlp.limit),
                        {"gate_up_weight": Concat((p + "gate", p + "up"), dim=0), "down_weight": p + "down"})
    experts = [f"{p}e{j}." for j in range(mlp.experts)]
    return PartSpec("moe", dict(hidden_size=width, inner_size=mlp.ff, num_experts=mlp.experts, top=mlp.top, gate="silu",
                                routing="table", vocab_size=vocab),
                    {"table": p + "table",
                     "gate_up_weight": Concat(tuple(e + w for e in experts for w in ("gate", "up")), dim=0),
                     "down_weight": Concat(tuple(e + "down" for e in experts), dim=0)})


def build_soporax_spec(cfg: SoporaxConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, lc in enumerate(cfg.layers):
        p = f"l{i}."
        named = dict(norm_input=("norm", PartSpec("rms_norm", dict(hidden_size=width, eps=eps), {"weight": p + "norm1"})),
                     mixer=("mixer", _mixer_spec(lc.type, lc.mixer, p + "mix.", width, eps)))
        if lc.mlp is not None:
            named["feed_forward"] = ("feed_forward", _feed_forward_spec(lc.mlp, p + "mlp.", width, cfg.vocab))
        layers.append(LayerSpec.of(PartSpec("parallel_sublayers", dict(feed_forward=lc.mlp is not None)), **named))
    # every run of a layer keeps pages under a number of its own: a repeated layer's passes do not share keys
    passes = cfg.passes()
    run_order = tuple(RunEntry(layer, instance=pos) for pos, (layer, _) in enumerate(passes))
    stream_parts, stream_inputs = (), ()
    if cfg.loop is not None:
        stream_parts = (PartSpec("pass_input", dict(hidden_size=width, passes=cfg.loop.times, readd_embedding=True),
                                 {"table": "loop.step"}),)
        stream_inputs = tuple(StreamInput(before=pos, part=0, args=(("index", t),))
                              for pos, (_, t) in enumerate(passes) if t is not None)
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, hidden_size=width), {"weight": "embed"}),
        position=PartSpec("none"),
        layers=tuple(layers),
        run_order=run_order,
        # the head is linear, so the logits' multiplier rides on the final norm's weight
        final_norm=PartSpec("rms_norm", dict(hidden_size=width, eps=eps, out_scale=cfg.logit_scale), {"weight": "final.norm"}),
        head=PartSpec("tied_to_embedding", dict(vocab_size=cfg.vocab, hidden_size=width)),
        eos_token_id=cfg.eos_token_id,
        stream_parts=stream_parts,
        stream_inputs=stream_inputs,
    )


register_architecture("Soporax", SoporaxConfig, build_soporax_spec, model_types=("soporax",), replace=True)
