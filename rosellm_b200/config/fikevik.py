"""Fikevik's typed configuration, read from the keys of its own ``config.json``.

Top level: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (the token rows' multiplier), ``postln_alpha``
(the stream's weight in every sum that a norm follows) and ``layers``, a list whose entries give ``type`` (the
mixer: ``gla`` or ``parallel``), the mixer's sizes and constants under ``mixer``, the feed-forward under ``mlp``
(null for none, or ``{"kind": "dense", "ff": n}``) and, optionally, ``weights_of``: the index of the layer
whose tensors this layer uses instead of tensors of its own (with a cache and state of its own).

Mixer keys: ``gla``: ``heads``, ``dim``, ``vdim``, ``tau`` (and, optionally, ``decay_rank``: the low rank of the
decay's projection, which a weight file shows by its tensors' shapes).  ``parallel``: ``left`` (windowed softmax
attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``rot.dims``, ``rot.base``),
``right`` (a matrix memory: ``heads``, ``dim``, ``vdim``, ``gate_cap``), ``left_scale`` and ``right_scale`` (the
weights of the two results).  Every size and constant comes from there; layers may differ from one another in all
of them.  The design has no position limit of its own (positions enter through rotations only): ``max_positions``,
where a folder gives it, bounds the sequences the engine plans for, else ``DEFAULT_MAX_POSITIONS``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig, optional, require

DEFAULT_MAX_POSITIONS = 131072
MIXER_TYPES = ("gla", "parallel")


def _positive(where: str, **values) -> None:
    for name, v in values.items():
        if v <= 0:
            raise ConfigError(f"config.json: {where}.{name} must be positive")


@dataclass(frozen=True)
class DecayedAttentionConfig:
    """``gla``: linear attention with a decay per key channel."""

    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int | None = None

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "DecayedAttentionConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where} must be an object")
        out = cls(heads=require(raw, "heads", int), dim=require(raw, "dim", int), vdim=require(raw, "vdim", int),
                  tau=require(raw, "tau", float), decay_rank=optional(raw, "decay_rank", int, None))
        _positive(where, heads=out.heads, dim=out.dim, vdim=out.vdim, tau=out.tau)
        if out.decay_rank is not None and out.decay_rank <= 0:
            raise ConfigError(f"config.json: {where}.decay_rank must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        return out


@dataclass(frozen=True)
class WindowAttentionConfig:
    """``parallel.left``: softmax attention over the latest ``window`` keys (``None``: over all)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "WindowAttentionConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where} must be an object")
        heads, dim = require(raw, "heads", int), require(raw, "dim", int)
        rot, mask = raw.get("rot"), raw.get("mask")
        if rot is not None and not isinstance(rot, dict):
            raise ConfigError(f"config.json: {where}.rot must be an object with dims and base")
        if mask is not None and not isinstance(mask, dict):
            raise ConfigError(f"config.json: {where}.mask must be an object with size")
        out = cls(heads=heads, kv_heads=optional(raw, "kv_heads", int, heads), dim=dim, vdim=require(raw, "vdim", int),
                  scale=optional(raw, "scale", float, float(max(dim, 1)) ** -0.5),
                  window=None if mask is None else require(mask, "size", int),
                  rot_dims=0 if rot is None else optional(rot, "dims", int, dim),
                  rot_base=10000.0 if rot is None else require(rot, "base", float))
        _positive(where, heads=out.heads, kv_heads=out.kv_heads, dim=out.dim, vdim=out.vdim)
        if out.heads % out.kv_heads:
            raise ConfigError(f"config.json: {where}: {out.heads} heads are not a multiple of {out.kv_heads} kv_heads")
        if out.window is not None and out.window <= 0:
            raise ConfigError(f"config.json: {where}.mask.size must be positive")
        if out.rot_dims < 0 or out.rot_dims % 2 or out.rot_dims > out.dim:
            raise ConfigError(f"config.json: {where}.rot.dims={out.rot_dims} must be even and at most dim={out.dim}")
        if out.rot_base <= 0:
            raise ConfigError(f"config.json: {where}.rot.base must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return out


@dataclass(frozen=True)
class MatrixMemoryConfig:
    """``parallel.right``: a matrix memory with exponential gates whose logits are bounded by ``gate_cap``."""

    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "MatrixMemoryConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where} must be an object")
        out = cls(heads=require(raw, "heads", int), dim=require(raw, "dim", int), vdim=require(raw, "vdim", int),
                  gate_cap=require(raw, "gate_cap", float))
        _positive(where, heads=out.heads, dim=out.dim, vdim=out.vdim, gate_cap=out.gate_cap)
        return out

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class SideBySideConfig:
    """``parallel``: both mixers read the layer's input; their results are summed with a weight each."""

    left: WindowAttentionConfig
    right: MatrixMemoryConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "SideBySideConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where} must be an object")
        return cls(left=WindowAttentionConfig.from_dict(raw.get("left"), where + ".left"),
                   right=MatrixMemoryConfig.from_dict(raw.get("right"), where + ".right"),
                   left_scale=optional(raw, "left_scale", float, 1.0), right_scale=optional(raw, "right_scale", float, 1.0))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


MIXER_CONFIGS = {"gla": DecayedAttentionConfig, "parallel": SideBySideConfig}


@dataclass(frozen=True)
class FikevikLayerConfig:
    type: str
    mixer: "DecayedAttentionConfig | SideBySideConfig"
    ff: int | None             # the dense feed-forward's inner size; None: the layer has none
    weights_of: int | None = None

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"type": self.type, "mixer": self.mixer.to_dict(),
                               "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


@dataclass(frozen=True)
class FikevikConfig(ModelConfig):
    architecture: ClassVar[str] = "Fikevik"

    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    postln_alpha: float
    layers: tuple[FikevikLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int | None = None

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0 or not self.layers:
            raise ConfigError("config.json: vocab, width and max_positions must be positive and layers non-empty")
        if self.width % 8:
            raise ConfigError(f"config.json: width={self.width}: the products read rows in 16-byte pieces, so the "
                              "width must be a multiple of 8")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        for i, l in enumerate(self.layers):
            if l.weights_of is None:
                continue
            j = l.weights_of
            if not 0 <= j < len(self.layers) or j == i:
                raise ConfigError(f"config.json: layers[{i}].weights_of={j} names no other layer")
            if self.layers[self.weight_owner(i)].type != l.type:
                raise ConfigError(f"config.json: layers[{i}] uses the tensors of layer {j}, a layer of another type")

    def weight_owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` reads (itself unless it names another with ``weights_of``)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of leads back to itself")
            seen.add(i)
            i = self.layers[i].weights_of
            if not 0 <= i < len(self.layers):
                raise ConfigError(f"config.json: weights_of={i} names no layer")
        return i

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "FikevikConfig":
        norm, emb = raw.get("norm"), raw.get("embedding")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: norm must be an object with eps")
        if emb is not None and not isinstance(emb, dict):
            raise ConfigError("config.json: embedding must be an object with scale")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list):
            raise ConfigError("config.json: layers must be a list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = require(lr, "type", str)
            if kind not in MIXER_CONFIGS:
                raise ConfigError(f"config.json: {where}.type={kind!r}; the design's mixers: {MIXER_TYPES}")
            mlp, ff = lr.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                if optional(mlp, "kind", str, "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind={mlp.get('kind')!r}; the design's feed-forward is dense")
                ff = require(mlp, "ff", int)
                if ff <= 0:
                    raise ConfigError(f"config.json: {where}.mlp.ff must be positive")
            layers.append(FikevikLayerConfig(kind, MIXER_CONFIGS[kind].from_dict(lr.get("mixer"), where + ".mixer"), ff,
                                             optional(lr, "weights_of", int, None)))
        return cls(
            vocab=require(raw, "vocab", int), width=require(raw, "width", int), norm_eps=require(norm, "eps", float),
            embedding_scale=1.0 if emb is None else optional(emb, "scale", float, 1.0),
            postln_alpha=optional(raw, "postln_alpha", float, 1.0), layers=tuple(layers),
            max_positions=optional(raw, "max_positions", int, DEFAULT_MAX_POSITIONS),
            eos_token_id=optional(raw, "eos_token_id", int, None),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "postln_alpha": self.postln_alpha, "layers": [l.to_dict() for l in self.layers],
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out
