"""Soporax's typed configuration, read from the keys of its own ``config.json``.

Top level: ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` (the logits' multiplier), ``layers`` and, optionally,
``loop`` (``start``, ``stop``, ``times``: layers ``start .. stop - 1`` run ``times`` times in a row on the same
tensors, each pass with a cache of its own).  A layer gives ``type`` (its mixer: ``attention``, ``attention_2`` or
``latent_attention``), the mixer's sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (null for
none; ``{"kind": "dense", "ff", "limit"}``; or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}``).

Mixer keys.  ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (absent: all earlier
keys).  ``attention_2``: the same sizes and ``scale``, and ``rot`` (``dims``, ``base``, optionally ``scaling``).
``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``rot`` (``base``,
optionally ``scaling``; its ``dims`` is ``rot_dim``).  ``rot.scaling`` holds ``factor`` and ``original`` and either
``low`` and ``high`` (frequencies scaled by their wavelength) or ``fast`` and ``slow`` (a ramp over the pairs'
indices).  Every size and constant comes from there; layers may differ from one another in all of them.  The design
has no position limit of its own: ``max_positions``, where a folder gives it, bounds the sequences the engine
plans for, else ``DEFAULT_MAX_POSITIONS``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig, optional, require

DEFAULT_MAX_POSITIONS = 131072
MIXER_TYPES = ("attention", "attention_2", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _object(raw: Any, where: str) -> dict:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    return raw


def _positive(where: str, **values) -> None:
    for name, v in values.items():
        if v <= 0:
            raise ConfigError(f"config.json: {where}.{name} must be positive")


@dataclass(frozen=True)
class RotationConfig:
    """``rot``: ``dims`` turned entries a head, ``base``, and the frequencies' scaling: ``scaling_kind``
    ``"wavelength"`` (``factor``, ``low``, ``high``, ``original``), ``"ramp"`` (``factor``, ``original``, ``fast``,
    ``slow``) or ``None``."""

    dims: int
    base: float
    scaling_kind: str | None = None
    scaling: tuple[tuple[str, float], ...] = ()

    @classmethod
    def from_dict(cls, raw: Any, where: str, dims: int | None = None) -> "RotationConfig":
        raw = _object(raw, where)
        d = optional(raw, "dims", int, dims)
        if d is None:
            raise ConfigError(f"config.json: missing required key {where}.dims")
        if dims is not None and d > dims:
            raise ConfigError(f"config.json: {where}.dims={d} exceeds the mixer's rot_dim={dims}")
        base = require(raw, "base", float)
        if d < 0 or d % 2 or base <= 0:
            raise ConfigError(f"config.json: {where}: dims must be even and not negative, base positive")
        sc = raw.get("scaling")
        kind, values = None, ()
        if sc is not None:
            sc = _object(sc, where + ".scaling")
            if "fast" in sc or "slow" in sc:
                kind, keys = "ramp", ("factor", "original", "fast", "slow")
            else:
                kind, keys = "wavelength", ("factor", "original", "low", "high")
            values = tuple((k, require(sc, k, float)) for k in keys)
            if any(v <= 0 for k, v in values if k in ("factor", "original", "fast", "slow")):
                raise ConfigError(f"config.json: {where}.scaling: factor, original, fast and slow must be positive")
            if kind == "wavelength" and dict(values)["low"] == dict(values)["high"]:
                raise ConfigError(f"config.json: {where}.scaling: low and high must differ")
            if kind == "ramp" and base == 1.0:
                raise ConfigError(f"config.json: {where}: a ramp needs a base other than 1")
        return cls(d, base, kind, values)

    def scaling_params(self) -> dict | None:
        """What ``RotaryPositions(scaling=...)`` takes."""
        return None if self.scaling_kind is None else dict(self.scaling, kind=self.scaling_kind)

    def to_dict(self, with_dims: bool = True) -> dict[str, Any]:
        out: dict[str, Any] = {"base": self.base}
        if with_dims:
            out["dims"] = self.dims
        if self.scaling_kind is not None:
            sc = dict(self.scaling)
            sc["original"] = int(sc["original"]) if float(sc["original"]).is_integer() else sc["original"]
            out["scaling"] = sc
        return out


@dataclass(frozen=True)
class GroupedAttentionConfig:
    """``attention`` and ``attention_2``: ``heads`` query heads on ``kv_heads`` key/value heads.  ``window``: the
    latest keys a query sees (``None``: all); ``rot``: ``None`` where positions do not enter."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None = None
    rot: RotationConfig | None = None

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "GroupedAttentionConfig":
        raw = _object(raw, where)
        heads, dim = require(raw, "heads", int), require(raw, "dim", int)
        mask, rot = raw.get("mask"), raw.get("rot")
        out = cls(heads=heads, kv_heads=optional(raw, "kv_heads", int, heads), dim=dim,
                  vdim=optional(raw, "vdim", int, dim), scale=optional(raw, "scale", float, float(max(dim, 1)) ** -0.5),
                  window=None if mask is None else require(_object(mask, where + ".mask"), "size", int),
                  rot=None if rot is None else RotationConfig.from_dict(rot, where + ".rot"))
        _positive(where, heads=out.heads, kv_heads=out.kv_heads, dim=out.dim, vdim=out.vdim)
        if out.heads % out.kv_heads:
            raise ConfigError(f"config.json: {where}: {out.heads} heads are not a multiple of {out.kv_heads} kv_heads")
        if out.window is not None and out.window <= 0:
            raise ConfigError(f"config.json: {where}.mask.size must be positive")
        if out.rot is not None and out.rot.dims > out.dim:
            raise ConfigError(f"config.json: {where}.rot.dims={out.rot.dims} exceeds dim={out.dim}")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class LatentAttentionConfig:
    """``latent_attention``: per head ``dim`` plain and ``rot_dim`` turned query/key entries, values of ``vdim``; a
    key/value latent of ``kv_rank`` and a query latent of ``q_rank`` (``None``: queries straight from the input)."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int | None
    scale: float
    rot: RotationConfig | None = None

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "LatentAttentionConfig":
        raw = _object(raw, where)
        dim, rot_dim = require(raw, "dim", int), optional(raw, "rot_dim", int, 0)
        rot = raw.get("rot")
        out = cls(heads=require(raw, "heads", int), dim=dim, rot_dim=rot_dim, vdim=optional(raw, "vdim", int, dim),
                  kv_rank=require(raw, "kv_rank", int), q_rank=optional(raw, "q_rank", int, None),
                  scale=optional(raw, "scale", float, float(max(dim + rot_dim, 1)) ** -0.5),
                  rot=None if rot is None or rot_dim == 0 else RotationConfig.from_dict(rot, where + ".rot", dims=rot_dim))
        _positive(where, heads=out.heads, dim=out.dim, vdim=out.vdim, kv_rank=out.kv_rank)
        if out.rot_dim < 0 or out.rot_dim % 2:
            raise ConfigError(f"config.json: {where}.rot_dim must be even and not negative")
        if out.q_rank is not None and out.q_rank <= 0:
            raise ConfigError(f"config.json: {where}.q_rank must be positive")
        return out

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "kv_rank": self.kv_rank, "scale": self.scale}
        if self.q_rank is not None:
            out["q_rank"] = self.q_rank
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


MIXER_CONFIGS = {"attention": GroupedAttentionConfig, "attention_2": GroupedAttentionConfig,
                 "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class FeedForwardConfig:
    """``dense``: inner size ``ff`` and the gate's ``limit``; ``moe``: ``experts`` of inner size ``ff``, of which a
    token uses ``top``, named by a table indexed by its id."""

    kind: str
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, raw: Any, where: str) -> "FeedForwardConfig":
        raw = _object(raw, where)
        kind = require(raw, "kind", str)
        if kind == "dense":
            out = cls("dense", require(raw, "ff", int), limit=require(raw, "limit", float))
            _positive(where, ff=out.ff, limit=out.limit)
        elif kind == "moe":
            router = _object(raw.get("router"), where + ".router")
            out = cls("moe", require(_object(raw.get("expert"), where + ".expert"), "ff", int),
                      experts=require(router, "experts", int), top=require(router, "top", int))
            _positive(where, ff=out.ff, experts=out.experts, top=out.top)
            if out.top > out.experts:
                raise ConfigError(f"config.json: {where}.router: top={out.top} of {out.experts} experts")
        else:
            raise ConfigError(f"config.json: {where}.kind={kind!r}; the design's feed-forwards: {MLP_KINDS}")
        return out

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff, "limit": self.limit}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class SoporaxLayerConfig:
    type: str
    mixer: "GroupedAttentionConfig | LatentAttentionConfig"
    mlp: FeedForwardConfig | None

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int

    def to_dict(self) -> dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class SoporaxConfig(ModelConfig):
    architecture: ClassVar[str] = "Soporax"

    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: tuple[SoporaxLayerConfig, ...]
    loop: LoopConfig | None = None
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
        lp = self.loop
        if lp is not None and not (0 <= lp.start < lp.stop <= len(self.layers) and lp.times >= 1):
            raise ConfigError(f"config.json: loop={lp.to_dict()}: 0 <= start < stop <= {len(self.layers)} layers, times >= 1")

    def passes(self) -> list[tuple[int, int | None]]:
        """(layer, pass) for every run of a layer in order: ``pass`` is the pass's number at the first layer of a
        pass of the repeated stretch and ``None`` everywhere else."""
        n, lp = len(self.layers), self.loop
        if lp is None:
            return [(i, None) for i in range(n)]
        out: list[tuple[int, int | None]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return out + [(i, None) for i in range(lp.stop, n)]

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "SoporaxConfig":
        norm = _object(raw.get("norm"), "norm")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list):
            raise ConfigError("config.json: layers must be a list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            lr = _object(lr, where)
            kind = require(lr, "type", str)
            if kind not in MIXER_CONFIGS:
                raise ConfigError(f"config.json: {where}.type={kind!r}; the design's mixers: {MIXER_TYPES}")
            mlp = lr.get("mlp")
            layers.append(SoporaxLayerConfig(kind, MIXER_CONFIGS[kind].from_dict(lr.get("mixer"), where + ".mixer"),
                                             None if mlp is None else FeedForwardConfig.from_dict(mlp, where + ".mlp")))
        loop = raw.get("loop")
        if loop is not None:
            loop = _object(loop, "loop")
            loop = LoopConfig(require(loop, "start", int), require(loop, "stop", int), require(loop, "times", int))
        return cls(
            vocab=require(raw, "vocab", int), width=require(raw, "width", int), norm_eps=require(norm, "eps", float),
            logit_scale=optional(raw, "logit_scale", float, 1.0), layers=tuple(layers), loop=loop,
            max_positions=optional(raw, "max_positions", int, DEFAULT_MAX_POSITIONS),
            eos_token_id=optional(raw, "eos_token_id", int, None),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
            "layers": [l.to_dict() for l in self.layers],
        }
        if self.loop is not None:
            out["loop"] = self.loop.to_dict()
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out
