"""Typed configuration of the Dedizen decoder, read from its own ``config.json`` keys.

``layers`` lists the layers in order; each names its mixer ``type`` (``parallel``: chunked
attention with a sink beside linear attention with a fixed decay per head; ``mlstm``: a matrix
memory with exponential gates; ``rglru``: a gated diagonal recurrence behind a short convolution),
the mixer's sizes under ``mixer`` and its feed-forward under ``mlp`` (or null).  ``norm`` holds
what all layers share.  Every size and constant is taken from the file.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, ClassVar

from emberserve_b200.config.damolorn import DEFAULT_MAX_POSITIONS, _need
from emberserve_b200.config.model import ConfigError, ModelConfig

MIXER_TYPES = ("parallel", "mlstm", "rglru")


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: int
    fast: float
    slow: float

    def to_dict(self) -> dict[str, Any]:
        return {"factor": self.factor, "fast": self.fast, "original": self.original, "slow": self.slow}


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int | None  # mask.size
    rot_dims: int
    rot_base: float
    rot_scaling: YarnScaling | None

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "SinkAttentionConfig":
        rot = d.get("rot") or {}
        scaling = rot.get("scaling") if rot else None
        mask = d.get("mask") or {}
        m = cls(heads=_need(d, "heads", where), kv_heads=int(d.get("kv_heads") or _need(d, "heads", where)),
                dim=_need(d, "dim", where), vdim=int(d.get("vdim") or _need(d, "dim", where)),
                scale=_need(d, "scale", where, float),
                chunk=_need(mask, "size", where + ".mask") if mask else None,
                rot_dims=_need(rot, "dims", where + ".rot") if rot else 0,
                rot_base=_need(rot, "base", where + ".rot", float) if rot else 10000.0,
                rot_scaling=None if not scaling else YarnScaling(
                    _need(scaling, "factor", where + ".rot.scaling", float),
                    _need(scaling, "original", where + ".rot.scaling"),
                    _need(scaling, "fast", where + ".rot.scaling", float),
                    _need(scaling, "slow", where + ".rot.scaling", float)))
        if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads or m.dim <= 0:
            raise ConfigError(f"config.json: {where}: heads={m.heads}, kv_heads={m.kv_heads}, dim={m.dim}")
        if m.vdim != m.dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so vdim={m.vdim} must equal dim={m.dim}")
        if m.rot_dims < 0 or m.rot_dims % 2 or m.rot_dims > m.dim or (m.rot_dims and m.rot_base <= 0):
            raise ConfigError(f"config.json: {where}.rot: dims={m.rot_dims} must be even and at most dim={m.dim}")
        if m.chunk is not None and m.chunk <= 0:
            raise ConfigError(f"config.json: {where}.mask.size must be positive")
        if m.rot_scaling is not None and (m.rot_scaling.factor <= 0 or m.rot_scaling.original <= 0
                                          or m.rot_scaling.fast <= 0 or m.rot_scaling.slow <= 0):
            raise ConfigError(f"config.json: {where}.rot.scaling: all four numbers must be positive")
        return m

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                             "vdim": self.vdim}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                d["rot"]["scaling"] = self.rot_scaling.to_dict()
        return d


@dataclass(frozen=True)
class DecayAttentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "DecayAttentionConfig":
        decay = _need(d, "decay", where, list)
        m = cls(_need(d, "heads", where), _need(d, "dim", where), _need(d, "vdim", where),
                tuple(float(x) for x in decay))
        if m.heads <= 0 or m.dim <= 0 or m.vdim <= 0 or len(m.decay) != m.heads:
            raise ConfigError(f"config.json: {where}: {m.heads} heads need as many decays, got {len(m.decay)}")
        return m

    def to_dict(self) -> dict[str, Any]:
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SinkAttentionConfig
    right: DecayAttentionConfig

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "ParallelMixerConfig":
        return cls(SinkAttentionConfig.from_dict(_need(d, "left", where, dict), where + ".left"),
                   DecayAttentionConfig.from_dict(_need(d, "right", where, dict), where + ".right"))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class MLSTMConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "MLSTMConfig":
        m = cls(_need(d, "heads", where), _need(d, "dim", where), _need(d, "vdim", where),
                _need(d, "gate_cap", where, float))
        if m.heads <= 0 or m.dim <= 0 or m.vdim <= 0 or not m.gate_cap > 0:
            raise ConfigError(f"config.json: {where}: heads, dim, vdim and gate_cap must be positive")
        return m

    def to_dict(self) -> dict[str, Any]:
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class RGLRUConfig:
    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "RGLRUConfig":
        m = cls(_need(d, "width", where), _need(d, "blocks", where), _need(d, "conv", where))
        if m.width <= 0 or m.blocks <= 0 or m.width % m.blocks or m.conv < 1:
            raise ConfigError(f"config.json: {where}: width={m.width} in {m.blocks} blocks, {m.conv} taps")
        return m

    def to_dict(self) -> dict[str, Any]:
        return {"blocks": self.blocks, "conv": self.conv, "width": self.width}


_MIXER_CONFIGS = {"parallel": ParallelMixerConfig, "mlstm": MLSTMConfig, "rglru": RGLRUConfig}


@dataclass(frozen=True)
class DenseMLPConfig:
    ff: int

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "DenseMLPConfig":
        kind = _need(d, "kind", where, str)
        if kind != "dense":
            raise ConfigError(f"config.json: {where}.kind {kind!r}: this design has dense feed-forwards only")
        m = cls(_need(d, "ff", where))
        if m.ff <= 0:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return m

    def to_dict(self) -> dict[str, Any]:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class DedizenLayerConfig:
    type: str
    mixer: "ParallelMixerConfig | MLSTMConfig | RGLRUConfig"
    mlp: DenseMLPConfig | None


@dataclass(frozen=True)
class DedizenConfig(ModelConfig):
    architecture: ClassVar[str] = "Dedizen"

    vocab_size: int
    width: int
    layers: tuple[DedizenLayerConfig, ...]
    norm_eps: float
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.max_positions <= 0:
            raise ConfigError("max_positions must be positive")

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "DedizenConfig":
        layers = []
        for i, entry in enumerate(_need(cfg, "layers", "the file", list)):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where, str)
            if kind not in _MIXER_CONFIGS:
                raise ConfigError(f"config.json: {where}.type {kind!r}: one of {MIXER_TYPES}")
            mlp = entry.get("mlp")
            layers.append(DedizenLayerConfig(
                kind, _MIXER_CONFIGS[kind].from_dict(_need(entry, "mixer", where, dict), where + ".mixer"),
                None if mlp is None else DenseMLPConfig.from_dict(mlp, where + ".mlp")))
        norm = _need(cfg, "norm", "the file", dict)
        eos = cfg.get("eos_token_id", ())
        eos = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(e) for e in eos)
        return cls(vocab_size=_need(cfg, "vocab", "the file"), width=_need(cfg, "width", "the file"),
                   layers=tuple(layers), norm_eps=_need(norm, "eps", "norm", float),
                   max_positions=int(cfg.get("max_positions", DEFAULT_MAX_POSITIONS)), eos_token_ids=eos)

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict(),
                        "type": L.type} for L in self.layers],
            "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width,
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def replace(self, **changes: Any) -> "DedizenConfig":
        return dataclasses.replace(self, **changes)
