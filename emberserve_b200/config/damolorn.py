"""Typed configuration of the Damolorn decoder, read from its own ``config.json`` keys.

The file is nested: ``layers`` lists the layers in order, each with its mixer ``type``, the
mixer's sizes and its feed-forward (or none); ``loop`` names a range of layers that runs several
times in a row; ``norm`` and ``canon`` hold what all layers share.  Every size and constant is
taken from the file; nothing about a particular model is assumed.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, ClassVar

from emberserve_b200.config.model import ConfigError, ModelConfig

MIXER_TYPES = ("latent_attention", "latent_attention_2")
# Positions the rotary tables are built for when the file does not say (an engine limit, not a
# property of the model: the design has no trained position range).
DEFAULT_MAX_POSITIONS = 1 << 17


def _need(d: dict[str, Any], key: str, where: str, kind: type = int) -> Any:
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    v = d[key]
    if kind is int and (isinstance(v, bool) or not isinstance(v, int)):
        raise ConfigError(f"config.json: {where}.{key} must be an integer, got {v!r}")
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
        return float(v)
    return v


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int  # unrotated query/key numbers per head
    rot_dim: int  # rotated query numbers per head, and the size of the shared key part
    vdim: int
    kv_rank: int
    q_rank: int
    rot_base: float
    rot_dims: int  # how many leading numbers of the rotated part turn
    scale: float

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "LatentMixerConfig":
        rot = _need(d, "rot", where, dict)
        m = cls(heads=_need(d, "heads", where), dim=_need(d, "dim", where), rot_dim=_need(d, "rot_dim", where),
                vdim=_need(d, "vdim", where), kv_rank=_need(d, "kv_rank", where), q_rank=_need(d, "q_rank", where),
                rot_base=_need(rot, "base", where + ".rot", float), rot_dims=_need(rot, "dims", where + ".rot"),
                scale=_need(d, "scale", where, float))
        for name in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
            if getattr(m, name) <= 0:
                raise ConfigError(f"config.json: {where}.{name} must be positive")
        if m.rot_dim < 0 or m.rot_dims < 0 or m.rot_dims % 2 or m.rot_dims > m.rot_dim:
            raise ConfigError(f"config.json: {where}: rot.dims={m.rot_dims} must be even and at most "
                              f"rot_dim={m.rot_dim}")
        if m.rot_dims and m.rot_base <= 0:
            raise ConfigError(f"config.json: {where}.rot.base must be positive")
        return m

    def to_dict(self) -> dict[str, Any]:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank,
                "rot": {"base": self.rot_base, "dims": self.rot_dims}, "rot_dim": self.rot_dim,
                "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" or "moe"
    ff: int  # of the dense layer, or of one expert
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "FeedForwardConfig":
        kind = _need(d, "kind", where, str)
        if kind == "dense":
            f = cls("dense", _need(d, "ff", where))
        elif kind == "moe":
            router = _need(d, "router", where, dict)
            f = cls("moe", _need(_need(d, "expert", where, dict), "ff", where + ".expert"),
                    _need(router, "experts", where + ".router"), _need(router, "top", where + ".router"))
            if not 1 <= f.top <= f.experts:
                raise ConfigError(f"config.json: {where}.router: top={f.top} of {f.experts} experts")
        else:
            raise ConfigError(f"config.json: {where}.kind {kind!r} is neither 'dense' nor 'moe'")
        if f.ff <= 0:
            raise ConfigError(f"config.json: {where}: ff must be positive")
        return f

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class DamolornLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: FeedForwardConfig | None


@dataclass(frozen=True)
class DamolornConfig(ModelConfig):
    architecture: ClassVar[str] = "Damolorn"

    vocab_size: int
    width: int
    layers: tuple[DamolornLayerConfig, ...]
    norm_eps: float
    norm_groups: int
    canon_taps: int  # 0: no input convolution
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if self.norm_groups <= 0 or self.width % self.norm_groups:
            raise ConfigError(f"norm.groups={self.norm_groups} does not divide width={self.width}")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.canon_taps < 0:
            raise ConfigError("canon.taps must not be negative")
        if self.has_loop and not (0 <= self.loop_start < self.loop_stop <= len(self.layers) and self.loop_times >= 1):
            raise ConfigError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit "
                              f"{len(self.layers)} layers")
        if self.max_positions <= 0:
            raise ConfigError("max_positions must be positive")

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start or self.loop_times != 1

    def layer_runs(self) -> list[tuple[int, int | None]]:
        """(layer, number of the pass that begins with this run or None), in the order the layers run."""
        n = len(self.layers)
        if not self.has_loop:
            return [(i, None) for i in range(n)]
        out: list[tuple[int, int | None]] = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            out += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, None) for i in range(self.loop_stop, n)]

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "DamolornConfig":
        layers = []
        raw = _need(cfg, "layers", "the file", list)
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where, str)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r}: one of {MIXER_TYPES}")
            mlp = entry.get("mlp")
            layers.append(DamolornLayerConfig(
                kind, LatentMixerConfig.from_dict(_need(entry, "mixer", where, dict), where + ".mixer"),
                None if mlp is None else FeedForwardConfig.from_dict(mlp, where + ".mlp")))
        norm = _need(cfg, "norm", "the file", dict)
        canon = cfg.get("canon") or {}
        loop = cfg.get("loop")
        eos = cfg.get("eos_token_id", ())
        eos = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(e) for e in eos)
        return cls(
            vocab_size=_need(cfg, "vocab", "the file"), width=_need(cfg, "width", "the file"),
            layers=tuple(layers), norm_eps=_need(norm, "eps", "norm", float),
            norm_groups=int(norm.get("groups", 1)), canon_taps=int(canon.get("taps", 0)),
            loop_start=0 if not loop else _need(loop, "start", "loop"),
            loop_stop=0 if not loop else _need(loop, "stop", "loop"),
            loop_times=1 if not loop else _need(loop, "times", "loop"),
            max_positions=int(cfg.get("max_positions", DEFAULT_MAX_POSITIONS)), eos_token_ids=eos)

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict(),
                        "type": L.type} for L in self.layers],
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "vocab": self.vocab_size, "width": self.width,
        }
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def replace(self, **changes: Any) -> "DamolornConfig":
        return dataclasses.replace(self, **changes)
