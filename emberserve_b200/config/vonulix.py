"""Typed configuration of the Vonulix decoder, read from its own ``config.json`` keys.

``layers`` lists the layers in order; each names its mixer ``type`` (``attention``: grouped-query
attention behind a window that also keeps the first keys, with unit-RMS values that are turned by
their positions, and a sigmoid gate per head), the mixer's sizes under ``mixer`` and its feed-forward
under ``mlp`` (a mixture of experts with sigmoid scores and an optional shared expert, or null).
``embedding.scale`` multiplies the embedding row, ``token_side.dim`` is the number of columns of the
second embedding table that each layer reads, ``norm.eps`` serves every norm.  Every size and constant
is taken from the file.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, ClassVar

from emberserve_b200.config.damolorn import DEFAULT_MAX_POSITIONS, _need
from emberserve_b200.config.model import ConfigError, ModelConfig

MIXER_TYPES = ("attention",)
# the slope inside the sigmoid of an expert's activation: g * sigmoid(1.702 g)
EXPERT_ACT_ALPHA = 1.702


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None  # mask.size (None: every earlier key is seen)
    keep_first: int  # mask.keep_first
    rot_dims: int
    rot_base: float
    rot_factor: float  # rot.scaling.factor (1: no scaling)

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "WindowAttentionConfig":
        rot = _need(d, "rot", where, dict)
        scaling = rot.get("scaling") or {}
        mask = d.get("mask") or {}
        m = cls(heads=_need(d, "heads", where), kv_heads=int(d.get("kv_heads") or _need(d, "heads", where)),
                dim=_need(d, "dim", where), vdim=int(d.get("vdim") or _need(d, "dim", where)),
                scale=_need(d, "scale", where, float),
                window=_need(mask, "size", where + ".mask") if mask.get("size") is not None else None,
                keep_first=int(mask.get("keep_first") or 0),
                rot_dims=_need(rot, "dims", where + ".rot"), rot_base=_need(rot, "base", where + ".rot", float),
                rot_factor=_need(scaling, "factor", where + ".rot.scaling", float) if scaling else 1.0)
        if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads or m.dim <= 0 or m.vdim <= 0:
            raise ConfigError(f"config.json: {where}: heads={m.heads}, kv_heads={m.kv_heads}, dim={m.dim}, "
                              f"vdim={m.vdim}")
        if m.vdim % 2:
            raise ConfigError(f"config.json: {where}.vdim={m.vdim}: the values are turned in pairs")
        if m.rot_dims < 0 or m.rot_dims % 2 or m.rot_dims > m.dim or not m.rot_base > 0:
            raise ConfigError(f"config.json: {where}.rot: dims={m.rot_dims} must be even and at most dim={m.dim}, "
                              f"base positive")
        if not m.rot_factor > 0:
            raise ConfigError(f"config.json: {where}.rot.scaling.factor must be positive")
        if (m.window is not None and m.window <= 0) or m.keep_first < 0:
            raise ConfigError(f"config.json: {where}.mask: size must be positive, keep_first not negative")
        return m

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                             "vdim": self.vdim, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.rot_factor != 1.0:
            d["rot"]["scaling"] = {"factor": self.rot_factor}
        if self.window is not None or self.keep_first:
            d["mask"] = {"keep_first": self.keep_first, "size": self.window}
        return d


@dataclass(frozen=True)
class CappedExpertConfig:
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "CappedExpertConfig":
        m = cls(_need(d, "ff", where), _need(d, "limit", where, float))
        if m.ff <= 0 or not m.limit > 0:
            raise ConfigError(f"config.json: {where}: ff and limit must be positive")
        return m

    def to_dict(self) -> dict[str, Any]:
        return {"ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class SigmoidMoEConfig:
    experts: int
    top: int
    expert: CappedExpertConfig
    shared: CappedExpertConfig | None

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "SigmoidMoEConfig":
        kind = _need(d, "kind", where, str)
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind {kind!r}: this design has mixtures of experts only")
        router = _need(d, "router", where, dict)
        shared = d.get("shared")
        m = cls(_need(router, "experts", where + ".router"), _need(router, "top", where + ".router"),
                CappedExpertConfig.from_dict(_need(d, "expert", where, dict), where + ".expert"),
                None if not shared else CappedExpertConfig.from_dict(shared, where + ".shared"))
        if m.experts <= 0 or not 0 < m.top <= m.experts:
            raise ConfigError(f"config.json: {where}.router: top={m.top} of {m.experts} experts")
        return m

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"expert": self.expert.to_dict(), "kind": "moe",
                             "router": {"experts": self.experts, "top": self.top}}
        if self.shared is not None:
            d["shared"] = self.shared.to_dict()
        return d


@dataclass(frozen=True)
class VonulixLayerConfig:
    type: str
    mixer: WindowAttentionConfig
    mlp: SigmoidMoEConfig | None


@dataclass(frozen=True)
class VonulixConfig(ModelConfig):
    architecture: ClassVar[str] = "Vonulix"

    vocab_size: int
    width: int
    layers: tuple[VonulixLayerConfig, ...]
    norm_eps: float
    embed_scale: float = 1.0
    side_dim: int = 0  # token_side.dim (0: the layers have no input of their own)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.side_dim < 0:
            raise ConfigError("token_side.dim must not be negative")
        if self.max_positions <= 0:
            raise ConfigError("max_positions must be positive")

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "VonulixConfig":
        layers = []
        for i, entry in enumerate(_need(cfg, "layers", "the file", list)):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where, str)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r}: one of {MIXER_TYPES}")
            mlp = entry.get("mlp")
            layers.append(VonulixLayerConfig(
                kind, WindowAttentionConfig.from_dict(_need(entry, "mixer", where, dict), where + ".mixer"),
                None if mlp is None else SigmoidMoEConfig.from_dict(mlp, where + ".mlp")))
        norm = _need(cfg, "norm", "the file", dict)
        emb = cfg.get("embedding") or {}
        side = cfg.get("token_side") or {}
        eos = cfg.get("eos_token_id", ())
        eos = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(e) for e in eos)
        return cls(vocab_size=_need(cfg, "vocab", "the file"), width=_need(cfg, "width", "the file"),
                   layers=tuple(layers), norm_eps=_need(norm, "eps", "norm", float),
                   embed_scale=_need(emb, "scale", "embedding", float) if emb else 1.0,
                   side_dim=_need(side, "dim", "token_side") if side else 0,
                   max_positions=int(cfg.get("max_positions", DEFAULT_MAX_POSITIONS)), eos_token_ids=eos)

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embed_scale},
            "layers": [{"mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict(),
                        "type": L.type} for L in self.layers],
            "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width,
        }
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def replace(self, **changes: Any) -> "VonulixConfig":
        return dataclasses.replace(self, **changes)
