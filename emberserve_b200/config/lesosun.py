"""Typed configuration of the Lesosun decoder, read from its own ``config.json`` keys.

``layers`` lists the layers in order; each names its mixer ``type`` (``parallel``: grouped-query
attention with capped scores behind short convolutions, beside a selective state space with a scalar
decay per head; ``channel_delta``: the delta rule with a decay per key channel), the mixer's sizes
under ``mixer`` and its feed-forward under ``mlp`` (``dense``, ``moe`` or null).  ``norm`` holds what
all layers share; ``residual_mult`` multiplies what a layer adds to the stream; ``logit_softcap``
caps the logits.  Every size and constant is taken from the file.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, ClassVar

from emberserve_b200.config.damolorn import DEFAULT_MAX_POSITIONS, _need
from emberserve_b200.config.model import ConfigError, ModelConfig

MIXER_TYPES = ("parallel", "channel_delta")


@dataclass(frozen=True)
class CappedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    softcap: float | None
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "CappedAttentionConfig":
        rot = d.get("rot") or {}
        cap = d.get("softcap")
        m = cls(heads=_need(d, "heads", where), kv_heads=int(d.get("kv_heads") or _need(d, "heads", where)),
                dim=_need(d, "dim", where), vdim=int(d.get("vdim") or _need(d, "dim", where)),
                conv=int(d.get("conv") or 1), scale=_need(d, "scale", where, float),
                softcap=None if not cap else _need(d, "softcap", where, float),
                rot_dims=_need(rot, "dims", where + ".rot") if rot else 0,
                rot_base=_need(rot, "base", where + ".rot", float) if rot else 10000.0)
        if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads or m.dim <= 0 or m.vdim <= 0 or m.conv < 1:
            raise ConfigError(f"config.json: {where}: heads={m.heads}, kv_heads={m.kv_heads}, dim={m.dim}, "
                              f"vdim={m.vdim}, conv={m.conv}")
        if m.rot_dims < 0 or m.rot_dims % 2 or m.rot_dims > m.dim or (m.rot_dims and m.rot_base <= 0):
            raise ConfigError(f"config.json: {where}.rot: dims={m.rot_dims} must be even and at most dim={m.dim}")
        if m.softcap is not None and not m.softcap > 0:
            raise ConfigError(f"config.json: {where}.softcap must be positive")
        return m

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                             "scale": self.scale, "vdim": self.vdim}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "StateSpaceConfig":
        m = cls(heads=_need(d, "heads", where), vdim=_need(d, "vdim", where), state=_need(d, "state", where),
                groups=int(d.get("groups") or 1), norm_groups=int(d.get("norm_groups") or 1),
                conv=int(d.get("conv") or 1))
        if m.heads <= 0 or m.vdim <= 0 or m.state <= 0 or m.groups <= 0 or m.heads % m.groups or m.conv < 1:
            raise ConfigError(f"config.json: {where}: heads={m.heads} in {m.groups} groups, vdim={m.vdim}, "
                              f"state={m.state}, conv={m.conv}")
        if m.norm_groups <= 0 or (m.heads * m.vdim) % m.norm_groups:
            raise ConfigError(f"config.json: {where}: {m.heads * m.vdim} channels do not split into "
                              f"{m.norm_groups} equal norm groups")
        return m

    def to_dict(self) -> dict[str, Any]:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: CappedAttentionConfig
    right: StateSpaceConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "ParallelMixerConfig":
        return cls(CappedAttentionConfig.from_dict(_need(d, "left", where, dict), where + ".left"),
                   StateSpaceConfig.from_dict(_need(d, "right", where, dict), where + ".right"),
                   float(d["left_scale"]) if d.get("left_scale") is not None else 1.0,
                   float(d["right_scale"]) if d.get("right_scale") is not None else 1.0)

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    # Inner sizes of the two-step projections of the decay and of the output gate.  The file need not
    # give them: the shapes of the checkpoint's tensors do (`LesosunConfig.with_tensor_shapes`).
    decay_rank: int | None = None
    gate_rank: int | None = None

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "ChannelDeltaConfig":
        m = cls(heads=_need(d, "heads", where), kv_heads=int(d.get("kv_heads") or _need(d, "heads", where)),
                dim=_need(d, "dim", where), vdim=_need(d, "vdim", where), conv=int(d.get("conv") or 1),
                decay_rank=int(d["decay_rank"]) if d.get("decay_rank") else None,
                gate_rank=int(d["gate_rank"]) if d.get("gate_rank") else None)
        if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads or m.dim <= 0 or m.vdim <= 0 or m.conv < 1:
            raise ConfigError(f"config.json: {where}: heads={m.heads}, kv_heads={m.kv_heads}, dim={m.dim}, "
                              f"vdim={m.vdim}, conv={m.conv}")
        return m

    def to_dict(self) -> dict[str, Any]:
        d = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            d["gate_rank"] = self.gate_rank
        return d


_MIXER_CONFIGS = {"parallel": ParallelMixerConfig, "channel_delta": ChannelDeltaConfig}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str  # "dense" or "moe"
    ff: int  # of the dense feed-forward, or of one expert
    experts: int = 0  # experts with weights
    identity: int = 0  # further router outputs whose expert returns its input
    top: int = 0
    route_scale: float = 1.0
    shared_ff: int | None = None

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "FeedForwardConfig":
        kind = _need(d, "kind", where, str)
        if kind == "dense":
            f = cls("dense", _need(d, "ff", where))
        elif kind == "moe":
            router = _need(d, "router", where, dict)
            shared = d.get("shared")
            f = cls("moe", _need(_need(d, "expert", where, dict), "ff", where + ".expert"),
                    experts=_need(router, "experts", where + ".router"), identity=int(router.get("identity") or 0),
                    top=_need(router, "top", where + ".router"),
                    route_scale=float(router["scale"]) if router.get("scale") is not None else 1.0,
                    shared_ff=None if not shared else _need(shared, "ff", where + ".shared"))
            if f.experts <= 0 or f.identity < 0 or not 1 <= f.top <= f.experts + f.identity:
                raise ConfigError(f"config.json: {where}.router: top={f.top} of {f.experts} experts and "
                                  f"{f.identity} identity experts")
            if f.shared_ff is not None and f.shared_ff <= 0:
                raise ConfigError(f"config.json: {where}.shared.ff must be positive")
        else:
            raise ConfigError(f"config.json: {where}.kind {kind!r}: 'dense' or 'moe'")
        if f.ff <= 0:
            raise ConfigError(f"config.json: {where}: ff must be positive")
        return f

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        d: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe",
                             "router": {"experts": self.experts, "identity": self.identity,
                                        "scale": self.route_scale, "top": self.top}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class LesosunLayerConfig:
    type: str
    mixer: "ParallelMixerConfig | ChannelDeltaConfig"
    mlp: FeedForwardConfig | None


@dataclass(frozen=True)
class LesosunConfig(ModelConfig):
    architecture: ClassVar[str] = "Lesosun"
    wants_tensor_shapes: ClassVar[bool] = True

    vocab_size: int
    width: int
    layers: tuple[LesosunLayerConfig, ...]
    norm_eps: float
    residual_mult: float = 1.0
    logit_softcap: float | None = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        if self.max_positions <= 0:
            raise ConfigError("max_positions must be positive")

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "LesosunConfig":
        layers = []
        for i, entry in enumerate(_need(cfg, "layers", "the file", list)):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where, str)
            if kind not in _MIXER_CONFIGS:
                raise ConfigError(f"config.json: {where}.type {kind!r}: one of {MIXER_TYPES}")
            mlp = entry.get("mlp")
            layers.append(LesosunLayerConfig(
                kind, _MIXER_CONFIGS[kind].from_dict(_need(entry, "mixer", where, dict), where + ".mixer"),
                None if mlp is None else FeedForwardConfig.from_dict(mlp, where + ".mlp")))
        norm = _need(cfg, "norm", "the file", dict)
        eos = cfg.get("eos_token_id", ())
        eos = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(e) for e in eos)
        cap = cfg.get("logit_softcap")
        return cls(vocab_size=_need(cfg, "vocab", "the file"), width=_need(cfg, "width", "the file"),
                   layers=tuple(layers), norm_eps=_need(norm, "eps", "norm", float),
                   residual_mult=float(cfg["residual_mult"]) if cfg.get("residual_mult") is not None else 1.0,
                   logit_softcap=None if not cap else _need(cfg, "logit_softcap", "the file", float),
                   max_positions=int(cfg.get("max_positions", DEFAULT_MAX_POSITIONS)), eos_token_ids=eos)

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict(),
                        "type": L.type} for L in self.layers],
            "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab_size,
            "width": self.width,
        }
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def with_tensor_shapes(self, shapes: "dict[str, tuple[int, ...]]") -> "LesosunConfig":
        """The inner sizes of the two-step projections of every channel_delta layer, from the rows of
        ``l<i>.mix.a1`` and ``l<i>.mix.g1``."""
        layers = []
        for i, L in enumerate(self.layers):
            if isinstance(L.mixer, ChannelDeltaConfig):
                a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
                m = L.mixer
                for name, shape, given in (("a1", a1, m.decay_rank), ("g1", g1, m.gate_rank)):
                    if shape is not None and given is not None and shape[0] != given:
                        raise ConfigError(f"layers[{i}].mixer: the file says {given} rows for l{i}.mix.{name}, "
                                          f"the tensor has {shape[0]}")
                m = dataclasses.replace(m, decay_rank=m.decay_rank if a1 is None else int(a1[0]),
                                        gate_rank=m.gate_rank if g1 is None else int(g1[0]))
                L = dataclasses.replace(L, mixer=m)
            layers.append(L)
        return dataclasses.replace(self, layers=tuple(layers))

    def replace(self, **changes: Any) -> "LesosunConfig":
        return dataclasses.replace(self, **changes)
