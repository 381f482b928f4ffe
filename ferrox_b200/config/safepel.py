"""Typed configuration of the Safepel design, read from its own ``config.json``.

The file is nested: ``layers`` lists the layers in order, each with its ``type`` (which mixer: ``delta`` or
``parallel``), the mixer's sizes under ``mixer`` and its feed-forward under ``mlp`` (null: none).  Every size and
every constant that differs between models of the design is read from there; nothing is assumed about how many
layers of which type there are or in which order.  A key that is not listed is ignored (the file may carry
book-keeping); a layer type, a feed-forward kind or a value that the engine does not implement is refused by name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .schema import ConfigError, Key, positive, read_keys

ARCHITECTURE = "Safepel"
DEFAULT_MAX_POSITIONS = 1 << 17   # the design has no position limit; the engine's block tables need one

_TOP = (
    Key("vocab", int, check=positive),
    Key("width", int, check=positive),
    Key("layers", list),
    Key("norm", object),
    Key("logit_scale", float, default=1.0),
    Key("max_positions", int, default=DEFAULT_MAX_POSITIONS, check=positive),
)

_DELTA = (
    Key("heads", int, check=positive), Key("kv_heads", int, check=positive), Key("dim", int, check=positive),
    Key("vdim", int, check=positive), Key("conv", int, check=positive),
)
_LEFT = (
    Key("heads", int, check=positive), Key("kv_heads", int, check=positive), Key("dim", int, check=positive),
    Key("vdim", int, check=positive), Key("scale", float), Key("softcap", float, check=positive),
    Key("mask", object), Key("rot", object),
)
_RIGHT = (
    Key("heads", int, check=positive), Key("dim", int, check=positive), Key("vdim", int, check=positive),
    Key("decay", list),
)
_PARALLEL = (Key("left", object), Key("right", object), Key("left_scale", float), Key("right_scale", float))
_MLP = (Key("kind", str), Key("ff", int, check=positive))


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    window: int
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class LinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: LinearAttentionConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class LayerConfig:
    type: str                 # delta | parallel
    mixer: object             # DeltaMixerConfig | ParallelMixerConfig
    ff: Optional[int]         # width of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class SafepelConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    max_positions: int
    layers: Tuple[LayerConfig, ...]

    @classmethod
    def from_json(cls, obj: dict) -> "SafepelConfig":
        v = read_keys(obj, _TOP)
        if not isinstance(v["norm"], dict):
            raise ConfigError("config.json: norm must be an object with 'eps'")
        eps = read_keys(v["norm"], (Key("eps", float, check=positive),), where="config.json: norm")["eps"]
        layers = []
        for i, raw in enumerate(v["layers"]):
            where = f"config.json: layers[{i}]"
            if not isinstance(raw, dict):
                raise ConfigError(f"{where}: must be an object")
            lv = read_keys(raw, (Key("type", str), Key("mixer", object), Key("mlp", object, default=None, nullable=True)),
                           where=where)
            if not isinstance(lv["mixer"], dict):
                raise ConfigError(f"{where}: mixer must be an object")
            if lv["type"] == "delta":
                m = read_keys(lv["mixer"], _DELTA, where=where + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: heads must be a multiple of kv_heads")
                mixer = DeltaMixerConfig(**m)
            elif lv["type"] == "parallel":
                mixer = _parallel(lv["mixer"], where + ".mixer")
            else:
                raise ConfigError(f"{where}: layer type {lv['type']!r} is not implemented (delta, parallel)")
            ff = None
            if lv["mlp"] is not None:
                if not isinstance(lv["mlp"], dict):
                    raise ConfigError(f"{where}: mlp must be an object or null")
                mv = read_keys(lv["mlp"], _MLP, where=where + ".mlp")
                if mv["kind"] != "dense":
                    raise ConfigError(f"{where}.mlp: kind {mv['kind']!r} is not implemented (dense)")
                ff = mv["ff"]
            layers.append(LayerConfig(lv["type"], mixer, ff))
        if not layers:
            raise ConfigError("config.json: layers is empty")
        return cls(vocab=v["vocab"], width=v["width"], norm_eps=eps, logit_scale=v["logit_scale"],
                   max_positions=v["max_positions"], layers=tuple(layers))


def _parallel(raw: dict, where: str) -> ParallelMixerConfig:
    p = read_keys(raw, _PARALLEL, where=where)
    for side in ("left", "right"):
        if not isinstance(p[side], dict):
            raise ConfigError(f"{where}.{side}: must be an object")
    l = read_keys(p["left"], _LEFT, where=where + ".left")
    problems = []
    if not isinstance(l["mask"], dict) or not isinstance(l["mask"].get("size"), int) or l["mask"]["size"] < 1:
        problems.append("mask.size must be a positive integer")
    if not isinstance(l["rot"], dict) or not isinstance(l["rot"].get("dims"), int) or "base" not in l["rot"]:
        problems.append("rot needs 'dims' and 'base'")
    elif l["rot"]["dims"] % 2 or not 0 <= l["rot"]["dims"] <= l["dim"]:
        problems.append("rot.dims must be even and at most dim")
    if l["heads"] % l["kv_heads"]:
        problems.append("heads must be a multiple of kv_heads")
    if l["vdim"] != l["dim"]:
        problems.append("vdim must equal dim (the values are the keys)")
    if problems:
        raise ConfigError(f"{where}.left: " + "; ".join(problems))
    left = WindowAttentionConfig(heads=l["heads"], kv_heads=l["kv_heads"], dim=l["dim"], vdim=l["vdim"],
                                 scale=l["scale"], softcap=l["softcap"], window=l["mask"]["size"],
                                 rot_dims=l["rot"]["dims"], rot_base=float(l["rot"]["base"]))
    r = read_keys(p["right"], _RIGHT, where=where + ".right")
    try:
        decay = tuple(float(d) for d in r["decay"])
    except (TypeError, ValueError):
        raise ConfigError(f"{where}.right: decay must list numbers") from None
    if len(decay) != r["heads"]:
        raise ConfigError(f"{where}.right: decay lists {len(decay)} values for {r['heads']} heads")
    right = LinearAttentionConfig(heads=r["heads"], dim=r["dim"], vdim=r["vdim"], decay=decay)
    return ParallelMixerConfig(left, right, p["left_scale"], p["right_scale"])
