"""Typed configuration of the Bobepel design, read from its own ``config.json``.

The file is nested like Safepel's: ``layers`` lists the layers in order, each with its ``type`` (which mixer:
``attention``, ``latent_attention`` or ``latent_attention_2``), the mixer's sizes and constants under ``mixer`` and
its feed-forward under ``mlp`` (null: none).  A layer may carry ``weights_of: j``: it then has no tensors of its own
and runs with layer j's, against a cache of its own.  Every size and every constant that differs between models of
the design is read from the file; nothing is assumed about how many layers of which type there are, in which order,
or which of them share weights.  A key that is not listed is ignored; a layer type, a feed-forward kind or a value
that the engine does not implement is refused by name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .schema import ConfigError, Key, positive, read_keys

ARCHITECTURE = "Bobepel"
DEFAULT_MAX_POSITIONS = 1 << 17   # the design has no position limit; the engine's block tables need one

_TOP = (
    Key("vocab", int, check=positive),
    Key("width", int, check=positive),
    Key("layers", list),
    Key("norm", object),
    Key("max_positions", int, default=DEFAULT_MAX_POSITIONS, check=positive),
)
_ATTENTION = (
    Key("heads", int, check=positive), Key("kv_heads", int, default=lambda v: v["heads"], check=positive),
    Key("dim", int, check=positive), Key("vdim", int, default=lambda v: v["dim"], check=positive), Key("scale", float), Key("q_temp", object, default=None, nullable=True),
    Key("mask", object, default=None, nullable=True),
)
_LATENT = (
    Key("heads", int, check=positive), Key("dim", int, check=positive), Key("rot_dim", int, check=positive),
    Key("vdim", int, check=positive), Key("kv_rank", int, check=positive), Key("scale", float), Key("rot", object),
    Key("q_rank", int, default=None, nullable=True, check=positive), Key("mask", object, default=None, nullable=True),
)
_MLP = (Key("kind", str), Key("expert", object), Key("router", object), Key("shared", object, default=None, nullable=True))
_EXPERT = (Key("ff", int, check=positive), Key("limit", float, check=positive))
_ROUTER = (Key("experts", int, check=positive), Key("top", int, check=positive))


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[Tuple[float, int]]   # (coef, every)
    window: Optional[int]


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: Optional[int]     # None: queries straight from the input
    scale: float
    rot_dims: int
    rot_base: float
    window: Optional[int]
    output_gate: bool


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int            # 0: no shared expert
    shared_limit: float


@dataclass(frozen=True)
class LayerConfig:
    type: str                 # attention | latent_attention | latent_attention_2
    mixer: object             # AttentionConfig | LatentAttentionConfig
    mlp: Optional[MoeConfig]  # None: the layer has no feed-forward
    weights_of: Optional[int]  # index of the layer whose tensors this one uses; None: its own


@dataclass(frozen=True)
class BobepelConfig:
    vocab: int
    width: int
    norm_eps: float
    max_positions: int
    layers: Tuple[LayerConfig, ...]

    @classmethod
    def from_json(cls, obj: dict) -> "BobepelConfig":
        v = read_keys(obj, _TOP)
        if not isinstance(v["norm"], dict):
            raise ConfigError("config.json: norm must be an object with 'eps'")
        eps = read_keys(v["norm"], (Key("eps", float, check=positive),), where="config.json: norm")["eps"]
        layers = []
        for i, raw in enumerate(v["layers"]):
            where = f"config.json: layers[{i}]"
            if not isinstance(raw, dict):
                raise ConfigError(f"{where}: must be an object")
            lv = read_keys(raw, (Key("type", str), Key("mixer", object), Key("mlp", object, default=None, nullable=True),
                                 Key("weights_of", int, default=None, nullable=True)), where=where)
            if not isinstance(lv["mixer"], dict):
                raise ConfigError(f"{where}: mixer must be an object")
            if lv["type"] == "attention":
                mixer = _attention(lv["mixer"], where + ".mixer")
            elif lv["type"] in ("latent_attention", "latent_attention_2"):
                mixer = _latent(lv["mixer"], where + ".mixer", second=lv["type"] == "latent_attention_2")
            else:
                raise ConfigError(f"{where}: layer type {lv['type']!r} is not implemented "
                                  "(attention, latent_attention, latent_attention_2)")
            mlp = _mlp(lv["mlp"], where + ".mlp") if lv["mlp"] is not None else None
            layers.append(LayerConfig(lv["type"], mixer, mlp, lv["weights_of"]))
        if not layers:
            raise ConfigError("config.json: layers is empty")
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            where = f"config.json: layers[{i}]"
            if not 0 <= j < len(layers) or j == i:
                raise ConfigError(f"{where}: weights_of={j} names no other layer")
            if layers[j].weights_of is not None:
                raise ConfigError(f"{where}: weights_of={j}, a layer that has no tensors of its own")
            if (layers[j].type, layers[j].mixer, layers[j].mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"{where}: its entry differs from that of layer {j}, whose weights it uses")
        return cls(vocab=v["vocab"], width=v["width"], norm_eps=eps, max_positions=v["max_positions"],
                   layers=tuple(layers))


def _window(mask, where: str) -> Optional[int]:
    if mask is None:
        return None
    if not isinstance(mask, dict) or not isinstance(mask.get("size"), int) or isinstance(mask.get("size"), bool) \
            or mask["size"] < 1:
        raise ConfigError(f"{where}: mask.size must be a positive integer")
    return mask["size"]


def _attention(raw: dict, where: str) -> AttentionConfig:
    m = read_keys(raw, _ATTENTION, where=where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
    q_temp = None
    if m["q_temp"] is not None:
        if not isinstance(m["q_temp"], dict):
            raise ConfigError(f"{where}: q_temp must be an object with 'coef' and 'every'")
        t = read_keys(m["q_temp"], (Key("coef", float), Key("every", int, check=positive)), where=where + ".q_temp")
        q_temp = (t["coef"], t["every"])
    return AttentionConfig(heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], scale=m["scale"],
                           q_temp=q_temp, window=_window(m["mask"], where))


def _latent(raw: dict, where: str, second: bool) -> LatentAttentionConfig:
    m = read_keys(raw, _LATENT, where=where)
    if not isinstance(m["rot"], dict):
        raise ConfigError(f"{where}: rot must be an object with 'dims' and 'base'")
    r = read_keys(m["rot"], (Key("dims", int), Key("base", float, check=positive)), where=where + ".rot")
    if r["dims"] % 2 or not 0 <= r["dims"] <= m["rot_dim"]:
        raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim")
    if second and m["q_rank"] is None:
        raise ConfigError(f"{where}: q_rank: required key is missing")
    return LatentAttentionConfig(
        heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"],
        q_rank=m["q_rank"] if second else None, scale=m["scale"], rot_dims=r["dims"], rot_base=r["base"],
        window=_window(m["mask"], where), output_gate=not second)


def _mlp(raw, where: str) -> MoeConfig:
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: must be an object or null")
    m = read_keys(raw, _MLP, where=where)
    if m["kind"] != "moe":
        raise ConfigError(f"{where}: kind {m['kind']!r} is not implemented (moe)")
    for key in ("expert", "router"):
        if not isinstance(m[key], dict):
            raise ConfigError(f"{where}.{key}: must be an object")
    e = read_keys(m["expert"], _EXPERT, where=where + ".expert")
    r = read_keys(m["router"], _ROUTER, where=where + ".router")
    if r["top"] > r["experts"]:
        raise ConfigError(f"{where}.router: top={r['top']} exceeds experts={r['experts']}")
    shared_ff, shared_limit = 0, 0.0
    if m["shared"] is not None:
        if not isinstance(m["shared"], dict):
            raise ConfigError(f"{where}.shared: must be an object or null")
        sh = read_keys(m["shared"], _EXPERT, where=where + ".shared")
        shared_ff, shared_limit = sh["ff"], sh["limit"]
    return MoeConfig(experts=r["experts"], top=r["top"], ff=e["ff"], limit=e["limit"], shared_ff=shared_ff,
                     shared_limit=shared_limit)
