"""Typed configuration of the Rotepel decoder, read from config.json's own keys.

A Rotepel model is a list of layers, each with one of three mixers (`general_delta`, `retention`,
`latent_attention`) and an optional dense feed-forward, over a residual kept in `streams` streams
(hyper-connections) and normalised by an RMS norm in `norm.groups` groups. A range of the layers
(`loop`) may run several times in a row with the same weights. Every size and every constant that
may differ between two models of the design is read here; nothing below holds a number of any one
checkpoint.

    {"architecture": "Rotepel", "vocab": ..., "width": ..., "streams": ..., "norm": {"eps": ..., "groups": ...},
     "loop": {"start": ..., "stop": ..., "times": ...},
     "layers": [{"type": "general_delta", "mixer": {"heads": ..., "dim": ...}, "mlp": {"kind": "dense", "ff": ...}},
                {"type": "retention", "mixer": {"heads", "dim", "vdim", "decay": [...], "rot": {"dims", "base"}}, "mlp": null},
                {"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
                                                       "rot": {"dims", "base"}}, "mlp": {...}}]}

`streams` absent: one residual and no stream coefficients among the tensors. `loop` absent: every
layer runs once. The rank of a `general_delta` mixer's decay projection is no key of config.json:
it is the shape of the tensor (`mixer.decay_rank` may state it, and must where weights are drawn at
random instead of read).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from .model_config import _need, _typed

NAME = "Rotepel"
MIXERS = ("general_delta", "retention", "latent_attention")


def _obj(d, key, where, optional=False):
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object")
    return v


@dataclass(frozen=True)
class RotepelLayer:
    type: str
    heads: int
    dim: int
    vdim: int = 0                       # retention, latent_attention
    decay: Tuple[float, ...] = ()       # retention: one per head
    rot_dims: int = 0                   # retention: rotated features per head; latent_attention: = rot_dim
    rot_base: float = 0.0
    rot_dim: int = 0                    # latent_attention
    kv_rank: int = 0                    # latent_attention
    scale: float = 0.0                  # latent_attention
    decay_rank: Optional[int] = None    # general_delta: None = whatever the tensor's shape says
    ff: int = 0                         # 0: the layer has no feed-forward

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "RotepelLayer":
        if not isinstance(d, dict):
            raise ConfigError(f"{where}: a layer must be an object")
        kind = d.get("type")
        if kind not in MIXERS:
            raise ConfigError(f"{where}: 'type' must be one of {', '.join(MIXERS)}, got {kind!r}")
        m = _obj(d, "mixer", where)
        mw = where + ".mixer"
        kw = dict(type=kind, heads=_need(m, "heads", int, mw), dim=_need(m, "dim", int, mw))
        if kind == "general_delta":
            if "decay_rank" in m and m["decay_rank"] is not None:
                kw["decay_rank"] = _typed(m, "decay_rank", int, mw)
        if kind in ("retention", "latent_attention"):
            kw["vdim"] = _need(m, "vdim", int, mw)
            rot = _obj(m, "rot", mw)
            kw["rot_dims"] = _need(rot, "dims", int, mw + ".rot")
            kw["rot_base"] = _need(rot, "base", float, mw + ".rot")
        if kind == "retention":
            dec = m.get("decay")
            if not isinstance(dec, list) or len(dec) != kw["heads"] or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in dec):
                raise ConfigError(f"{mw}: 'decay' must list one number per head ({kw['heads']})")
            kw["decay"] = tuple(float(x) for x in dec)
            if kw["rot_dims"] % 2 or not 0 <= kw["rot_dims"] <= kw["dim"]:
                raise ConfigError(f"{mw}: rot.dims {kw['rot_dims']} must be even and at most dim {kw['dim']}")
        if kind == "latent_attention":
            kw["rot_dim"] = _need(m, "rot_dim", int, mw)
            kw["kv_rank"] = _need(m, "kv_rank", int, mw)
            kw["scale"] = _need(m, "scale", float, mw)
            if kw["rot_dims"] != kw["rot_dim"] or kw["rot_dim"] % 2 or kw["rot_dim"] <= 0:
                raise ConfigError(f"{mw}: rot.dims must equal rot_dim, an even number; got {kw['rot_dims']} and {kw['rot_dim']}")
        mlp = _obj(d, "mlp", where, optional=True)
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise ConfigError(f"{where}.mlp: kind {mlp.get('kind')!r} is not known (dense)")
            kw["ff"] = _need(mlp, "ff", int, where + ".mlp")
        layer = cls(**kw)
        for name in ("heads", "dim") + (("vdim",) if kind != "general_delta" else ()) + (("kv_rank",) if kind == "latent_attention" else ()):
            if getattr(layer, name) <= 0:
                raise ConfigError(f"{mw}: '{name}' must be positive")
        return layer

    def to_dict(self) -> dict:
        m = {"heads": self.heads, "dim": self.dim}
        if self.type == "general_delta" and self.decay_rank is not None:
            m["decay_rank"] = self.decay_rank
        if self.type in ("retention", "latent_attention"):
            m["vdim"] = self.vdim
            m["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        if self.type == "retention":
            m["decay"] = list(self.decay)
        if self.type == "latent_attention":
            m.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank, scale=self.scale)
        return {"type": self.type, "mixer": m, "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@dataclass(frozen=True)
class RotepelConfig:
    vocab: int
    width: int
    layers: Tuple[RotepelLayer, ...]
    norm_eps: float
    norm_groups: int = 1
    streams: Optional[int] = None       # None: one residual, no stream coefficients
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times)
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "RotepelConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        norm = _obj(d, "norm", where)
        streams = _typed(d, "streams", int, where) if d.get("streams") is not None else None
        loop = None
        lp = _obj(d, "loop", where, optional=True)
        if lp is not None:
            loop = (_need(lp, "start", int, where + ".loop"), _need(lp, "stop", int, where + ".loop"),
                    _need(lp, "times", int, where + ".loop"))
        cfg = cls(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where),
                  layers=tuple(RotepelLayer.from_dict(x, f"{where}: layers[{i}]") for i, x in enumerate(layers)),
                  norm_eps=_need(norm, "eps", float, where + ".norm"),
                  norm_groups=_typed(norm, "groups", int, where + ".norm") if norm.get("groups") is not None else 1,
                  streams=streams, loop=loop)
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{where}: vocab and width must be positive")
        if self.norm_groups < 1 or self.width % self.norm_groups:
            raise ConfigError(f"{where}: a width of {self.width} cannot be cut into {self.norm_groups} norm groups")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise ConfigError(f"{where}: streams must be 1..8, got {self.streams}")
        if self.loop is not None:
            a, b, times = self.loop
            if not (0 <= a <= b <= len(self.layers)) or times < 1:
                raise ConfigError(f"{where}: loop {self.loop} does not fit {len(self.layers)} layers")

    def run_order(self) -> Tuple[int, ...]:
        """Layer numbers in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    def param_count(self) -> int:
        from ..models.rotepel import rotepel_manifest
        total = 0
        for spec in rotepel_manifest(self).values():
            n = 1
            for x in spec.shape:
                n *= max(int(x), 0)
            total += n
        return total

    def to_dict(self) -> dict:
        d = {"architecture": NAME, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
             "layers": [x.to_dict() for x in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d
