"""Typed configuration of the Lomopel decoder, read from config.json's own keys.

A Lomopel model is a list of layers. A layer of type `attention` has softmax attention over all
earlier tokens (biased projections, no rotation, a query factor that grows with the position, a sink
in the softmax, optionally values mixed with those of the first such layer); a layer of type
`parallel` has two mixers side by side on the same input, attention over a sliding window (partial
rotary positions, q and k at unit root mean square, a sigmoid output gate) and a gated delta rule
(short causal convolutions, a decay per key channel), whose results are added with two weights.
Each layer may have a dense gated feed-forward. Norm weights are stored around zero, every
sub-layer's result is scaled per feature, the embedding is multiplied by a constant.

    {"architecture": "Lomopel", "vocab": ..., "width": ..., "embedding": {"scale": ...}, "norm": {"eps": ...},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "q_temp": {"coef", "every"}, "v_mix": true},
                 "mlp": {"kind": "dense", "ff": ...}},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"dims", "base"}},
                           "right": {"heads", "kv_heads", "dim", "vdim", "conv"}, "left_scale": ..., "right_scale": ...},
                 "mlp": null}]}

Every size and every constant that may differ between two models of the design is read here.
The ranks of the delta rule's two low-rank projections are no keys of config.json: they are the
shapes of the tensors (`right.decay_rank` / `right.gate_rank` may state them, and must where
weights are drawn at random instead of read). Optional keys: `q_temp` (absent: no query factor),
`v_mix` (absent: false), `rot` (absent: no rotation), `mask` (absent: every earlier token is seen).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from .model_config import _need, _typed
from .rotepel_config import _obj

NAME = "Lomopel"
LAYER_TYPES = ("attention", "parallel")


def _heads(m: dict, where: str) -> dict:
    kw = dict(heads=_need(m, "heads", int, where), kv_heads=_need(m, "kv_heads", int, where), dim=_need(m, "dim", int, where),
              vdim=_need(m, "vdim", int, where))
    for name, v in kw.items():
        if v <= 0:
            raise ConfigError(f"{where}: '{name}' must be positive")
    if kw["heads"] % kw["kv_heads"]:
        raise ConfigError(f"{where}: {kw['heads']} heads are not a multiple of {kw['kv_heads']} kv_heads")
    return kw


@dataclass(frozen=True)
class SoftmaxMixerConfig:
    """Softmax attention: the `attention` layer's mixer and the `left` half of a `parallel` one."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                       # keys a query sees, itself included; 0: all earlier ones
    rot_dims: int = 0                     # rotated features per head; 0: no rotation
    rot_base: float = 0.0
    q_temp: Optional[Tuple[float, int]] = None      # (coef, every)
    v_mix: bool = False

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "SoftmaxMixerConfig":
        kw = _heads(m, where)
        kw["scale"] = _need(m, "scale", float, where)
        mask = _obj(m, "mask", where, optional=True)
        if mask is not None:
            kw["window"] = _need(mask, "size", int, where + ".mask")
            if kw["window"] <= 0:
                raise ConfigError(f"{where}.mask: 'size' must be positive")
        rot = _obj(m, "rot", where, optional=True)
        if rot is not None:
            kw["rot_dims"] = _need(rot, "dims", int, where + ".rot")
            kw["rot_base"] = _need(rot, "base", float, where + ".rot")
            if kw["rot_dims"] % 2 or not 0 <= kw["rot_dims"] <= kw["dim"] or kw["rot_base"] <= 0:
                raise ConfigError(f"{where}.rot: dims {kw['rot_dims']} must be even and at most dim {kw['dim']}, base positive")
        qt = _obj(m, "q_temp", where, optional=True)
        if qt is not None:
            kw["q_temp"] = (_need(qt, "coef", float, where + ".q_temp"), _need(qt, "every", int, where + ".q_temp"))
            if kw["q_temp"][1] <= 0:
                raise ConfigError(f"{where}.q_temp: 'every' must be positive")
        if m.get("v_mix") is not None:
            kw["v_mix"] = _typed(m, "v_mix", bool, where)
        return cls(**kw)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dims:
            d["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        if self.q_temp is not None:
            d["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        if self.v_mix:
            d["v_mix"] = True
        return d


@dataclass(frozen=True)
class GatedDeltaConfig:
    """The `right` half of a `parallel` mixer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                             # taps of the short convolutions
    decay_rank: Optional[int] = None      # None: whatever the tensors' shapes say
    gate_rank: Optional[int] = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "GatedDeltaConfig":
        kw = _heads(m, where)
        kw["conv"] = _need(m, "conv", int, where)
        if kw["conv"] < 1:
            raise ConfigError(f"{where}: 'conv' must be at least 1")
        for key in ("decay_rank", "gate_rank"):
            if m.get(key) is not None:
                kw[key] = _typed(m, key, int, where)
        return cls(**kw)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            d["gate_rank"] = self.gate_rank
        return d


@dataclass(frozen=True)
class LomopelLayer:
    type: str
    attention: Optional[SoftmaxMixerConfig] = None      # type "attention"
    left: Optional[SoftmaxMixerConfig] = None           # type "parallel"
    right: Optional[GatedDeltaConfig] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    ff: int = 0                                         # 0: the layer has no feed-forward

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "LomopelLayer":
        if not isinstance(d, dict):
            raise ConfigError(f"{where}: a layer must be an object")
        kind = d.get("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}: 'type' must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
        m = _obj(d, "mixer", where)
        mw = where + ".mixer"
        kw = dict(type=kind)
        if kind == "attention":
            kw["attention"] = SoftmaxMixerConfig.from_dict(m, mw)
        else:
            kw["left"] = SoftmaxMixerConfig.from_dict(_obj(m, "left", mw), mw + ".left")
            kw["right"] = GatedDeltaConfig.from_dict(_obj(m, "right", mw), mw + ".right")
            kw["left_scale"] = _need(m, "left_scale", float, mw)
            kw["right_scale"] = _need(m, "right_scale", float, mw)
            if kw["left"].v_mix or kw["left"].q_temp is not None:
                raise ConfigError(f"{mw}.left: 'v_mix' and 'q_temp' belong to layers of type attention")
        mlp = _obj(d, "mlp", where, optional=True)
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise ConfigError(f"{where}.mlp: kind {mlp.get('kind')!r} is not known (dense)")
            kw["ff"] = _need(mlp, "ff", int, where + ".mlp")
            if kw["ff"] <= 0:
                raise ConfigError(f"{where}.mlp: 'ff' must be positive")
        return cls(**kw)

    def to_dict(self) -> dict:
        if self.type == "attention":
            m = self.attention.to_dict()
        else:
            m = {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                 "right_scale": self.right_scale}
        return {"type": self.type, "mixer": m, "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@dataclass(frozen=True)
class LomopelConfig:
    vocab: int
    width: int
    layers: Tuple[LomopelLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "LomopelConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        norm = _obj(d, "norm", where)
        emb = _obj(d, "embedding", where, optional=True)
        cfg = cls(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where),
                  layers=tuple(LomopelLayer.from_dict(x, f"{where}: layers[{i}]") for i, x in enumerate(layers)),
                  norm_eps=_need(norm, "eps", float, where + ".norm"),
                  embedding_scale=_need(emb, "scale", float, where + ".embedding") if emb is not None else 1.0)
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{where}: vocab and width must be positive")
        mixing = [x.attention for x in self.layers if x.type == "attention" and x.attention.v_mix]
        for a in mixing[1:]:
            if (a.kv_heads, a.vdim) != (mixing[0].kv_heads, mixing[0].vdim):
                raise ConfigError(f"{where}: layers that mix values must agree in kv_heads and vdim "
                                  f"({mixing[0].kv_heads} x {mixing[0].vdim} against {a.kv_heads} x {a.vdim})")

    def first_mixing_layer(self) -> Optional[int]:
        """The first layer whose attention says v_mix: the one whose values the later ones mix in."""
        for i, x in enumerate(self.layers):
            if x.type == "attention" and x.attention.v_mix:
                return i
        return None

    def param_count(self) -> int:
        from ..models.lomopel import lomopel_manifest
        total = 0
        for spec in lomopel_manifest(self).values():
            n = 1
            for x in spec.shape:
                n *= max(int(x), 0)
            total += n
        return total

    def to_dict(self) -> dict:
        return {"architecture": NAME, "vocab": self.vocab, "width": self.width, "embedding": {"scale": self.embedding_scale},
                "norm": {"eps": self.norm_eps}, "layers": [x.to_dict() for x in self.layers]}
