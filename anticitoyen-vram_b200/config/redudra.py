"""Typed configuration of the Redudra design.

A small decoder-only model over a float32 residual stream.  Every layer is
pre-norm (layer norms with weight and bias) with a token shift in front of its
mixer and a constant ``residual_mult`` on what its parts add to the stream; the
mixer is either ``parallel`` (a softmax attention under a sliding window that
keeps a request's first tokens, beside a retention, their outputs summed with
weights) or ``rglru`` (a gated linear recurrence behind a short convolution);
the feed-forward is a gated unit with biases, or absent.  A stretch of layers may
run several times over the same weights (``loop``), each pass with a state of its
own and a vector of its own added to the stream first.  The logits pass through a
soft cap.  config.json is nested:

    {"architecture": "Redudra", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "logit_softcap": c, "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "keep_first"},
                                    "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                           "right": {"heads", "dim", "vdim", "decay": [...], "rot": {"base", "dims"}},
                           "left_scale", "right_scale"},
                 "mlp": null | {"kind": "dense", "ff": F}},
                {"type": "rglru", "mixer": {"width", "blocks", "conv"}, "mlp": ...}, ...]}

Every size and constant that may differ between models is read from there.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, take_float, take_int

MAX_POSITIONS = 1 << 17     # rows of the rotary tables; the design itself names no longest sequence


def _section(cfg: Mapping[str, Any], key: str, where: str, optional: bool = False):
    value = cfg.get(key)
    if value is None and optional:
        return None
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}'{key}' must be an object")
    return value


@dataclass(frozen=True)
class RotarySpec:
    base: float
    dims: int
    scaling: tuple[float, float, float, float] | None = None     # (factor, original length, fast, slow)

    @classmethod
    def from_dict(cls, r: Mapping[str, Any], where: str, head_dim: int) -> "RotarySpec":
        dims = take_int(r, "dims", minimum=2)
        if dims % 2 or dims > head_dim:
            raise ConfigError(f"{where}rot.dims {dims} must be even and at most the head's {head_dim}")
        sc = r.get("scaling")
        scaling = None
        if sc is not None:
            if not isinstance(sc, Mapping):
                raise ConfigError(f"{where}rot.scaling must be an object or absent")
            scaling = (take_float(sc, "factor"), take_float(sc, "original"), take_float(sc, "fast"), take_float(sc, "slow"))
        return cls(take_float(r, "base"), dims, scaling)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            f, o, fast, slow = self.scaling
            out["scaling"] = {"factor": f, "original": int(o) if float(o).is_integer() else o, "fast": fast, "slow": slow}
        return out


@dataclass(frozen=True)
class WindowedAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int             # 0: every earlier key is seen
    keep_first: int
    rot: RotarySpec | None

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "WindowedAttentionSpec":
        heads, dim = take_int(m, "heads"), take_int(m, "dim")
        kv = take_int(m, "kv_heads", heads)
        if heads % kv:
            raise ConfigError(f"{where}heads {heads} is not a multiple of kv_heads {kv}")
        mask = _section(m, "mask", where, optional=True)
        rot = _section(m, "rot", where, optional=True)
        return cls(heads, kv, dim, take_int(m, "vdim", dim), take_float(m, "scale", dim ** -0.5),
                   take_int(mask, "size", 0, minimum=0) if mask else 0,
                   take_int(mask, "keep_first", 0, minimum=0) if mask else 0,
                   RotarySpec.from_dict(rot, where, dim) if rot else None)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.window:
            out["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class RetentionSpec:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: RotarySpec | None

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "RetentionSpec":
        heads, dim = take_int(m, "heads"), take_int(m, "dim")
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads or \
                any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"{where}'decay' must list one number for each of the {heads} heads")
        rot = _section(m, "rot", where, optional=True)
        return cls(heads, dim, take_int(m, "vdim", dim), tuple(float(d) for d in decay),
                   RotarySpec.from_dict(rot, where, dim) if rot else None)

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class ParallelSpec:
    left: WindowedAttentionSpec
    right: RetentionSpec
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "ParallelSpec":
        return cls(WindowedAttentionSpec.from_dict(_section(m, "left", where), where + "left: "),
                   RetentionSpec.from_dict(_section(m, "right", where), where + "right: "),
                   take_float(m, "left_scale", 1.0, positive=False), take_float(m, "right_scale", 1.0, positive=False))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class RecurrenceSpec:
    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "RecurrenceSpec":
        self = cls(take_int(m, "width"), take_int(m, "blocks", 1), take_int(m, "conv", 1))
        if self.width % self.blocks:
            raise ConfigError(f"{where}width {self.width} does not split into {self.blocks} equal blocks")
        return self

    def to_dict(self) -> dict:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class RedudraLayer:
    type: str                               # "parallel" | "rglru"
    mixer: ParallelSpec | RecurrenceSpec
    ff: int                                 # 0: the layer has no feed-forward


@dataclass(frozen=True)
class RedudraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_softcap: float        # 0: none
    loop: tuple[int, int, int] | None       # (start, stop, times)
    layers: tuple[RedudraLayer, ...]

    architecture = "Redudra"
    MIXERS = {"parallel": ParallelSpec, "rglru": RecurrenceSpec}

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "RedudraConfig":
        raw = cfg.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]: "
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where}must be an object")
            kind = entry.get("type")
            spec = cls.MIXERS.get(kind)
            if spec is None:
                raise ConfigError(f"{where}'type' = {kind!r}: the mixers built for this design are: {', '.join(sorted(cls.MIXERS))}")
            mixer = spec.from_dict(_section(entry, "mixer", where), where)
            mlp = entry.get("mlp")
            ff = 0
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}'mlp' must be an object or null")
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}mlp.kind = {mlp.get('kind')!r}: the design's feed-forward is 'dense'")
                ff = take_int(mlp, "ff")
            layers.append(RedudraLayer(kind, mixer, ff))
        loop = None
        raw_loop = cfg.get("loop")
        if raw_loop is not None:
            if not isinstance(raw_loop, Mapping):
                raise ConfigError("'loop' must be an object or absent")
            start, stop = take_int(raw_loop, "start", minimum=0), take_int(raw_loop, "stop", minimum=0)
            times = take_int(raw_loop, "times", 1)
            if not start < stop <= len(layers):
                raise ConfigError(f"loop: start {start} and stop {stop} must name a stretch of the {len(layers)} layers")
            loop = (start, stop, times)
        cap = cfg.get("logit_softcap")
        return cls(vocab=take_int(cfg, "vocab"), width=take_int(cfg, "width"),
                   norm_eps=take_float(_section(cfg, "norm", ""), "eps"),
                   residual_mult=take_float(cfg, "residual_mult", 1.0, positive=False),
                   logit_softcap=take_float(cfg, "logit_softcap") if cap else 0.0, loop=loop, layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None}
                       for l in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out
