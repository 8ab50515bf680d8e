"""Typed configuration of the Zotonex design.

A small decoder-only model: pre-norm layers whose mixer is a differential
attention without positions under a chunked causal mask (a layer may read the
keys and values of an earlier layer instead of projecting its own) and whose
feed-forward, where a layer has one, is a mixture of experts with a gated shared
expert.  config.json is nested:

    {"architecture": "Zotonex", "vocab": V, "width": W, "norm": {"eps": e},
     "embedding": {"scale": s}, "logit_scale": c,
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff", "mask": {"size"}, "kv_from"?},
                 "mlp": null | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff", "limit"},
                                "shared"?: {"ff", "limit"}}}, ...]}

Every size and constant that may differ between models is read from there; what
the design fixes (the activation's 1.702, sigmoid scores that are not
renormalised, the weight on the expert's input) lives in the plan builder
(``models/zotonex.py``) as parameters of the parts.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, take_float, take_int

MAX_POSITIONS = 1 << 20     # the design has no position signal: the limit is the block tables' width alone


def _section(cfg: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = cfg.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}'{key}' must be an object")
    return value


@dataclass(frozen=True)
class ZotonexMixer:
    heads: int
    kv_heads: int
    dim: int            # elements of one query or key vector (a head has two of each)
    vdim: int           # elements of a head's value vector
    scale: float
    diff: float
    mask_size: int      # 0: every earlier key is seen
    kv_from: int | None = None

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "ZotonexMixer":
        mask = m.get("mask")
        if mask is not None and not isinstance(mask, Mapping):
            raise ConfigError(f"{where}'mask' must be an object or absent")
        kv_from = m.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"{where}'kv_from' must be a layer index, got {kv_from!r}")
        heads, dim = take_int(m, "heads"), take_int(m, "dim")
        self = cls(heads=heads, kv_heads=take_int(m, "kv_heads", heads), dim=dim, vdim=take_int(m, "vdim"),
                   scale=take_float(m, "scale", dim ** -0.5), diff=take_float(m, "diff", positive=False),
                   mask_size=take_int(mask, "size") if mask else 0, kv_from=kv_from)
        if self.heads % self.kv_heads:
            raise ConfigError(f"{where}heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        return self

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
               "diff": self.diff}
        if self.mask_size:
            out["mask"] = {"size": self.mask_size}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class ZotonexMoE:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int = 0          # 0: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, f: Mapping[str, Any], where: str) -> "ZotonexMoE":
        kind = f.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}'kind' = {kind!r}: the design's feed-forward is 'moe'")
        router, expert = _section(f, "router", where), _section(f, "expert", where)
        shared = f.get("shared")
        if shared is not None and not isinstance(shared, Mapping):
            raise ConfigError(f"{where}'shared' must be an object or absent")
        self = cls(experts=take_int(router, "experts"), top=take_int(router, "top"), ff=take_int(expert, "ff"),
                   limit=take_float(expert, "limit"), shared_ff=take_int(shared, "ff") if shared else 0,
                   shared_limit=take_float(shared, "limit") if shared else 0.0)
        if self.top > self.experts:
            raise ConfigError(f"{where}router.top {self.top} exceeds router.experts {self.experts}")
        return self

    def to_dict(self) -> dict:
        out = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff, "limit": self.limit}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


@dataclass(frozen=True)
class ZotonexLayer:
    mixer: ZotonexMixer
    mlp: ZotonexMoE | None
    type: str = "attention"


@dataclass(frozen=True)
class ZotonexConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple[ZotonexLayer, ...]

    architecture = "Zotonex"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "ZotonexConfig":
        raw = cfg.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]: "
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where}must be an object")
            kind = entry.get("type")
            if kind != "attention":
                raise ConfigError(f"{where}'type' = {kind!r}: the mixers built for this design are: attention")
            mixer = ZotonexMixer.from_dict(_section(entry, "mixer", where), where)
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}'mlp' must be an object or null")
            layers.append(ZotonexLayer(mixer, ZotonexMoE.from_dict(mlp, where) if mlp is not None else None, kind))
        for i, layer in enumerate(layers):
            j = layer.mixer.kv_from
            if j is None:
                continue
            if j >= i or layers[j].mixer.kv_from is not None:
                raise ConfigError(f"layers[{i}]: 'kv_from' = {j} must name an earlier layer that has keys and values of its own")
            a, b = layer.mixer, layers[j].mixer
            if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                raise ConfigError(f"layers[{i}]: kv_heads, dim and vdim must equal those of layer {j}, whose keys and values it reads")
        embedding = cfg.get("embedding") or {}
        return cls(vocab=take_int(cfg, "vocab"), width=take_int(cfg, "width"),
                   norm_eps=take_float(_section(cfg, "norm", ""), "eps"),
                   embedding_scale=take_float(embedding, "scale", 1.0),
                   logit_scale=take_float(cfg, "logit_scale", 1.0), layers=tuple(layers))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": l.mlp.to_dict() if l.mlp else None}
                           for l in self.layers]}
