"""Typed configuration of the Zoferax decoder.

config.json of this design is nested: ``architecture`` (a string), ``width``, ``vocab``,
``embedding.scale``, ``norm.eps`` and ``layers``, a list with one entry per layer: ``type`` (the kind of
mixer; ``attention`` is the one kind), ``mixer`` (``heads``, ``kv_heads``, ``dim`` = the query/key size of
a head, ``vdim`` = its value size, ``scale`` = the factor on the scores, and optionally ``kv_from`` = the
index of an earlier layer whose keys and values this layer reads instead of projecting its own) and ``mlp``
(null for a layer without feed-forward, else ``kind`` = ``moe`` with ``expert.ff``, ``router.experts`` and
``router.top``).  Every size and constant that a model of the design may set is read from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, required_float, required_int

_FAMILY = "zoferax"


def _mapping(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError.unsupported(f"{_FAMILY} config {where} missing {key}")
    return value


@dataclass(frozen=True)
class ZoferaxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class ZoferaxExperts:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class ZoferaxLayer:
    kind: str
    mixer: ZoferaxAttention
    mlp: Optional[ZoferaxExperts]


@dataclass(frozen=True)
class ZoferaxConfig:
    width: int
    vocab: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[ZoferaxLayer, ...]

    architecture = "Zoferax"
    SINUSOID_BASE = 10000.0  # fixed by the design

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZoferaxConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError.unsupported(f"config is not a {cls.architecture} model: architecture={raw.get('architecture')!r}")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError.unsupported(f"{_FAMILY} config missing layers")
        layers = []
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            if not isinstance(entry, Mapping):
                raise ConfigError.invalid(f"{_FAMILY} config {where} must be an object")
            kind = entry.get("type")
            if kind != "attention":
                raise ConfigError.unsupported(f"{_FAMILY} config {where}: layer type {kind!r} is unsupported; only 'attention' is")
            m = _mapping(entry, "mixer", where)
            heads, kv_heads = required_int(m, "heads", _FAMILY), required_int(m, "kv_heads", _FAMILY)
            if heads % kv_heads:
                raise ConfigError.invalid(f"{_FAMILY} config {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
            kv_from = m.get("kv_from")
            if kv_from is not None:
                if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < index:
                    raise ConfigError.invalid(f"{_FAMILY} config {where}: kv_from must name an earlier layer, got {kv_from!r}")
                source = layers[kv_from].mixer
                if source.kv_from is not None:
                    raise ConfigError.invalid(f"{_FAMILY} config {where}: layer {kv_from} has no keys and values of its own")
            mixer = ZoferaxAttention(heads=heads, kv_heads=kv_heads, dim=required_int(m, "dim", _FAMILY),
                                     vdim=required_int(m, "vdim", _FAMILY), scale=required_float(m, "scale", _FAMILY),
                                     kv_from=kv_from)
            if kv_from is not None:
                source = layers[kv_from].mixer
                if (source.kv_heads, source.dim, source.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                    raise ConfigError.invalid(f"{_FAMILY} config {where}: layer {kv_from}'s keys and values do not fit this layer's heads")
            mlp = entry.get("mlp")
            experts = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
                    raise ConfigError.unsupported(f"{_FAMILY} config {where}: feed-forward kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is unsupported; only 'moe' is")
                router = _mapping(mlp, "router", where + ".mlp")
                experts = ZoferaxExperts(experts=required_int(router, "experts", _FAMILY), top=required_int(router, "top", _FAMILY),
                                         ff=required_int(_mapping(mlp, "expert", where + ".mlp"), "ff", _FAMILY))
                if experts.top > experts.experts:
                    raise ConfigError.invalid(f"{_FAMILY} config {where}: top {experts.top} exceeds {experts.experts} experts")
            layers.append(ZoferaxLayer(kind, mixer, experts))
        eps = required_float(_mapping(raw, "norm", "root"), "eps", _FAMILY)
        if eps < 0.0:
            raise ConfigError.invalid(f"{_FAMILY} config norm.eps must be non-negative")
        return cls(width=required_int(raw, "width", _FAMILY), vocab=required_int(raw, "vocab", _FAMILY),
                   embedding_scale=required_float(_mapping(raw, "embedding", "root"), "scale", _FAMILY), norm_eps=eps,
                   layers=tuple(layers))

    def to_dict(self) -> dict:
        """The config.json content that parses back to this configuration."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer = {"dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "scale": m.scale, "vdim": m.vdim}
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            mlp = None
            if layer.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": layer.mlp.ff},
                       "router": {"experts": layer.mlp.experts, "top": layer.mlp.top}}
            layers.append({"type": layer.kind, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers}
