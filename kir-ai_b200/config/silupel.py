"""Typed configuration of the Silupel decoder.

config.json of this design is nested: ``architecture`` (a string), ``width``, ``vocab``, ``norm.eps``, ``layers`` and
optionally ``loop``.  Every entry of ``layers`` has ``type`` (the kind of mixer), ``mixer`` (its sizes and constants)
and ``mlp`` (null for a layer without feed-forward, else ``kind`` = ``dense`` with ``ff``).  The kinds of mixer:

* ``mingru``: ``width`` of the recurrence;
* ``attention``: ``heads``, ``kv_heads``, ``dim`` (query/key size of a head), ``vdim`` (its value size), ``scale``
  (the factor on the scores), ``rot`` (``base``, ``dims`` = how many leading columns of a head are rotated, and
  optionally ``scaling`` with ``factor``, ``low``, ``high``, ``original``), and optionally ``softcap`` and ``mask``
  (``size`` of the chunks inside which a position sees earlier ones);
* ``latent_attention``: ``heads``, ``dim`` (unrotated) and ``rot_dim`` (rotated query/key columns of a head),
  ``vdim``, ``q_rank`` and ``kv_rank`` (sizes of the two latents), ``scale``, ``rot`` (``base``; ``dims`` equals
  ``rot_dim``; optionally ``scaling``).

``loop`` = {``start``, ``stop``, ``times``}: layers start .. stop - 1 run ``times`` times in a row with the same
weights before the rest follows.  Every size and constant that a model of the design may set is read from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, optional_int, required_float, required_int

_FAMILY = "silupel"
MIXER_KINDS = ("mingru", "attention", "latent_attention")


def _mapping(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError.unsupported(f"{_FAMILY} config {where} missing {key}")
    return value


def _optional_float(raw: Mapping[str, Any], key: str) -> Optional[float]:
    return None if raw.get(key) is None else required_float(raw, key, _FAMILY)


@dataclass(frozen=True)
class FrequencyScaling:
    factor: float
    low: float
    high: float
    original: float

    def to_dict(self) -> dict:
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "high": self.high, "low": self.low, "original": original}


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[FrequencyScaling] = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "Rotation":
        scaling = None
        if raw.get("scaling") is not None:
            sc = _mapping(raw, "scaling", where)
            scaling = FrequencyScaling(*(required_float(sc, key, _FAMILY) for key in ("factor", "low", "high", "original")))
            if scaling.high == scaling.low or scaling.factor <= 0.0:
                raise ConfigError.invalid(f"{_FAMILY} config {where}.scaling needs high != low and a positive factor")
        dims = required_int(raw, "dims", _FAMILY)
        if dims % 2:
            raise ConfigError.invalid(f"{_FAMILY} config {where}.dims must be even, got {dims}")
        return cls(base=required_float(raw, "base", _FAMILY), dims=dims, scaling=scaling)

    def to_dict(self) -> dict:
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_dict()
        return out


@dataclass(frozen=True)
class MinGRUMixer:
    width: int

    def to_dict(self) -> dict:
        return {"width": self.width}


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation
    softcap: Optional[float] = None
    chunk: Optional[int] = None

    def to_dict(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": self.rot.to_dict(), "scale": self.scale,
               "vdim": self.vdim}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Rotation

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "rot": self.rot.to_dict(),
                "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class DenseMLP:
    ff: int


@dataclass(frozen=True)
class SilupelLayer:
    kind: str
    mixer: object
    mlp: Optional[DenseMLP]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


def _mixer(kind: str, m: Mapping[str, Any], where: str):
    if kind == "mingru":
        return MinGRUMixer(width=required_int(m, "width", _FAMILY))
    rot = Rotation.from_dict(_mapping(m, "rot", where), where + ".rot")
    if kind == "attention":
        heads, kv_heads = required_int(m, "heads", _FAMILY), required_int(m, "kv_heads", _FAMILY)
        if heads % kv_heads:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        dim = required_int(m, "dim", _FAMILY)
        if rot.dims > dim:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: rot.dims {rot.dims} exceeds dim {dim}")
        chunk = None
        if m.get("mask") is not None:
            chunk = required_int(_mapping(m, "mask", where), "size", _FAMILY)
        softcap = _optional_float(m, "softcap")
        if softcap is not None and softcap <= 0.0:
            raise ConfigError.invalid(f"{_FAMILY} config {where}: softcap must be positive, got {softcap}")
        return AttentionMixer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=required_int(m, "vdim", _FAMILY),
                              scale=required_float(m, "scale", _FAMILY), rot=rot, softcap=softcap, chunk=chunk)
    rot_dim = required_int(m, "rot_dim", _FAMILY)
    if rot.dims != rot_dim:
        raise ConfigError.invalid(f"{_FAMILY} config {where}: rot.dims {rot.dims} must equal rot_dim {rot_dim}")
    return LatentMixer(heads=required_int(m, "heads", _FAMILY), dim=required_int(m, "dim", _FAMILY), rot_dim=rot_dim,
                       vdim=required_int(m, "vdim", _FAMILY), q_rank=required_int(m, "q_rank", _FAMILY),
                       kv_rank=required_int(m, "kv_rank", _FAMILY), scale=required_float(m, "scale", _FAMILY), rot=rot)


@dataclass(frozen=True)
class SilupelConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: Tuple[SilupelLayer, ...]
    loop: Optional[Loop] = None

    architecture = "Silupel"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def layer_runs(self) -> Tuple[int, ...]:
        """The indices of the layers in the order in which they run, a looped stretch repeated."""
        count = len(self.layers)
        if self.loop is None:
            return tuple(range(count))
        inner = list(range(self.loop.start, self.loop.stop)) * self.loop.times
        return tuple(list(range(self.loop.start)) + inner + list(range(self.loop.stop, count)))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SilupelConfig":
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
            if kind not in MIXER_KINDS:
                raise ConfigError.unsupported(f"{_FAMILY} config {where}: layer type {kind!r} is unsupported; known: {', '.join(MIXER_KINDS)}")
            mixer = _mixer(kind, _mapping(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            dense = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError.unsupported(f"{_FAMILY} config {where}: feed-forward kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is unsupported; only 'dense' is")
                dense = DenseMLP(ff=required_int(mlp, "ff", _FAMILY))
            layers.append(SilupelLayer(kind, mixer, dense))
        eps = required_float(_mapping(raw, "norm", "root"), "eps", _FAMILY)
        if eps < 0.0:
            raise ConfigError.invalid(f"{_FAMILY} config norm.eps must be non-negative")
        loop = None
        if raw.get("loop") is not None:
            lp = _mapping(raw, "loop", "root")
            loop = Loop(start=optional_int(lp, "start", _FAMILY, 0), stop=required_int(lp, "stop", _FAMILY, minimum=0),
                        times=required_int(lp, "times", _FAMILY))
            if not 0 <= loop.start <= loop.stop <= len(layers):
                raise ConfigError.invalid(f"{_FAMILY} config loop {loop.start}..{loop.stop} does not lie inside {len(layers)} layers")
        return cls(width=required_int(raw, "width", _FAMILY), vocab=required_int(raw, "vocab", _FAMILY), norm_eps=eps,
                   layers=tuple(layers), loop=loop)

    def to_dict(self) -> dict:
        """The config.json content that parses back to this configuration."""
        layers = [{"type": layer.kind, "mixer": layer.mixer.to_dict(),
                   "mlp": None if layer.mlp is None else {"kind": "dense", "ff": layer.mlp.ff}} for layer in self.layers]
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.norm_eps},
               "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out
