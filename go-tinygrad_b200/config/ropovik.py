"""Typed configuration of the Ropovik decoder.

Its config.json lists the layers one by one: ``layers`` is a list of objects
with ``type`` ("attention" or "mamba2"), ``mixer`` (that mixer's sizes) and
``mlp`` (``{"kind": "dense", "ff": n}`` or null for a layer without a
feed-forward).  ``loop`` (``start``, ``stop``, ``times``) makes the layers
start..stop-1 run `times` times in a row with the same weights.  Further keys:
``vocab``, ``width``, ``norm.eps`` and ``logit_softcap``.  Every size and every
constant a model of this design may choose comes from there; nothing here
names a model size.  The reference has no such architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError


def _get(block: Mapping[str, Any], key: str, where: str, kind=int, positive: bool = True):
    if not isinstance(block, Mapping) or key not in block or block[key] is None:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    v = block[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and not isinstance(v, int)):
        raise ConfigError(f"config.json: {where}.{key} must be a{'n integer' if kind is int else ' number'}, got {v!r}")
    if positive and not v > 0:
        raise ConfigError(f"config.json: {where}.{key} must be positive, got {v!r}")
    return kind(v)


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_json(self) -> dict:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: Optional[YarnScaling] = None

    def to_json(self) -> dict:
        return {"dims": self.dims, "base": self.base, "scaling": self.scaling.to_json() if self.scaling else None}


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation]

    def to_json(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, "rot": self.rot.to_json() if self.rot else None}


@dataclass(frozen=True)
class Mamba2Mixer:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_json(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "conv": self.conv, "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_json(self) -> dict:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class RopovikLayer:
    type: str                          # "attention" | "mamba2"
    mixer: Any                         # AttentionMixer | Mamba2Mixer
    mlp: Optional[DenseMlp]

    def to_json(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int

    def to_json(self) -> dict:
        return {"start": self.start, "stop": self.stop, "times": self.times}


def _read_attention(m: Mapping[str, Any], where: str) -> AttentionMixer:
    heads, kv = _get(m, "heads", where), _get(m, "kv_heads", where)
    dim = _get(m, "dim", where)
    vdim = _get(m, "vdim", where) if m.get("vdim") is not None else dim
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} query heads cannot share {kv} key/value heads")
    if vdim != dim:
        raise ConfigError(f"config.json: {where}: the values are the keys, so vdim ({vdim}) must equal dim ({dim})")
    rot = None
    if m.get("rot") is not None:
        r = m["rot"]
        dims, base = _get(r, "dims", where + ".rot"), _get(r, "base", where + ".rot", float)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        if base <= 1.0:
            raise ConfigError(f"config.json: {where}.rot.base must exceed 1, got {base}")
        scaling = None
        if r.get("scaling") is not None:
            s, w = r["scaling"], where + ".rot.scaling"
            scaling = YarnScaling(_get(s, "factor", w, float), _get(s, "original", w, float),
                                  _get(s, "fast", w, float), _get(s, "slow", w, float))
        rot = Rotation(dims, base, scaling)
    return AttentionMixer(heads, kv, dim, vdim, _get(m, "scale", where, float), rot)


def _read_mamba2(m: Mapping[str, Any], where: str) -> Mamba2Mixer:
    mixer = Mamba2Mixer(_get(m, "heads", where), _get(m, "vdim", where), _get(m, "state", where),
                        _get(m, "groups", where), _get(m, "conv", where),
                        _get(m, "norm_groups", where) if m.get("norm_groups") is not None else 1)
    if mixer.heads % mixer.groups:
        raise ConfigError(f"config.json: {where}: {mixer.heads} heads cannot share {mixer.groups} groups")
    if (mixer.heads * mixer.vdim) % mixer.norm_groups:
        raise ConfigError(f"config.json: {where}: norm_groups {mixer.norm_groups} does not divide "
                          f"heads * vdim = {mixer.heads * mixer.vdim}")
    return mixer


@dataclass(frozen=True)
class RopovikConfig:
    vocab: int
    width: int
    layers: Tuple[RopovikLayer, ...]
    loop: Optional[Loop]
    norm_eps: float
    logit_softcap: Optional[float]

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "RopovikConfig":
        vocab, width = _get(raw, "vocab", "the model"), _get(raw, "width", "the model")
        if not isinstance(raw.get("layers"), (list, tuple)) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = entry.get("type")
            if kind == "attention":
                mixer = _read_attention(entry.get("mixer"), where + ".mixer")
            elif kind == "mamba2":
                mixer = _read_mamba2(entry.get("mixer"), where + ".mixer")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not known: 'attention' or 'mamba2'")
            mlp = None
            if entry.get("mlp") is not None:
                if entry["mlp"].get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {entry['mlp'].get('kind')!r} is not known: 'dense'")
                mlp = DenseMlp(_get(entry["mlp"], "ff", where + ".mlp"))
            layers.append(RopovikLayer(kind, mixer, mlp))
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            loop = Loop(_get(lp, "start", "loop", positive=False), _get(lp, "stop", "loop", positive=False),
                        _get(lp, "times", "loop"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop {loop.start}..{loop.stop} does not lie within the "
                                  f"{len(layers)} layers")
        norm = raw.get("norm") or {}
        eps = _get(norm, "eps", "norm", float)
        cap = raw.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
            raise ConfigError(f"config.json: logit_softcap must be a positive number or null, got {cap!r}")
        return RopovikConfig(vocab, width, tuple(layers), loop, eps, float(cap) if cap else None)

    def to_json(self) -> dict:
        return {"architecture": "Ropovik", "vocab": self.vocab, "width": self.width,
                "layers": [layer.to_json() for layer in self.layers],
                "loop": self.loop.to_json() if self.loop else None,
                "norm": {"eps": self.norm_eps}, "logit_softcap": self.logit_softcap}
