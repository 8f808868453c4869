"""Typed configuration of the Senupel decoder.

Its config.json lists the layers one by one: ``layers`` is a list of objects
with ``type`` ("latent_attention"), ``mixer`` (the mixer's sizes: ``heads``,
``dim`` unrotated and ``rot_dim`` rotated query/key channels per head,
``vdim``, ``kv_rank``, ``scale``, ``mask.size`` the causal window, ``rot``
with ``dims``, ``base`` and optionally ``scaling``; ``kv_from``: j for a layer
that has no down projection and reads layer j's latents) and ``mlp``
(``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n},
"router": {"experts": E, "top": k}}`` or null).  Further keys: ``vocab``,
``width``, ``norm.eps``.  Every size and every constant a model of this design
may choose comes from there; nothing here names a model size.  The reference
has no such architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .llama import ConfigError
from .ropovik import Rotation, YarnScaling, _get


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot: Rotation
    kv_from: Optional[int] = None

    def to_json(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
               "kv_rank": self.kv_rank, "scale": self.scale,
               "rot": {"dims": self.rot.dims, "base": self.rot.base}}
        if self.rot.scaling is not None:
            out["rot"]["scaling"] = self.rot.scaling.to_json()
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_json(self) -> dict:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class ExpertMlp:
    ff: int
    experts: int
    top: int

    def to_json(self) -> dict:
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class SenupelLayer:
    type: str
    mixer: LatentMixer
    mlp: Union[DenseMlp, ExpertMlp, None]

    def to_json(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


def _read_mixer(m: Mapping[str, Any], where: str, index: int) -> LatentMixer:
    heads, dim, rot_dim = _get(m, "heads", where), _get(m, "dim", where), _get(m, "rot_dim", where)
    vdim, rank = _get(m, "vdim", where), _get(m, "kv_rank", where)
    scale = _get(m, "scale", where, float)
    if rot_dim % 2:
        raise ConfigError(f"config.json: {where}.rot_dim must be even, got {rot_dim}")
    r = m.get("rot")
    dims, base = _get(r, "dims", where + ".rot"), _get(r, "base", where + ".rot", float)
    if dims % 2 or dims > rot_dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most rot_dim ({rot_dim}), got {dims}")
    if base <= 1.0:
        raise ConfigError(f"config.json: {where}.rot.base must exceed 1, got {base}")
    scaling = None
    if r.get("scaling") is not None:
        s, w = r["scaling"], where + ".rot.scaling"
        scaling = YarnScaling(_get(s, "factor", w, float), _get(s, "original", w, float),
                              _get(s, "fast", w, float), _get(s, "slow", w, float))
    window = None
    if m.get("mask") is not None:
        window = _get(m["mask"], "size", where + ".mask")
    kv_from = m.get("kv_from")
    if kv_from is not None:
        if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < index:
            raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer, got {kv_from!r}")
    return LatentMixer(heads, dim, rot_dim, vdim, rank, scale, window, Rotation(dims, base, scaling), kv_from)


def _read_mlp(mlp: Any, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping):
        raise ConfigError(f"config.json: {where} must be an object or null")
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return DenseMlp(_get(mlp, "ff", where))
    if kind == "moe":
        router = mlp.get("router")
        out = ExpertMlp(_get(mlp.get("expert"), "ff", where + ".expert"), _get(router, "experts", where + ".router"),
                        _get(router, "top", where + ".router"))
        if out.top > out.experts:
            raise ConfigError(f"config.json: {where}.router: a token cannot use {out.top} of {out.experts} experts")
        return out
    raise ConfigError(f"config.json: {where}.kind {kind!r} is not known: 'dense' or 'moe'")


@dataclass(frozen=True)
class SenupelConfig:
    vocab: int
    width: int
    layers: Tuple[SenupelLayer, ...]
    norm_eps: float

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "SenupelConfig":
        vocab, width = _get(raw, "vocab", "the model"), _get(raw, "width", "the model")
        if not isinstance(raw.get("layers"), (list, tuple)) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = entry.get("type")
            if kind != "latent_attention":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not known: 'latent_attention'")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} lacks 'mixer'")
            mixer = _read_mixer(entry["mixer"], where + ".mixer", i)
            if mixer.kv_from is not None:
                src = layers[mixer.kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"config.json: {where}.mixer.kv_from names layer {mixer.kv_from}, which has no "
                                      f"down projection of its own")
                if (src.kv_rank, src.rot_dim, src.rot) != (mixer.kv_rank, mixer.rot_dim, mixer.rot):
                    raise ConfigError(f"config.json: {where}.mixer reads layer {mixer.kv_from}'s latents, so kv_rank, "
                                      f"rot_dim and rot must equal that layer's")
            layers.append(SenupelLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + ".mlp")))
        eps = _get(raw.get("norm") or {}, "eps", "norm", float)
        return SenupelConfig(vocab, width, tuple(layers), eps)

    def to_json(self) -> dict:
        return {"architecture": "Senupel", "vocab": self.vocab, "width": self.width,
                "layers": [layer.to_json() for layer in self.layers], "norm": {"eps": self.norm_eps}}
