"""Typed configuration of the Megerax decoder.

Its config.json lists the layers one by one: ``layers`` is a list of objects
with ``type``, ``mixer`` (that mixer's sizes) and ``mlp`` (``{"kind": "dense",
"ff": n}`` or null for a layer without a feed-forward).  The mixers:

* ``attention``: ``heads``, ``kv_heads``, ``dim`` (channels of a query or key
  head), ``vdim`` (of a value head), ``scale``, and optionally ``conv`` (taps of
  the causal convolution over q, k and v), ``rot`` (``dims``, ``base`` and
  optionally ``scaling`` with ``factor``, ``low``, ``high``, ``original``),
  ``softcap``, ``mask.size`` (the sliding window) and ``kv_from``: j for a layer
  that has no key and value projections and reads layer j's cache;
* ``latent_attention``: ``heads``, ``dim`` unrotated and ``rot_dim`` rotated
  query/key channels per head, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``,
  ``rot`` (``dims``, ``base``) and optionally ``mask.size``;
* ``channel_delta``: ``heads``, ``kv_heads``, ``dim``, ``vdim`` and optionally
  ``conv``; the widths of its two low-rank projections are those of its tensors
  unless ``decay_rank`` and ``gate_rank`` name them.

Further keys: ``vocab``, ``width``, ``norm.eps`` and ``logit_scale``.  Every size
and every constant a model of this design may choose comes from there; nothing
here names a model size.  The reference has no such architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError
from .ropovik import DenseMlp, _get

MIXER_TYPES = ("attention", "latent_attention", "channel_delta")


@dataclass(frozen=True)
class WavelengthScaling:
    factor: float
    low: float
    high: float
    original: float

    def to_json(self) -> dict:
        return {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}


@dataclass(frozen=True)
class ScaledRotation:
    dims: int
    base: float
    scaling: Optional[WavelengthScaling] = None

    def to_json(self) -> dict:
        out = {"dims": self.dims, "base": self.base}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_json()
        return out


@dataclass(frozen=True)
class ConvAttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: Optional[int]
    rot: Optional[ScaledRotation]
    softcap: Optional[float]
    window: Optional[int]
    kv_from: Optional[int] = None

    def to_json(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.conv is not None:
            out["conv"] = self.conv
        if self.rot is not None:
            out["rot"] = self.rot.to_json()
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class SinkLatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: ScaledRotation
    window: Optional[int]

    def to_json(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
               "q_rank": self.q_rank, "scale": self.scale, "rot": self.rot.to_json()}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: Optional[int]
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None

    def to_json(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim}
        if self.conv is not None:
            out["conv"] = self.conv
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            out["gate_rank"] = self.gate_rank
        return out


@dataclass(frozen=True)
class MegeraxLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseMlp]

    def to_json(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


def _optional(m: Mapping[str, Any], key: str, where: str, kind=int):
    return _get(m, key, where, kind) if m.get(key) is not None else None


def _read_rotation(r: Any, where: str, most: int) -> Optional[ScaledRotation]:
    if r is None:
        return None
    dims, base = _get(r, "dims", where), _get(r, "base", where, float)
    if dims % 2 or dims > most:
        raise ConfigError(f"config.json: {where}.dims must be even and at most {most}, got {dims}")
    if base <= 1.0:
        raise ConfigError(f"config.json: {where}.base must exceed 1, got {base}")
    scaling = None
    if r.get("scaling") is not None:
        s, w = r["scaling"], where + ".scaling"
        scaling = WavelengthScaling(_get(s, "factor", w, float), _get(s, "low", w, float), _get(s, "high", w, float),
                                    _get(s, "original", w, float))
        if scaling.high <= scaling.low:
            raise ConfigError(f"config.json: {w}.high must exceed low, got {scaling.high} and {scaling.low}")
    return ScaledRotation(dims, base, scaling)


def _window(m: Mapping[str, Any], where: str) -> Optional[int]:
    return _get(m["mask"], "size", where + ".mask") if m.get("mask") is not None else None


def _heads(m: Mapping[str, Any], where: str) -> Tuple[int, int]:
    heads, kv = _get(m, "heads", where), _get(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads cannot share {kv} key/value heads")
    return heads, kv


def _read_attention(m: Mapping[str, Any], where: str, index: int) -> ConvAttentionMixer:
    heads, kv = _heads(m, where)
    dim, vdim = _get(m, "dim", where), _get(m, "vdim", where)
    cap = _optional(m, "softcap", where, float)
    kv_from = m.get("kv_from")
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < index):
        raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer, got {kv_from!r}")
    return ConvAttentionMixer(heads, kv, dim, vdim, _get(m, "scale", where, float), _optional(m, "conv", where),
                              _read_rotation(m.get("rot"), where + ".rot", dim), cap, _window(m, where), kv_from)


def _read_latent(m: Mapping[str, Any], where: str) -> SinkLatentMixer:
    rot_dim = _get(m, "rot_dim", where)
    if rot_dim % 2:
        raise ConfigError(f"config.json: {where}.rot_dim must be even, got {rot_dim}")
    rot = _read_rotation(m.get("rot"), where + ".rot", rot_dim)
    if rot is None:
        raise ConfigError(f"config.json: {where} lacks 'rot'")
    return SinkLatentMixer(_get(m, "heads", where), _get(m, "dim", where), rot_dim, _get(m, "vdim", where),
                           _get(m, "kv_rank", where), _get(m, "q_rank", where), _get(m, "scale", where, float), rot,
                           _window(m, where))


def _read_delta(m: Mapping[str, Any], where: str) -> DeltaMixer:
    heads, kv = _heads(m, where)
    return DeltaMixer(heads, kv, _get(m, "dim", where), _get(m, "vdim", where), _optional(m, "conv", where),
                      _optional(m, "decay_rank", where), _optional(m, "gate_rank", where))


@dataclass(frozen=True)
class MegeraxConfig:
    vocab: int
    width: int
    layers: Tuple[MegeraxLayer, ...]
    norm_eps: float
    logit_scale: float

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "MegeraxConfig":
        vocab, width = _get(raw, "vocab", "the model"), _get(raw, "width", "the model")
        if not isinstance(raw.get("layers"), (list, tuple)) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not known: {', '.join(map(repr, MIXER_TYPES))}")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} lacks 'mixer'")
            m, w = entry["mixer"], where + ".mixer"
            if kind == "attention":
                mixer = _read_attention(m, w, i)
                if mixer.kv_from is not None:
                    src = layers[mixer.kv_from]
                    if src.type != "attention" or src.mixer.kv_from is not None:
                        raise ConfigError(f"config.json: {w}.kv_from names layer {mixer.kv_from}, which has no keys and "
                                          f"values of its own for this layer to read")
                    s = src.mixer
                    if (s.kv_heads, s.dim, s.vdim, s.rot) != (mixer.kv_heads, mixer.dim, mixer.vdim, mixer.rot):
                        raise ConfigError(f"config.json: {w} reads layer {mixer.kv_from}'s keys and values, so kv_heads, "
                                          f"dim, vdim and rot must equal that layer's")
            elif kind == "latent_attention":
                mixer = _read_latent(m, w)
            else:
                mixer = _read_delta(m, w)
            mlp = None
            if entry.get("mlp") is not None:
                if not isinstance(entry["mlp"], Mapping) or entry["mlp"].get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind is not known: 'dense'")
                mlp = DenseMlp(_get(entry["mlp"], "ff", where + ".mlp"))
            layers.append(MegeraxLayer(kind, mixer, mlp))
        eps = _get(raw.get("norm") or {}, "eps", "norm", float)
        scale = _get(raw, "logit_scale", "the model", float) if raw.get("logit_scale") is not None else 1.0
        return MegeraxConfig(vocab, width, tuple(layers), eps, scale)

    def to_json(self) -> dict:
        return {"architecture": "Megerax", "vocab": self.vocab, "width": self.width,
                "layers": [layer.to_json() for layer in self.layers], "norm": {"eps": self.norm_eps},
                "logit_scale": self.logit_scale}
