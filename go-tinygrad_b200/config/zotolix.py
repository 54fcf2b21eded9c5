"""Typed configuration of the Zotolix decoder.

Its config.json lists the layers one by one: ``layers`` is a list of objects
with ``type`` ("attention": queries and keys divided by their root mean square
after the rotation; "attention_2": a sigmoid gate per head on the attention's
output), ``mixer`` (``heads``, ``kv_heads``, ``dim`` channels of a query or key
head, ``vdim`` of a value head, ``scale``, ``rot`` with ``dims`` and ``base``,
``mask.size``: keys are seen within stretches of so many positions, ``v_mix``:
the layer's values are blended with those of the first such layer) and ``mlp``
(``{"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k}}``
or null).  Further keys: ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``residual_mult`` (what a sublayer's output is multiplied
by before it joins the hidden state) and ``streams`` (how many copies of the
hidden state the hyper-connections keep; absent: the ordinary residual sum).
Every size and every constant a model of this design may choose comes from
there; nothing here names a model size.  The reference has no such
architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError
from .ropovik import Rotation, _get
from .senupel import ExpertMlp, _read_mlp

MIXER_TYPES = ("attention", "attention_2")
MAX_STREAMS = 8


@dataclass(frozen=True)
class ChunkedMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotation]
    chunk: Optional[int]
    v_mix: bool

    def to_json(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
               "scale": self.scale, "v_mix": self.v_mix}
        if self.rot is not None:
            out["rot"] = {"dims": self.rot.dims, "base": self.rot.base}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class ZotolixLayer:
    type: str
    mixer: ChunkedMixer
    mlp: Optional[ExpertMlp]

    def to_json(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


def _read_mixer(m: Mapping[str, Any], where: str) -> ChunkedMixer:
    heads, kv_heads = _get(m, "heads", where), _get(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: {heads} query heads cannot share {kv_heads} key/value heads")
    dim, vdim = _get(m, "dim", where), _get(m, "vdim", where)
    scale = _get(m, "scale", where, float)
    rot = None
    if m.get("rot") is not None:
        r = m["rot"]
        dims, base = _get(r, "dims", where + ".rot"), _get(r, "base", where + ".rot", float)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        if base <= 1.0:
            raise ConfigError(f"config.json: {where}.rot.base must exceed 1, got {base}")
        rot = Rotation(dims, base)
    chunk = None
    if m.get("mask") is not None:
        chunk = _get(m["mask"], "size", where + ".mask")
    v_mix = m.get("v_mix", False)
    if not isinstance(v_mix, bool):
        raise ConfigError(f"config.json: {where}.v_mix must be true or false, got {v_mix!r}")
    return ChunkedMixer(heads, kv_heads, dim, vdim, scale, rot, chunk, v_mix)


@dataclass(frozen=True)
class ZotolixConfig:
    vocab: int
    width: int
    layers: Tuple[ZotolixLayer, ...]
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    streams: Optional[int]

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "ZotolixConfig":
        vocab, width = _get(raw, "vocab", "the model"), _get(raw, "width", "the model")
        if not isinstance(raw.get("layers"), (list, tuple)) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        first_blend = None
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not known: {' or '.join(map(repr, MIXER_TYPES))}")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} lacks 'mixer'")
            mixer = _read_mixer(entry["mixer"], where + ".mixer")
            if mixer.v_mix:
                if first_blend is None:
                    first_blend = mixer
                elif (first_blend.kv_heads, first_blend.vdim) != (mixer.kv_heads, mixer.vdim):
                    raise ConfigError(f"config.json: {where}.mixer blends its values with those of the first layer that "
                                      f"does, so kv_heads and vdim must equal that layer's")
            mlp = _read_mlp(entry.get("mlp"), where + ".mlp")
            if mlp is not None and not isinstance(mlp, ExpertMlp):
                raise ConfigError(f"config.json: {where}.mlp.kind must be 'moe'")
            layers.append(ZotolixLayer(kind, mixer, mlp))
        eps = _get(raw.get("norm") or {}, "eps", "norm", float)
        scale = 1.0
        if raw.get("embedding") is not None:
            scale = _get(raw["embedding"], "scale", "embedding", float)
        mult = 1.0
        if raw.get("residual_mult") is not None:
            mult = _get(raw, "residual_mult", "the model", float)
        streams = None
        if raw.get("streams") is not None:
            streams = _get(raw, "streams", "the model")
            if streams > MAX_STREAMS:
                raise ConfigError(f"config.json: streams must be at most {MAX_STREAMS}, got {streams}")
        return ZotolixConfig(vocab, width, tuple(layers), eps, scale, mult, streams)

    def to_json(self) -> dict:
        out = {"architecture": "Zotolix", "vocab": self.vocab, "width": self.width,
               "layers": [layer.to_json() for layer in self.layers], "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult}
        if self.streams is not None:
            out["streams"] = self.streams
        return out
