"""Typed configuration of the Fuvuvik decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``streams`` (copies of the residual), ``norm`` {eps}, ``embedding`` {scale}
and ``layers``, a list whose entries give ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (a
dense gated feed-forward, or null).  Every size and constant of a model comes from this file; what the design fixes
for a mixer type (which of them has convolutions, unit-normed queries and keys, chunks, a sink) is fixed here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .fuvozen_config import _get
from .model_config import ConfigError

MIXERS = ("attention", "attention_2", "mingru")
MAX_STREAMS = 16            # what the kernels of the residual streams keep in registers


@dataclass(frozen=True)
class GatedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int            # query/key size of a head
    vdim: int           # value size of a head
    scale: float
    rot_base: float
    rot_dims: int       # how many of a head's first entries turn (pairs i, i + rot_dims/2); the rest pass unchanged
    conv: int           # taps of the causal convolution over time after the q, k and v projections; 0: none
    qk_norm: bool       # queries and keys divided by their root mean square over the head, after the rotation
    mask: str           # "full": every earlier key; "chunk": only keys of the query's own chunk of ``mask_size`` positions
    mask_size: int
    sink: bool          # one added to the softmax's denominator


@dataclass(frozen=True)
class MinGruConfig:
    width: int


@dataclass(frozen=True)
class GatedMlpConfig:
    ff: int


@dataclass(frozen=True)
class FuvuvikLayer:
    type: str
    mixer: Any
    mlp: Any            # GatedMlpConfig or None


@dataclass(frozen=True)
class FuvuvikConfig:
    vocab: int
    width: int
    streams: int
    norm_eps: float
    embedding_scale: float
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: int | None = None

    ARCHITECTURE = "Fuvuvik"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "FuvuvikConfig":
        layers = _get(data, "layers", list)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one entry")
        parsed = []
        for i, entry in enumerate(layers):
            kind = _get(entry, "type", str)
            if kind in ("attention", "attention_2"):
                chunked = kind == "attention_2"
                dim = _get(entry, "mixer.dim", int)
                mixer = GatedAttentionConfig(
                    heads=_get(entry, "mixer.heads", int), kv_heads=_get(entry, "mixer.kv_heads", int), dim=dim,
                    vdim=_get(entry, "mixer.vdim", int), scale=_get(entry, "mixer.scale", float),
                    rot_base=_get(entry, "mixer.rot.base", float), rot_dims=_get(entry, "mixer.rot.dims", int),
                    conv=0 if chunked else _get(entry, "mixer.conv", int, default=0, required=False), qk_norm=not chunked,
                    mask="chunk" if chunked else "full", mask_size=_get(entry, "mixer.mask.size", int) if chunked else 0,
                    sink=chunked)
                if min(mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim) <= 0 or mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"layer {i}: head counts and sizes must be positive, heads a multiple of kv_heads")
                if mixer.rot_dims < 0 or mixer.rot_dims % 2 or mixer.rot_dims > dim:
                    raise ConfigError(f"layer {i}: rot.dims must be even and at most dim")
                if mixer.conv < 0 or (chunked and mixer.mask_size <= 0):
                    raise ConfigError(f"layer {i}: conv must not be negative and mask.size must be positive")
            elif kind == "mingru":
                mixer = MinGruConfig(width=_get(entry, "mixer.width", int))
                if mixer.width <= 0:
                    raise ConfigError(f"layer {i}: the width of the recurrence must be positive")
            else:
                raise ConfigError(f"layer {i}: unknown mixer type {kind!r}; known: {', '.join(MIXERS)}")
            mlp_data = entry.get("mlp")
            if mlp_data is None:
                mlp = None
            elif _get(mlp_data, "kind", str) == "dense":
                mlp = GatedMlpConfig(ff=_get(mlp_data, "ff", int))
                if mlp.ff <= 0:
                    raise ConfigError(f"layer {i}: mlp.ff must be positive")
            else:
                raise ConfigError(f"layer {i}: unknown mlp kind {mlp_data['kind']!r}; known: dense")
            parsed.append(FuvuvikLayer(kind, mixer, mlp))
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(vocab=_get(data, "vocab", int), width=_get(data, "width", int),
                  streams=_get(data, "streams", int, default=1, required=False),
                  norm_eps=_get(data, "norm.eps", float),
                  embedding_scale=_get(data, "embedding.scale", float, default=1.0, required=False),
                  layers=tuple(parsed), eos_token_ids=eos_ids,
                  bos_token_id=None if data.get("bos_token_id") is None else int(data["bos_token_id"]))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        if not 1 <= cfg.streams <= MAX_STREAMS:
            raise ConfigError(f"config.json: streams must be between 1 and {MAX_STREAMS}")
        if not cfg.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg
