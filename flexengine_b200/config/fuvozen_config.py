"""Typed configuration of the Fuvozen decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``norm`` {eps, groups}, ``embedding`` {bigram {buckets, mul_prev,
mul_cur}} and ``layers``, a list whose entries give ``type`` (which mixer), ``mixer`` (its sizes and
constants) and ``mlp`` (a dense or a routed feed-forward, or null).  Every size and constant of a model comes
from this file; nothing of a particular model lives in code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .model_config import ConfigError

MIXERS = ("latent_attention", "wkv")


def _get(data: Mapping[str, Any], path: str, kind, default=None, required=True):
    node: Any = data
    for key in path.split("."):
        if not isinstance(node, Mapping) or key not in node or node[key] is None:
            if required:
                raise ConfigError(f"config.json: required key {path!r} is missing")
            return default
        node = node[key]
    if kind is int:
        if isinstance(node, bool) or not isinstance(node, int):
            raise ConfigError(f"config.json: {path!r} must be an integer, got {node!r}")
        return int(node)
    if kind is float:
        if isinstance(node, bool) or not isinstance(node, (int, float)):
            raise ConfigError(f"config.json: {path!r} must be a number, got {node!r}")
        return float(node)
    return node


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int            # unrotated query/key size of a head
    rot_dim: int        # rotated query/key size of a head (the key part is shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    window: int         # 0: every earlier key is visible
    rot_base: float
    rot_dims: int       # how many of the rotated part's entries turn; the rest pass unchanged


@dataclass(frozen=True)
class WkvConfig:
    heads: int
    dim: int


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class MoeMlpConfig:
    experts: int
    top: int
    scale: float
    expert_ff: int
    shared_ff: int      # 0: no shared expert


@dataclass(frozen=True)
class FuvozenLayer:
    type: str
    mixer: Any
    mlp: Any            # DenseMlpConfig, MoeMlpConfig or None


@dataclass(frozen=True)
class FuvozenConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: int | None = None

    ARCHITECTURE = "Fuvozen"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "FuvozenConfig":
        layers = _get(data, "layers", list)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one entry")
        parsed = []
        for i, entry in enumerate(layers):
            kind = _get(entry, "type", str)
            if kind == "latent_attention":
                rot_dim = _get(entry, "mixer.rot_dim", int)
                mixer = LatentAttentionConfig(
                    heads=_get(entry, "mixer.heads", int), dim=_get(entry, "mixer.dim", int), rot_dim=rot_dim,
                    vdim=_get(entry, "mixer.vdim", int), kv_rank=_get(entry, "mixer.kv_rank", int),
                    scale=_get(entry, "mixer.scale", float),
                    window=_get(entry, "mixer.mask.size", int, default=0, required=False),
                    rot_base=_get(entry, "mixer.rot.base", float),
                    rot_dims=_get(entry, "mixer.rot.dims", int, default=rot_dim, required=False))
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"layer {i}: rot.dims must be even and at most rot_dim")
                if min(mixer.heads, mixer.dim, mixer.vdim, mixer.kv_rank) <= 0 or mixer.rot_dim < 0 or mixer.window < 0:
                    raise ConfigError(f"layer {i}: sizes of the latent attention must be positive")
            elif kind == "wkv":
                mixer = WkvConfig(heads=_get(entry, "mixer.heads", int), dim=_get(entry, "mixer.dim", int))
                if mixer.heads <= 0 or mixer.dim <= 0:
                    raise ConfigError(f"layer {i}: sizes of the wkv mixer must be positive")
            else:
                raise ConfigError(f"layer {i}: unknown mixer type {kind!r}; known: {', '.join(MIXERS)}")
            mlp_data = entry.get("mlp")
            if mlp_data is None:
                mlp = None
            elif _get(mlp_data, "kind", str) == "dense":
                mlp = DenseMlpConfig(ff=_get(mlp_data, "ff", int))
            elif mlp_data["kind"] == "moe":
                mlp = MoeMlpConfig(experts=_get(mlp_data, "router.experts", int), top=_get(mlp_data, "router.top", int),
                                   scale=_get(mlp_data, "router.scale", float, default=1.0, required=False),
                                   expert_ff=_get(mlp_data, "expert.ff", int),
                                   shared_ff=_get(mlp_data, "shared.ff", int, default=0, required=False))
                if not (1 <= mlp.top <= mlp.experts):
                    raise ConfigError(f"layer {i}: a token uses between 1 and 'experts' experts")
            else:
                raise ConfigError(f"layer {i}: unknown mlp kind {mlp_data['kind']!r}; known: dense, moe")
            parsed.append(FuvozenLayer(kind, mixer, mlp))
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(vocab=_get(data, "vocab", int), width=_get(data, "width", int),
                  norm_eps=_get(data, "norm.eps", float), norm_groups=_get(data, "norm.groups", int, default=1, required=False),
                  bigram_buckets=_get(data, "embedding.bigram.buckets", int),
                  bigram_mul_prev=_get(data, "embedding.bigram.mul_prev", int),
                  bigram_mul_cur=_get(data, "embedding.bigram.mul_cur", int),
                  layers=tuple(parsed), eos_token_ids=eos_ids,
                  bos_token_id=None if data.get("bos_token_id") is None else int(data["bos_token_id"]))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.bigram_buckets <= 0:
            raise ConfigError("config.json: vocab, width and embedding.bigram.buckets must be positive")
        if cfg.norm_groups <= 0 or cfg.width % cfg.norm_groups:
            raise ConfigError("config.json: norm.groups must divide width")
        if not cfg.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg
