"""Typed configuration of the Rikolix decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``norm`` {eps}, ``embedding`` {scale} and ``layers``, a list whose entries give
``type`` (which mixer: ``attention`` or ``latent_attention``), ``mixer`` (its sizes and constants) and ``mlp`` (a dense or a
routed feed-forward, or null).  Every size and constant of a model comes from this file; what the design fixes (how the
norms read their weights, which entries are paired in a rotation, the activation) is fixed in the plan.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .fuvozen_config import _get
from .model_config import ConfigError

MIXERS = ("attention", "latent_attention")


@dataclass(frozen=True)
class SigmoidAttentionConfig:
    heads: int
    kv_heads: int
    dim: int             # query/key size of a head
    vdim: int            # value size of a head; all of it turns with the position
    scale: float         # what the scores are multiplied by
    rot_base: float
    rot_dims: int        # how many of a query or key head's first entries turn; 0: none


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int             # unrotated query/key size of a head
    rot_dim: int         # rotated query/key size of a head (the key part is shared by the heads)
    vdim: int
    kv_rank: int
    q_rank: int          # the queries' latent
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: int | None  # the layer whose cached latents this layer reads instead of making its own


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class MoeMlpConfig:
    experts: int         # experts with matrices of their own
    identity: int        # further router outputs that stand for experts which return their input
    top: int
    expert_ff: int
    groups: int          # the router's outputs form this many equal groups of neighbours ...
    keep: int            # ... of which the best ``keep`` can be chosen from


@dataclass(frozen=True)
class RikolixLayer:
    type: str
    mixer: Any
    mlp: Any             # DenseMlpConfig, MoeMlpConfig or None


@dataclass(frozen=True)
class RikolixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: int | None = None

    ARCHITECTURE = "Rikolix"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RikolixConfig":
        layers = _get(data, "layers", list)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one entry")
        parsed = []
        for i, entry in enumerate(layers):
            kind = _get(entry, "type", str)
            if kind == "attention":
                heads = _get(entry, "mixer.heads", int)
                mixer = SigmoidAttentionConfig(
                    heads=heads, kv_heads=_get(entry, "mixer.kv_heads", int, default=heads, required=False),
                    dim=_get(entry, "mixer.dim", int), vdim=_get(entry, "mixer.vdim", int), scale=_get(entry, "mixer.scale", float),
                    rot_base=_get(entry, "mixer.rot.base", float, default=10000.0, required=False),
                    rot_dims=_get(entry, "mixer.rot.dims", int, default=0, required=False))
                if min(mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim) <= 0 or mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"layer {i}: head counts and sizes must be positive, heads a multiple of kv_heads")
                if mixer.rot_dims < 0 or mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                    raise ConfigError(f"layer {i}: rot.dims must be even and at most dim")
                if mixer.vdim % 2:
                    raise ConfigError(f"layer {i}: vdim must be even (the values turn in pairs)")
            elif kind == "latent_attention":
                rot_dim = _get(entry, "mixer.rot_dim", int)
                source = entry["mixer"].get("kv_from")
                mixer = LatentMixerConfig(
                    heads=_get(entry, "mixer.heads", int), dim=_get(entry, "mixer.dim", int), rot_dim=rot_dim,
                    vdim=_get(entry, "mixer.vdim", int), kv_rank=_get(entry, "mixer.kv_rank", int),
                    q_rank=_get(entry, "mixer.q_rank", int), scale=_get(entry, "mixer.scale", float),
                    rot_base=_get(entry, "mixer.rot.base", float, default=10000.0, required=False),
                    rot_dims=_get(entry, "mixer.rot.dims", int, default=rot_dim, required=False),
                    kv_from=None if source is None else _get(entry, "mixer.kv_from", int))
                if min(mixer.heads, mixer.dim, mixer.vdim, mixer.kv_rank, mixer.q_rank) <= 0 or mixer.rot_dim < 0:
                    raise ConfigError(f"layer {i}: head count, sizes and ranks must be positive")
                if mixer.rot_dims < 0 or mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"layer {i}: rot.dims must be even and at most rot_dim")
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    origin = parsed[j].mixer if 0 <= j < i else None
                    if not isinstance(origin, LatentMixerConfig) or origin.kv_from is not None:
                        raise ConfigError(f"layer {i}: kv_from must name an earlier latent_attention layer that makes its own latents")
                    # the cached rows are the maker's: their layout has to fit; the reader's queries turn by its own rotation
                    if (origin.kv_rank, origin.rot_dim) != (mixer.kv_rank, mixer.rot_dim):
                        raise ConfigError(f"layer {i}: kv_rank and rot_dim must equal those of layer {j}, whose latents it reads")
            else:
                raise ConfigError(f"layer {i}: unknown mixer type {kind!r}; known: {', '.join(MIXERS)}")
            mlp_data = entry.get("mlp")
            if mlp_data is None:
                mlp = None
            elif _get(mlp_data, "kind", str) == "dense":
                mlp = DenseMlpConfig(ff=_get(mlp_data, "ff", int))
                if mlp.ff <= 0:
                    raise ConfigError(f"layer {i}: mlp.ff must be positive")
            elif mlp_data["kind"] == "moe":
                mlp = MoeMlpConfig(experts=_get(mlp_data, "router.experts", int),
                                   identity=_get(mlp_data, "router.identity", int, default=0, required=False),
                                   top=_get(mlp_data, "router.top", int), expert_ff=_get(mlp_data, "expert.ff", int),
                                   groups=_get(mlp_data, "router.groups.count", int, default=1, required=False),
                                   keep=_get(mlp_data, "router.groups.keep", int, default=1, required=False))
                outputs = mlp.experts + mlp.identity
                if mlp.experts < 1 or mlp.identity < 0 or mlp.expert_ff <= 0:
                    raise ConfigError(f"layer {i}: the router needs at least one expert of a positive size, and identity >= 0")
                if mlp.groups < 1 or outputs % mlp.groups or not (1 <= mlp.keep <= mlp.groups):
                    raise ConfigError(f"layer {i}: router.groups.count must divide experts + identity, keep lie between 1 and count")
                if not (1 <= mlp.top <= mlp.keep * (outputs // mlp.groups)):
                    raise ConfigError(f"layer {i}: a token uses between 1 and keep x (group size) experts")
            else:
                raise ConfigError(f"layer {i}: unknown mlp kind {mlp_data['kind']!r}; known: dense, moe")
            parsed.append(RikolixLayer(kind, mixer, mlp))
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(vocab=_get(data, "vocab", int), width=_get(data, "width", int), norm_eps=_get(data, "norm.eps", float),
                  embedding_scale=_get(data, "embedding.scale", float, default=1.0, required=False),
                  layers=tuple(parsed), eos_token_ids=eos_ids,
                  bos_token_id=None if data.get("bos_token_id") is None else int(data["bos_token_id"]))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        if not cfg.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg
