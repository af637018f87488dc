"""Typed configuration of the Fedutar decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``norm`` {eps}, ``embedding`` {scale}, ``logit_scale``, ``logit_softcap``,
``loop`` {start, stop, times} (layers start .. stop - 1 run ``times`` times in a row; absent: every layer once) and
``layers``, a list whose entries give ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (a dense or
a routed feed-forward, or null).  Every size and constant of a model comes from this file.  The one mixer type,
``parallel``, is two mixers side by side: ``left`` (softmax attention) and ``right`` (retention), with a scale each.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .fuvozen_config import _get
from .model_config import ConfigError

MIXERS = ("parallel",)


@dataclass(frozen=True)
class SoftmaxSideConfig:
    heads: int
    kv_heads: int
    dim: int             # query/key size of a head
    vdim: int            # value size of a head
    scale: float         # what the scores are multiplied by
    temp_coef: float     # queries at position p are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1); 0: by 1
    temp_every: int


@dataclass(frozen=True)
class RetentionSideConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple         # one number per head
    rot_base: float
    rot_dims: int        # how many of a head's first entries turn (pairs i, i + rot_dims/2); 0: none


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SoftmaxSideConfig
    right: RetentionSideConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class MoeMlpConfig:
    experts: int
    top: int
    expert_ff: int
    limit: float         # the gate product is cut off above it, the up product on both sides


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class FedutarLayer:
    type: str
    mixer: Any
    mlp: Any             # DenseMlpConfig, MoeMlpConfig or None


@dataclass(frozen=True)
class FedutarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float     # 0: logits are not squashed
    loop: LoopConfig | None
    layers: tuple
    eos_token_ids: tuple = ()
    bos_token_id: int | None = None

    ARCHITECTURE = "Fedutar"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "FedutarConfig":
        layers = _get(data, "layers", list)
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one entry")
        parsed = []
        for i, entry in enumerate(layers):
            kind = _get(entry, "type", str)
            if kind != "parallel":
                raise ConfigError(f"layer {i}: unknown mixer type {kind!r}; known: {', '.join(MIXERS)}")
            heads = _get(entry, "mixer.left.heads", int)
            left = SoftmaxSideConfig(
                heads=heads, kv_heads=_get(entry, "mixer.left.kv_heads", int, default=heads, required=False),
                dim=_get(entry, "mixer.left.dim", int), vdim=_get(entry, "mixer.left.vdim", int),
                scale=_get(entry, "mixer.left.scale", float),
                temp_coef=_get(entry, "mixer.left.q_temp.coef", float, default=0.0, required=False),
                temp_every=_get(entry, "mixer.left.q_temp.every", int, default=1, required=False))
            if min(left.heads, left.kv_heads, left.dim, left.vdim) <= 0 or left.heads % left.kv_heads:
                raise ConfigError(f"layer {i}: the left mixer's head counts and sizes must be positive, heads a multiple of kv_heads")
            if left.temp_every <= 0:
                raise ConfigError(f"layer {i}: q_temp.every must be positive")
            decay = _get(entry, "mixer.right.decay", list)
            right = RetentionSideConfig(
                heads=_get(entry, "mixer.right.heads", int), dim=_get(entry, "mixer.right.dim", int),
                vdim=_get(entry, "mixer.right.vdim", int), decay=tuple(float(x) for x in decay),
                rot_base=_get(entry, "mixer.right.rot.base", float, default=10000.0, required=False),
                rot_dims=_get(entry, "mixer.right.rot.dims", int, default=0, required=False))
            if min(right.heads, right.dim, right.vdim) <= 0:
                raise ConfigError(f"layer {i}: the right mixer's head count and sizes must be positive")
            if len(right.decay) != right.heads:
                raise ConfigError(f"layer {i}: 'decay' must list one number per head of the right mixer")
            if right.rot_dims < 0 or right.rot_dims % 2 or right.rot_dims > right.dim:
                raise ConfigError(f"layer {i}: rot.dims must be even and at most dim")
            mixer = ParallelMixerConfig(left, right, left_scale=_get(entry, "mixer.left_scale", float, default=1.0, required=False),
                                        right_scale=_get(entry, "mixer.right_scale", float, default=1.0, required=False))
            mlp_data = entry.get("mlp")
            if mlp_data is None:
                mlp = None
            elif _get(mlp_data, "kind", str) == "dense":
                mlp = DenseMlpConfig(ff=_get(mlp_data, "ff", int))
                if mlp.ff <= 0:
                    raise ConfigError(f"layer {i}: mlp.ff must be positive")
            elif mlp_data["kind"] == "moe":
                mlp = MoeMlpConfig(experts=_get(mlp_data, "router.experts", int), top=_get(mlp_data, "router.top", int),
                                   expert_ff=_get(mlp_data, "expert.ff", int), limit=_get(mlp_data, "expert.limit", float))
                if not (1 <= mlp.top <= mlp.experts) or mlp.expert_ff <= 0:
                    raise ConfigError(f"layer {i}: a token uses between 1 and 'experts' experts of a positive size")
                if not mlp.limit > 0.0:
                    raise ConfigError(f"layer {i}: expert.limit must be positive")
            else:
                raise ConfigError(f"layer {i}: unknown mlp kind {mlp_data['kind']!r}; known: dense, moe")
            parsed.append(FedutarLayer(kind, mixer, mlp))
        loop = None
        if data.get("loop") is not None:
            loop = LoopConfig(start=_get(data, "loop.start", int), stop=_get(data, "loop.stop", int), times=_get(data, "loop.times", int))
            if not (0 <= loop.start < loop.stop <= len(parsed)) or loop.times < 1:
                raise ConfigError("config.json: 'loop' must name a span of layers, start < stop, and run it at least once")
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(vocab=_get(data, "vocab", int), width=_get(data, "width", int), norm_eps=_get(data, "norm.eps", float),
                  embedding_scale=_get(data, "embedding.scale", float, default=1.0, required=False),
                  logit_scale=_get(data, "logit_scale", float, default=1.0, required=False),
                  logit_softcap=_get(data, "logit_softcap", float, default=0.0, required=False),
                  loop=loop, layers=tuple(parsed), eos_token_ids=eos_ids,
                  bos_token_id=None if data.get("bos_token_id") is None else int(data["bos_token_id"]))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        if not cfg.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")
        if cfg.logit_softcap < 0.0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        return cfg
