"""Rikolix as a plan of parts: a decoder whose layers have a norm before and after each sublayer (weights stored around
zero, used as 1 + w), a mixer that is either grouped-query attention with sigmoid weights (one RMS norm over the whole
query projection and one over the whole key projection, neighbouring entries rotated in pairs, values that turn with
their position and outputs that are turned back) or softmax attention over a cached latent (queries through a latent of
their own; a layer may read the latents of an earlier layer instead of making some), and a feed-forward that is dense
(squared relu) or routed (softmax router with a correction for the choice, groups of experts, experts that return their
input).

Checkpoint names: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.q|k|v|o|q.norm|k.norm|pb`` or ``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|o``, ``l<i>.mlp.up|down`` or
``l<i>.mlp.e<k>.up|down``, ``l<i>.mlp.router`` and ``l<i>.mlp.correction``.  Matrices are [out, in].  q, k and v are bound
as one matrix, all experts of a layer as one.

Cache groups: a paged group per distinct (key/value heads, head size) of the attention layers (head size: the larger of
the query/key and the value size, in steps of 16; the smaller is padded with zeros), and a paged group of one plane per
distinct row width of the latent layers (latent | rotated key part, padded to a multiple of 16).  A layer that reads
another layer's latents has that layer's group and slot and writes nothing.
"""
from __future__ import annotations

import math
from dataclasses import replace

from ..config.registry import register_architecture
from ..config.rikolix_config import DenseMlpConfig, LatentMixerConfig, MoeMlpConfig, RikolixConfig, SigmoidAttentionConfig
from ..parts.spec import (CacheGroupSpec, LayerSpec, ModelPlan, PartSpec, RunEntry, WeightBinding, WeightSource)


def build_rikolix_plan(cfg: RikolixConfig, present=None) -> ModelPlan:
    """``present``: the tensor names of a checkpoint; the second pair of norms of a layer without a feed-forward is then
    named as ignored where the checkpoint has it."""
    D, V = cfg.width, cfg.vocab
    norm = PartSpec("rmsnorm", {"hidden_size": D, "eps": cfg.norm_eps, "unit_offset": True})
    groups: list = []
    group_of: dict = {}            # key -> [group index, slots so far]
    place_of: dict = {}            # layer -> (group, slot) of the latents it wrote
    layers, bindings, ignored, run = [], [], [], []
    init = {}

    def src(name, *shape, rule=None):
        fan_in = shape[-1] if len(shape) > 1 else 1
        init[name] = rule or ("normal", 0.0, 1.0 / math.sqrt(max(fan_in, 1)))
        return WeightSource(name, tuple(shape))

    def slot_in(key, need):
        if key not in group_of:
            group_of[key] = [len(groups), 0]
            groups.append(need)
        gi, slot = group_of[key]
        group_of[key][1] += 1
        return gi, slot

    near_one, near_zero = ("normal", 1.0, 0.1), ("normal", 0.0, 0.1)
    bindings += [WeightBinding(("embedding", "weight"), (src("embed", V, D, rule=("normal", 0.0, 1.0)),)),
                 WeightBinding(("final_norm", "weight"), (src("final.norm", D, rule=near_zero),), kind="vector"),
                 WeightBinding(("lm_head", "weight"), (src("head", V, D),))]
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer

        def target(part, local):
            return ("layer", i, part, local)

        if isinstance(m, SigmoidAttentionConfig):
            head = -(-max(m.dim, m.vdim) // 16) * 16
            mixer = PartSpec("gated_attention", {
                "hidden_size": D, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                "rot_base": m.rot_base, "rot_dims": m.rot_dims, "rot_pairs": "interleaved", "qk_norm": True, "norm_weights": True,
                "norm_scope": "all", "eps": cfg.norm_eps, "rotate_values": True, "weights": "sigmoid", "gate": "none"})
            gi, slot = slot_in(("paged", m.kv_heads, head),
                               CacheGroupSpec(name=f"attention_{m.kv_heads}x{head}", kind="full", slots=0, kv_heads=m.kv_heads, head_dim=head))
            entry = RunEntry(layer=i, cache_group=gi, cache_slot=slot, write_cache=True)
            mp = p + "mix."
            bindings += [
                WeightBinding(target("mixer", "qkvg.weight"),
                              (src(mp + "q", m.heads * m.dim, D), src(mp + "k", m.kv_heads * m.dim, D), src(mp + "v", m.kv_heads * m.vdim, D))),
                WeightBinding(target("mixer", "o.weight"), (src(mp + "o", D, m.heads * m.vdim),)),
                WeightBinding(target("mixer", "q_norm.weight"), (src(mp + "q.norm", m.heads * m.dim, rule=near_one),), kind="vector"),
                WeightBinding(target("mixer", "k_norm.weight"), (src(mp + "k.norm", m.kv_heads * m.dim, rule=near_one),), kind="vector"),
                WeightBinding(target("mixer", "score_bias"), (src(mp + "pb", m.heads, rule=("normal", -1.0, 1.0)),), kind="vector"),
            ]
        else:
            assert isinstance(m, LatentMixerConfig)
            shared = m.kv_from is not None
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                "scale": m.scale, "eps": cfg.norm_eps, "window": 0, "rot_base": m.rot_base, "rot_dims": m.rot_dims,
                "q_rank": m.q_rank, "shared_latent": shared})
            if shared:
                gi, slot = place_of[m.kv_from]
            else:
                row = -(-(m.kv_rank + m.rot_dim) // 16) * 16
                gi, slot = slot_in(("latent", row),
                                   CacheGroupSpec(name=f"latent_{row}", kind="full", slots=0, kv_heads=1, head_dim=row, planes=1))
                place_of[i] = (gi, slot)
            entry = RunEntry(layer=i, cache_group=gi, cache_slot=slot, write_cache=not shared)
            mp = p + "mix."
            qw = m.heads * (m.dim + m.rot_dim)
            bindings += [
                WeightBinding(target("mixer", "dq.weight"), (src(mp + "dq", m.q_rank, D),)),
                WeightBinding(target("mixer", "dq_norm.weight"), (src(mp + "dq.norm", m.q_rank, rule=near_one),), kind="vector"),
                WeightBinding(target("mixer", "uq.weight"), (src(mp + "uq", qw, m.q_rank),)),
                WeightBinding(target("mixer", "uk.weight"), (src(mp + "uk", m.heads * m.dim, m.kv_rank),)),
                WeightBinding(target("mixer", "uv.weight"), (src(mp + "uv", m.heads * m.vdim, m.kv_rank),)),
                WeightBinding(target("mixer", "o.weight"), (src(mp + "o", D, m.heads * m.vdim),)),
            ]
            if not shared:
                bindings += [
                    WeightBinding(target("mixer", "dkv.weight"), (src(mp + "dkv", m.kv_rank + m.rot_dim, D),)),
                    WeightBinding(target("mixer", "dkv_norm.weight"), (src(mp + "dkv.norm", m.kv_rank, rule=near_one),), kind="vector"),
                ]
        run.append(entry)
        mlp = layer.mlp
        if mlp is None:
            feed_forward = None
            ignored += [p + "norm2", p + "norm2b"]
        elif isinstance(mlp, DenseMlpConfig):
            f = mlp.ff
            feed_forward = PartSpec("mlp", {"hidden_size": D, "intermediate_size": f, "activation": "relu2"})
            bindings += [WeightBinding(target("feed_forward", "up.weight"), (src(p + "mlp.up", f, D),)),
                         WeightBinding(target("feed_forward", "down.weight"), (src(p + "mlp.down", D, f),))]
        else:
            assert isinstance(mlp, MoeMlpConfig)
            f, outputs = mlp.expert_ff, mlp.experts + mlp.identity
            feed_forward = PartSpec("routed_experts", {
                "hidden_size": D, "experts": mlp.experts, "top": mlp.top, "expert_size": f, "router": "softmax_all",
                "activation": "relu2", "identity": mlp.identity, "correction": True, "groups": mlp.groups, "keep": mlp.keep})
            bindings += [
                WeightBinding(target("feed_forward", "router.weight"), (src(p + "mlp.router", outputs, D),), kind="float32"),
                WeightBinding(target("feed_forward", "router.correction"),
                              (src(p + "mlp.correction", outputs, rule=("normal", 0.0, 0.5 / outputs)),), kind="vector"),
                WeightBinding(target("feed_forward", "experts.up.weight"),
                              tuple(src(f"{p}mlp.e{e}.up", f, D) for e in range(mlp.experts))),
                WeightBinding(target("feed_forward", "experts.down.weight"),
                              tuple(src(f"{p}mlp.e{e}.down", D, f) for e in range(mlp.experts))),
            ]
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if feed_forward is not None else ()):
            bindings.append(WeightBinding(target(name, "weight"), (src(p + name, D, rule=near_zero),), kind="vector"))
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, norm=norm, block="sandwich"))

    counts = {gi: n for gi, n in group_of.values()}
    groups = [replace(g, slots=counts[gi]) for gi, g in enumerate(groups)]
    if present is not None:
        ignored = [name for name in ignored if name in present]
    embedding = PartSpec("token_table", {"vocab_size": V, "hidden_size": D, "scale": cfg.embedding_scale})
    return ModelPlan(architecture=RikolixConfig.ARCHITECTURE, vocab_size=V, hidden_size=D, layers=layers, run=run,
                     cache_groups=groups, final_norm=norm, bindings=bindings, embedding=embedding,
                     eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id,
                     init={"default": ("normal", 0.0, 0.02), "suffix": init},
                     ignored=tuple(ignored) if present is not None else ())


def plan_for_checkpoint(cfg: RikolixConfig, shapes) -> ModelPlan:
    return build_rikolix_plan(cfg, present=set(shapes))


register_architecture(RikolixConfig.ARCHITECTURE, RikolixConfig, build_rikolix_plan, refine=plan_for_checkpoint)
