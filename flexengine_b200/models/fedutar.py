"""Fedutar as a plan of parts: a decoder whose layers have a norm before and after each sublayer, a mixer that is two
mixers side by side (softmax attention with normed queries and keys, a query temperature and an elementwise output
gate; retention, a linear attention with one fixed decay per head) and a dense feed-forward with biases or a routed one
(softmax over the chosen logits, clamped expert activations).  A span of the layers may run several times in a row with
the same weights; every pass has cache and state of its own and begins with x <- W_in [x; x0].  Logits come from the
embedding table, scaled and squashed by tanh.

Checkpoint names: ``embed``, ``loop.in``, ``final.norm``, and per layer i ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.left.q|k|v|g|o|q.norm|k.norm``, ``l<i>.mix.right.q|k|v|g|o``, ``l<i>.mlp.gate|up|down`` (+ ``.b``) or
``l<i>.mlp.e<k>.gate|up|down`` and ``l<i>.mlp.router``.  Matrices are [out, in].  The projections of a side that read the
same rows are bound as one matrix, gate and up as one, all experts of a layer as one.

Cache groups: a paged group per distinct (key/value heads, head size) of the attention sides (head size: the larger of
the query/key and the value size, in steps of 16; the smaller is padded with zeros) and a float32 state group per
distinct state size of the retention sides, each with a slot per run of a layer (a layer of the repeated span has one
per pass).
"""
from __future__ import annotations

import math
from dataclasses import replace

from ..config.fedutar_config import DenseMlpConfig, FedutarConfig, MoeMlpConfig
from ..config.registry import register_architecture
from ..parts.spec import (CacheGroupSpec, LayerSpec, ModelPlan, PartSpec, RunEntry, WeightBinding, WeightSource)


def run_order(cfg: FedutarConfig):
    """[(layer, begins a pass)] in the order the layers run."""
    count = len(cfg.layers)
    if cfg.loop is None:
        return [(i, False) for i in range(count)]
    start, stop, times = cfg.loop.start, cfg.loop.stop, cfg.loop.times
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, count)]


def build_fedutar_plan(cfg: FedutarConfig, present=None) -> ModelPlan:
    """``present``: the tensor names of a checkpoint; tensors of it that belong to nothing the configuration has (the
    second pair of norms of a layer without a feed-forward, the pass matrix of a model without a repeated span) are then
    named as ignored instead of unexpected."""
    D, V = cfg.width, cfg.vocab
    norm = PartSpec("rmsnorm", {"hidden_size": D, "eps": cfg.norm_eps})
    groups: list = []
    group_of: dict = {}            # key -> [group index, slots so far]
    layers, bindings, ignored = [], [], []
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

    near_one = ("normal", 1.0, 0.1)
    bindings += [WeightBinding(("embedding", "weight"), (src("embed", V, D, rule=("normal", 0.0, 1.0 / math.sqrt(D))),)),
                 WeightBinding(("final_norm", "weight"), (src("final.norm", D, rule=near_one),), kind="vector"),
                 WeightBinding(("lm_head", "weight"), alias_of=("embedding", "weight"))]
    junctions = []
    if cfg.loop is not None:
        junctions.append(PartSpec("reinject", {"hidden_size": D}))
        bindings.append(WeightBinding(("junction", 0, "weight"), (src("loop.in", D, 2 * D),)))
    else:
        ignored.append("loop.in")
    places = []                    # per layer: (key and spec of the left side's group, of the right side's)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        L, R = m.left, m.right

        def target(part, local):
            return ("layer", i, part, local)

        head = -(-max(L.dim, L.vdim) // 16) * 16
        left = PartSpec("gated_attention", {
            "hidden_size": D, "heads": L.heads, "kv_heads": L.kv_heads, "dim": L.dim, "vdim": L.vdim, "scale": L.scale,
            "qk_norm": True, "norm_weights": True, "eps": cfg.norm_eps, "temp_coef": L.temp_coef, "temp_every": L.temp_every,
            "gate": "element"})
        right = PartSpec("retention", {"hidden_size": D, "heads": R.heads, "dim": R.dim, "vdim": R.vdim, "decay": R.decay,
                                       "rot_base": R.rot_base, "rot_dims": R.rot_dims, "eps": cfg.norm_eps})
        mixer = PartSpec("parallel", {"hidden_size": D, "sides": (("left", left, m.left_scale), ("right", right, m.right_scale))})
        places.append(((("paged", L.kv_heads, head),
                        CacheGroupSpec(name=f"attention_{L.kv_heads}x{head}", kind="full", slots=0, kv_heads=L.kv_heads, head_dim=head)),
                       (("retention", R.heads * R.dim * R.vdim),
                        CacheGroupSpec(name=f"retention_state_{R.heads * R.dim * R.vdim}", kind="state", slots=0,
                                       state_shape=(R.heads * R.dim * R.vdim,), state_dtype="float32"))))
        lp, rp = p + "mix.left.", p + "mix.right."
        bindings += [
            WeightBinding(target("mixer", "left.qkvg.weight"),
                          (src(lp + "q", L.heads * L.dim, D), src(lp + "k", L.kv_heads * L.dim, D),
                           src(lp + "v", L.kv_heads * L.vdim, D), src(lp + "g", L.heads * L.vdim, D))),
            WeightBinding(target("mixer", "left.o.weight"), (src(lp + "o", D, L.heads * L.vdim),)),
            WeightBinding(target("mixer", "left.q_norm.weight"), (src(lp + "q.norm", L.dim, rule=near_one),), kind="vector"),
            WeightBinding(target("mixer", "left.k_norm.weight"), (src(lp + "k.norm", L.dim, rule=near_one),), kind="vector"),
            WeightBinding(target("mixer", "right.qkvg.weight"),
                          (src(rp + "q", R.heads * R.dim, D), src(rp + "k", R.heads * R.dim, D),
                           src(rp + "v", R.heads * R.vdim, D), src(rp + "g", R.heads * R.vdim, D))),
            WeightBinding(target("mixer", "right.o.weight"), (src(rp + "o", D, R.heads * R.vdim),)),
        ]
        mlp = layer.mlp
        if mlp is None:
            feed_forward = None
            ignored += [p + "norm2", p + "norm2b"]
        elif isinstance(mlp, DenseMlpConfig):
            f = mlp.ff
            feed_forward = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": f, "activation": "silu", "bias": True})
            bias = ("normal", 0.0, 0.3)
            bindings += [
                WeightBinding(target("feed_forward", "gate_up.weight"), (src(p + "mlp.gate", f, D), src(p + "mlp.up", f, D))),
                WeightBinding(target("feed_forward", "gate_up.bias"), (src(p + "mlp.gate.b", f, rule=bias), src(p + "mlp.up.b", f, rule=bias)), kind="vector"),
                WeightBinding(target("feed_forward", "down.weight"), (src(p + "mlp.down", D, f),)),
                WeightBinding(target("feed_forward", "down.bias"), (src(p + "mlp.down.b", D, rule=bias),), kind="vector"),
            ]
        else:
            assert isinstance(mlp, MoeMlpConfig)
            f = mlp.expert_ff
            feed_forward = PartSpec("routed_experts", {"hidden_size": D, "experts": mlp.experts, "top": mlp.top, "expert_size": f,
                                                       "router": "softmax_chosen", "activation": "clamped", "limit": mlp.limit})
            bindings += [
                WeightBinding(target("feed_forward", "router.weight"), (src(p + "mlp.router", mlp.experts, D),), kind="float32"),
                WeightBinding(target("feed_forward", "experts.gate_up.weight"),
                              tuple(src(f"{p}mlp.e{e}.{which}", f, D) for e in range(mlp.experts) for which in ("gate", "up"))),
                WeightBinding(target("feed_forward", "experts.down.weight"),
                              tuple(src(f"{p}mlp.e{e}.down", D, f) for e in range(mlp.experts))),
            ]
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if feed_forward is not None else ()):
            bindings.append(WeightBinding(target(name, "weight"), (src(p + name, D, rule=near_one),), kind="vector"))
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, norm=norm, block="sandwich"))

    run = []
    for i, begins in run_order(cfg):
        (lk, lneed), (rk, rneed) = places[i]
        gi, slot = slot_in(lk, lneed)
        gj, slot2 = slot_in(rk, rneed)
        run.append(RunEntry(layer=i, cache_group=gi, cache_slot=slot, write_cache=True, more=((gj, slot2),), before=0 if begins else -1))
    counts = {gi: n for gi, n in group_of.values()}
    groups = [replace(g, slots=counts[gi]) for gi, g in enumerate(groups)]
    if present is not None:
        ignored = [name for name in ignored if name in present]
    embedding = PartSpec("token_table", {"vocab_size": V, "hidden_size": D, "scale": cfg.embedding_scale})
    head = PartSpec("linear", {"vocab_size": V, "hidden_size": D, "scale": cfg.logit_scale, "softcap": cfg.logit_softcap})
    return ModelPlan(architecture=FedutarConfig.ARCHITECTURE, vocab_size=V, hidden_size=D, layers=layers, run=run,
                     cache_groups=groups, final_norm=norm, bindings=bindings, embedding=embedding, head=head,
                     eos_token_ids=cfg.eos_token_ids, bos_token_id=cfg.bos_token_id,
                     init={"default": ("normal", 0.0, 0.02), "suffix": init}, junctions=tuple(junctions),
                     ignored=tuple(ignored) if present is not None else ())


def plan_for_checkpoint(cfg: FedutarConfig, shapes) -> ModelPlan:
    return build_fedutar_plan(cfg, present=set(shapes))


register_architecture(FedutarConfig.ARCHITECTURE, FedutarConfig, build_fedutar_plan, refine=plan_for_checkpoint)
