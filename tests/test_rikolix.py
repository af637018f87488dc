"""The Rikolix decoder in the engine against the plain implementation (``plain_rikolix``): each mechanism alone (norm weights
stored around zero, the sigmoid attention with its norm over whole projections, neighbouring rotation pairs and values that
turn, the latent attention with queries through a latent and with latents shared between layers, the dense squared-relu
feed-forward, the router with correction and groups, experts that return their input), whole prompts against token-by-token
decoding, portions down to two tokens, mixed batches with pages and seats used again, a far key among hundreds, keys on
page borders, the first tokens, long decoding, other sizes, and greedy generation through the engine's entry point.

Everything runs on the CPU with the reference kernels handed to the engine (host logic: plan, cache groups, run entries
that read another entry's cache, metadata) and, marked ``gpu``, with the CUDA kernels in float32 and bfloat16.  float32 is
compared row by row with the float64 oracle; bfloat16 through a whole model is measured against what rounding alone does.
"""
import json
import os
import random
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

import helpers
import kernel_refs
import plain_rikolix as plain
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import ConfigError, EngineConfig, resolve
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.engine.runtime import Engine
from flexengine_b200.parts import CacheGroupSpec, PartSpec, RunEntry, build_part
from flexengine_b200.weights import load_model, write_random_model
from test_fedutar import (CASES, DEVICES, F64, as64, bind_by_checkpoint_names, close, drive, ops_for, randn, row_errors,
                          simple_ctx, step_context)


# ---- configurations ---------------------------------------------------------------------------------------------------
def attention(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": scale if scale is not None else dim ** -0.5, "rot": {"base": base, "dims": rot_dims}}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, kv_from=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, groups=1, keep=1):
    router = {"experts": experts, "identity": identity, "top": top}
    if groups > 1 or keep > 1:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(vocab, width, eps, scale, layers):
    return {"architecture": "Rikolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}


# U: latents first and shared at once by the next layer and again by the last; value heads wider than key heads; part of a head
#    rotated; a layer without a feed-forward; three groups of which two are kept, one identity expert
# V: attention first; as many key/value heads as query heads in one layer and one key/value head in another; no rotation of
#    queries and keys in one layer; two latent layers that each make their own; no groups, no identity experts, one expert chosen
# W: head size 64 (the tensor-core kernels in bfloat16), groups of four query heads, cached rows of 128 + 32, four experts of
#    which all four are chosen beside two identity experts in three groups
CONFIGS = {
    "U": config(211, 64, 1e-5, 3.0, [
        (latent(3, 8, 4, 12, 20, 10, base=500.0), moe(5, 1, 2, 24, groups=3, keep=2)),
        (latent(2, 16, 4, 8, 20, 24, base=500.0, kv_from=0), dense(96)),
        (attention(4, 2, 16, 24, 8), None),
        (latent(4, 4, 4, 4, 20, 6, base=500.0, kv_from=0), moe(4, 0, 2, 16, groups=2, keep=1))]),
    "V": config(301, 96, 3e-6, 1.0, [
        (attention(3, 3, 16, 16, 0), moe(6, 0, 1, 40)),
        (latent(2, 24, 8, 24, 40, 32, rot_dims=4), dense(112)),
        (attention(5, 1, 8, 12, 8, base=77.0), dense(64)),
        (latent(1, 12, 2, 20, 24, 16), moe(3, 3, 3, 8, groups=6, keep=5))]),
    "W": config(400, 128, 1e-6, 0.5, [
        (attention(8, 2, 64, 64, 32, base=500000.0), dense(192)),
        (latent(4, 32, 32, 32, 128, 48, base=1e6), moe(4, 2, 4, 64, groups=3, keep=2)),
        (latent(4, 32, 32, 64, 128, 48, base=1e6, kv_from=1), dense(128)),
        (attention(4, 4, 64, 32, 64), moe(8, 0, 3, 32, groups=4, keep=2))]),
}
PAGE = {"U": 16, "V": 8, "W": 16}
LENGTHS = {"U": [5, 33, 70, 1, 47], "V": [2, 40, 77, 23], "W": [150, 64, 90]}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp(f"rikolix_{name}")
        write_random_model(cfg, str(d), seed=83 + i)
        out[name] = str(d)
    return out


def make_runner(model_dir, dtype, device, pages, page, seats=4):
    _cfg, plan, model = load_model(model_dir, dtype, device)
    cache = CacheManager(plan.cache_groups, pages, page, seats, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], device)
    return ModelRunner(model, cache, ops=ops_for(device))


def plain_logits(model_dir, ids, margins=None):
    cfg, weights = plain.read_model_folder(model_dir)
    return plain.forward_logits(cfg, weights, ids, margins=margins)


def as_rounding_allows(model_dir, pairs, what):
    """bfloat16 through a whole model.  Every sublayer's output is brought to unit size by a norm of its own, and a router's
    close call changes a token's experts, so small random models turn rounding into visible differences.  The measure is what
    rounding alone does: the same sequences through the reference kernels in bfloat16 (whole prompts, on the CPU), both
    against the float64 oracle.  The device's median and ninth-decile row errors may be twice the reference kernels' and
    0.03 / 0.06 more."""
    device_errors, reference_errors = [], []
    reference = make_runner(model_dir, "bfloat16", "cpu", 64, 16, seats=1)
    for ids, positions, rows in pairs:
        want = plain_logits(model_dir, ids)[positions]
        device_errors.append(row_errors(rows, want))
        rounded = reference.step([StepEntry("ref", ids, list(positions))])
        reference.finish("ref")
        reference_errors.append(row_errors(rounded, want))
    device_errors, reference_errors = torch.cat(device_errors), torch.cat(reference_errors)
    for q, slack in ((0.5, 0.03), (0.9, 0.06)):
        mine, allowed = float(device_errors.quantile(q)), 2.0 * float(reference_errors.quantile(q)) + slack
        assert mine <= allowed, f"{what}: quantile {q} of the row errors is {mine:.3f}, rounding alone allows {allowed:.3f}"


def compare(model_dir, results, requests, dtype, what):
    pairs = []
    for rid, ids in requests.items():
        rows = sorted(p for (r, p) in results if r == rid)
        assert rows == list(range(len(ids))), f"{what}: request {rid} misses rows"
        got = torch.stack([results[(rid, p)] for p in rows])
        if dtype == "float32":
            close(got, plain_logits(model_dir, ids), dtype, f"{what} request {rid}", bars=(3e-4, 0.0))
        pairs.append((ids, rows, got))
    if dtype != "float32":
        as_rounding_allows(model_dir, pairs, what)


def requests_for(name, seed=3):
    rng = random.Random(seed)
    return {f"r{i}": helpers.random_prompt(rng, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# ---- configuration and plan ---------------------------------------------------------------------------------------------
def test_plan_of_parts_and_cache_groups():
    _typed, plan = resolve(CONFIGS["U"])
    assert plan.architecture == "Rikolix" and [layer.block for layer in plan.layers] == ["sandwich"] * 4
    assert [layer.mixer.kind for layer in plan.layers] == ["latent_attention", "latent_attention", "gated_attention", "latent_attention"]
    assert [None if layer.feed_forward is None else layer.feed_forward.kind for layer in plan.layers] == ["routed_experts", "mlp", None, "routed_experts"]
    groups = {g.name: g for g in plan.cache_groups}
    # one slot of cached rows serves three layers; the rows are the latent and the rotated key part, padded to 16
    assert groups["latent_32"].slots == 1 and groups["latent_32"].planes == 1 and groups["latent_32"].head_dim == 32
    assert groups["attention_2x32"].slots == 1 and groups["attention_2x32"].head_dim == 32
    run = plan.run
    assert [(e.cache_group, e.cache_slot, e.write_cache) for e in run] == [(0, 0, True), (0, 0, False), (1, 0, True), (0, 0, False)]
    assert plan.final_norm.params["unit_offset"] is True
    _typed, plan = resolve(CONFIGS["V"])
    latents = [g for g in plan.cache_groups if g.name.startswith("latent")]
    assert sorted((g.head_dim, g.slots) for g in latents) == [(32, 1), (48, 1)]
    _typed, plan = resolve(CONFIGS["W"])
    names = {name for b in plan.bindings for name in [s.name for s in b.sources]}
    assert "l2.mix.dkv" not in names and "l1.mix.dkv" in names and "l1.mlp.correction" in names and "l1.mlp.e3.up" in names
    assert "l1.mlp.e4.up" not in names and "head" in names


def test_configuration_errors_are_named():
    def broken(change):
        cfg = json.loads(json.dumps(CONFIGS["U"]))
        change(cfg)
        return cfg

    cases = [
        (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
        (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
        (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
        (lambda c: c["layers"][1]["mixer"].update(kv_rank=24), "kv_rank"),
        (lambda c: c["layers"][3]["mixer"].update(rot_dim=8), "rot_dim"),
        (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
        (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "rot.dims"),
        (lambda c: c["layers"][2]["mixer"].update(vdim=13), "vdim"),
        (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
        (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "keep"),
        (lambda c: c["layers"][0].update(type="mystery"), "mystery"),
        (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
        (lambda c: c["norm"].update(eps=0.0), "eps"),
    ]
    for change, word in cases:
        with pytest.raises(ConfigError, match=word):
            resolve(broken(change))


def test_tensors_of_absent_parts_are_refused(tmp_path):
    """A layer that reads another layer's latents has no matrix of its own for them: a checkpoint that brings one is refused
    by name, as is one that lacks a tensor."""
    from flexengine_b200.weights.safetensors_io import write_safetensors
    cfg = CONFIGS["U"]
    write_random_model(cfg, str(tmp_path), seed=1)
    _c, weights = plain.read_model_folder(str(tmp_path))
    tensors = {k: v.to(torch.bfloat16) for k, v in weights.items()}

    def write():
        write_safetensors(str(tmp_path / "model.safetensors"), [(n, tuple(t.shape), t.dtype) for n, t in tensors.items()],
                          lambda n: tensors[n])
    tensors["l1.mix.dkv"] = torch.ones(24, 64, dtype=torch.bfloat16)
    write()
    with pytest.raises(Exception, match="l1.mix.dkv"):
        load_model(str(tmp_path), "float32", "cpu")
    del tensors["l1.mix.dkv"], tensors["l0.mlp.correction"]
    write()
    with pytest.raises(Exception, match="l0.mlp.correction"):
        load_model(str(tmp_path), "float32", "cpu")


# ---- each mechanism alone -----------------------------------------------------------------------------------------
def run_mixer(mixer, entry=None):
    entry = entry or RunEntry(layer=0, cache_group=0, cache_slot=0, write_cache=True)
    return lambda ctx, rows: mixer.forward(ctx, rows, entry)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("width", [40, 97, 192])
def test_norm_with_weights_stored_around_zero(device, dtype, width):
    dt = getattr(torch, dtype)
    norm = build_part("norm", PartSpec("rmsnorm", {"hidden_size": width, "eps": 1e-5, "unit_offset": True}))
    stored = randn(width, seed=1, scale=0.2)
    norm.bind({"weight": stored.to(device=device, dtype=torch.float32)})
    x = randn(9, width, seed=2, scale=3.0)
    delta = randn(9, width, seed=3)
    residual = x.to(device).float().clone()
    got = norm.forward(simple_ctx(device, dt), residual, delta.to(device=device, dtype=dt))
    want = plain.stream_norm(x.to(F64) + delta.to(F64), 1e-5, stored.to(F64))
    close(got.float().cpu(), want, dtype, f"norm of width {width}", bars=(1e-5, 2e-2))
    # as the norm after a sublayer: the stream receives the branch through (1 + w)
    after = norm.after(delta.to(device=device, dtype=dt))
    assert torch.equal(after.weight.cpu(), stored.float() + 1.0)


def attention_weights(D, m, seed):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"q": randn(H * d, D, seed=seed, scale=D ** -0.5), "k": randn(G * d, D, seed=seed + 1, scale=D ** -0.5),
            "v": randn(G * dv, D, seed=seed + 2, scale=D ** -0.5), "o": randn(D, H * dv, seed=seed + 3, scale=(H * dv) ** -0.5),
            "q.norm": 1.0 + randn(H * d, seed=seed + 4, scale=0.2), "k.norm": 1.0 + randn(G * d, seed=seed + 5, scale=0.2),
            "pb": randn(H, seed=seed + 6) - 1.0}


ATTENTION_NAMES = {"qkvg.weight": ["q", "k", "v"], "o.weight": ["o"], "q_norm.weight": ["q.norm"], "k_norm.weight": ["k.norm"],
                   "score_bias": ["pb"]}


def attention_part(D, m, weights, device, dt, eps=1e-5):
    spec = PartSpec("gated_attention", {
        "hidden_size": D, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
        "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"], "rot_pairs": "interleaved", "qk_norm": True, "norm_weights": True,
        "norm_scope": "all", "eps": eps, "rotate_values": True, "weights": "sigmoid", "gate": "none"})
    mixer = build_part("mixer", spec)
    bind_by_checkpoint_names(mixer, weights, ATTENTION_NAMES, device, dt)
    need = mixer.cache_need()
    return mixer, [CacheGroupSpec("kv", need["kind"], slots=1, kv_heads=need["kv_heads"], head_dim=need["head_dim"])]


# heads, kv_heads, dim, vdim, rotated entries: values wider and narrower than keys, one head, groups of one, two and four, no
# rotation, part of a head and a whole head, head size 64 and 128 (tensor-core kernels in bfloat16)
ATTENTION_SHAPES = [(4, 2, 16, 24, 8), (2, 1, 32, 16, 32), (3, 3, 16, 16, 0), (8, 2, 64, 64, 16), (1, 1, 40, 8, 2), (6, 3, 64, 128, 64),
                    (2, 1, 8, 32, 4), (8, 4, 16, 8, 8), (2, 1, 24, 64, 24), (12, 3, 128, 24, 2), (12, 4, 24, 64, 12)]


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_sigmoid_attention_alone(device, dtype, shape):
    dt = getattr(torch, dtype)
    D, T = 48, 41
    m = attention(*shape, base=300.0)["mixer"]
    weights = attention_weights(D, m, seed=10)
    mixer, specs = attention_part(D, m, weights, device, dt)
    h = randn(T, D, seed=11)
    want = plain.sigmoid_attention(h.to(F64), as64(weights), "", m, 1e-5)
    for cuts in ([T], [1] * T, [7, 2, 19, 2, 1, 10], [2, 37, 2], [1, 1, 2, 1, 36]):
        close(drive(run_mixer(mixer), specs, h, cuts, device, dt), want, dtype, f"sigmoid attention {shape} cut {cuts[:5]}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("far", [3, 15, 16, 640])
def test_a_far_key_among_hundreds(device, dtype, decoded, far):
    """Sigmoid weights are not normalised, so a far key does not compete with the near ones: it shows only if its own weight
    is computed.  The heads' biases are far below zero, so that ordinary keys weigh next to nothing; queries and keys read
    channels 0..15 of the input (no rotation of them: the score is the plain product), and the key at position ``far`` (early
    in the sequence, on both sides of a page border, or late) has the direction of the last query behind a scale that lifts
    its weight to about one.  Its value, turned by ``far`` and turned back by the last position, decides the output."""
    dt = getattr(torch, dtype)
    D, T = 32, 700
    m = attention(4, 2, 16, 16, 0, scale=1.0)["mixer"]
    weights = attention_weights(D, m, seed=30)
    weights["q.norm"][:] = 1.0
    weights["k.norm"][:] = 1.0
    weights["pb"][:] = -14.0
    for name in ("q", "k"):
        weights[name][:] = 0.0
        for head in range(weights[name].shape[0] // 16):
            weights[name][head * 16:(head + 1) * 16, :16] = torch.eye(16)
    mixer, specs = attention_part(D, m, weights, device, dt)
    h = randn(T, D, seed=31)
    direction = randn(16, seed=32)
    direction = direction / direction.norm() * 4.0
    h[:, :16] = h[:, :16] * 0.25
    h[far, :16] = direction * 2.0
    h[-1, :16] = direction * 2.0
    want = plain.sigmoid_attention(h.to(F64), as64(weights), "", m, 1e-5)
    blind = h.clone()
    blind[far, :16] = -direction
    assert (plain.sigmoid_attention(blind.to(F64), as64(weights), "", m, 1e-5)[-1] - want[-1]).abs().max() > 0.5 * want[-1].abs().max()
    cuts = [300, 399, 1] if decoded else [2, 330, 366, 2]
    close(drive(run_mixer(mixer), specs, h, cuts, device, dt, page=16, pages=64), want, dtype, f"far key at {far}")


def latent_weights(D, m, seed, shared=False):
    H, d, r, dv, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    w = {"dq": randn(qr, D, seed=seed, scale=D ** -0.5), "dq.norm": 1.0 + randn(qr, seed=seed + 1, scale=0.2),
         "uq": randn(H * (d + r), qr, seed=seed + 2, scale=qr ** -0.5), "uk": randn(H * d, rank, seed=seed + 3, scale=rank ** -0.5),
         "uv": randn(H * dv, rank, seed=seed + 4, scale=rank ** -0.5), "o": randn(D, H * dv, seed=seed + 5, scale=(H * dv) ** -0.5)}
    if not shared:
        w.update({"dkv": randn(rank + r, D, seed=seed + 6, scale=D ** -0.5), "dkv.norm": 1.0 + randn(rank, seed=seed + 7, scale=0.2)})
    return w


LATENT_NAMES = {"dq.weight": ["dq"], "dq_norm.weight": ["dq.norm"], "uq.weight": ["uq"], "uk.weight": ["uk"], "uv.weight": ["uv"],
                "o.weight": ["o"], "dkv.weight": ["dkv"], "dkv_norm.weight": ["dkv.norm"]}


def latent_part(D, m, weights, device, dt, shared=False, eps=1e-5):
    spec = PartSpec("latent_attention", {
        "hidden_size": D, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
        "scale": m["scale"], "eps": eps, "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"], "q_rank": m["q_rank"],
        "shared_latent": shared})
    mixer = build_part("mixer", spec)
    bind_by_checkpoint_names(mixer, weights, LATENT_NAMES, device, dt)
    need = mixer.cache_need()
    return mixer, [CacheGroupSpec("rows", need["kind"], slots=1, kv_heads=1, head_dim=need["head_dim"], planes=need["planes"])]


# heads, dim, rot_dim, vdim, kv_rank, q_rank: rows that need padding and rows that do not, one head, part of the rotated part
# turned, rows of 64 and 128 (tensor-core kernels in bfloat16) and of 272 (beyond them)
LATENT_SHAPES = [(3, 8, 4, 12, 20, 10, None), (2, 24, 8, 24, 40, 32, 4), (1, 12, 2, 20, 24, 16, None), (4, 32, 16, 32, 48, 24, None),
                 (6, 32, 16, 32, 112, 96, None), (2, 16, 16, 16, 256, 8, 8), (2, 4, 32, 12, 12, 4, 16), (4, 64, 8, 4, 112, 24, None)]


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", LATENT_SHAPES)
def test_latent_attention_with_a_query_latent_alone(device, dtype, shape):
    dt = getattr(torch, dtype)
    D, T = 48, 41
    m = latent(*shape[:6], base=300.0, rot_dims=shape[6])["mixer"]
    weights = latent_weights(D, m, seed=50)
    mixer, specs = latent_part(D, m, weights, device, dt)
    h = randn(T, D, seed=51)
    want, _ = plain.latent_attention(h.to(F64), as64(weights), "", m, 1e-5)
    for cuts in ([T], [1] * T, [7, 2, 19, 2, 1, 10], [2, 37, 2]):
        close(drive(run_mixer(mixer), specs, h, cuts, device, dt), want, dtype, f"latent attention {shape} cut {cuts[:5]}")


@pytest.mark.parametrize("device,dtype", CASES)
def test_latents_shared_between_layers(device, dtype):
    """Two mixers over one cache slot: the first writes its latents, the second (other heads, other sizes, no matrix for the
    latents) reads them through its own maps, and sees other input rows than the first."""
    dt = getattr(torch, dtype)
    D, T = 40, 37
    first = latent(3, 8, 4, 12, 28, 10, base=200.0)["mixer"]
    second = latent(2, 16, 4, 8, 28, 24, base=200.0, kv_from=0)["mixer"]
    w1, w2 = latent_weights(D, first, seed=60), latent_weights(D, second, seed=70, shared=True)
    maker, specs = latent_part(D, first, w1, device, dt)
    reader, _ = latent_part(D, second, w2, device, dt, shared=True)
    assert "dkv.weight" not in reader.parameter_shapes()
    h1, h2 = randn(T, D, seed=61), randn(T, D, seed=62)
    want1, made = plain.latent_attention(h1.to(F64), as64(w1), "", first, 1e-5)
    want2, _ = plain.latent_attention(h2.to(F64), as64(w2), "", second, 1e-5, shared=made)
    write, read = RunEntry(0, 0, 0, True), RunEntry(1, 0, 0, False)

    def both(ctx, rows):
        n = rows.shape[0] // 2
        return torch.cat([maker.forward(ctx, rows[:n].contiguous(), write), reader.forward(ctx, rows[n:].contiguous(), read)], dim=-1)

    for cuts in ([T], [1] * T, [5, 2, 28, 2]):
        # ``drive`` cuts one tensor of rows: the two layers' inputs ride side by side
        ops = ops_for(device)
        cache = CacheManager(specs, 64, 4, 2, dt, device)
        outs, fed = [], 0
        for n in cuts:
            cache.reserve("r", fed + n)
            ctx = step_context(device, dt, cache, [("r", n)], ops)
            a = maker.forward(ctx, h1[fed:fed + n].to(device=device, dtype=dt).contiguous(), write)
            b = reader.forward(ctx, h2[fed:fed + n].to(device=device, dtype=dt).contiguous(), read)
            outs.append(torch.cat([a, b], dim=-1).float().cpu())
            cache.commit("r", n)
            fed += n
        close(torch.cat(outs), torch.cat([want1, want2], dim=-1), dtype, f"shared latents cut {cuts[:4]}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("sizes", [(48, 72), (40, 100), (64, 256)])
def test_dense_feed_forward_alone(device, dtype, sizes):
    dt = getattr(torch, dtype)
    D, F = sizes
    weights = {"up": randn(F, D, seed=1, scale=D ** -0.5), "down": randn(D, F, seed=2, scale=F ** -0.5)}
    part = build_part("feed_forward", PartSpec("mlp", {"hidden_size": D, "intermediate_size": F, "activation": "relu2"}))
    bind_by_checkpoint_names(part, weights, {"up.weight": ["up"], "down.weight": ["down"]}, device, dt)
    for T in (1, 5, 33):
        h = randn(T, D, seed=3 + T)
        got = part.forward(simple_ctx(device, dt), h.to(device=device, dtype=dt))
        close(got.float().cpu(), plain.dense_feed_forward(h.to(F64), as64(weights), ""), dtype, f"dense {sizes} rows {T}")


def routed_part(D, mlp, weights, device, dt):
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    spec = PartSpec("routed_experts", {"hidden_size": D, "experts": r["experts"], "top": r["top"], "expert_size": mlp["expert"]["ff"],
                                       "router": "softmax_all", "activation": "relu2", "identity": r.get("identity", 0), "correction": True,
                                       "groups": groups["count"], "keep": groups["keep"]})
    part = build_part("feed_forward", spec)
    names = {"router.weight": ["router"], "router.correction": ["correction"],
             "experts.up.weight": [f"e{e}.up" for e in range(r["experts"])], "experts.down.weight": [f"e{e}.down" for e in range(r["experts"])]}
    bind_by_checkpoint_names(part, weights, names, device, dt)
    return part


def routed_weights(D, mlp, seed):
    r, F = mlp["router"], mlp["expert"]["ff"]
    outputs = r["experts"] + r.get("identity", 0)
    w = {"router": randn(outputs, D, seed=seed, scale=2.0 * D ** -0.5), "correction": randn(outputs, seed=seed + 1, scale=0.3 / outputs)}
    for e in range(r["experts"]):
        w[f"e{e}.up"] = randn(F, D, seed=seed + 10 + e, scale=D ** -0.5)
        w[f"e{e}.down"] = randn(D, F, seed=seed + 100 + e, scale=F ** -0.5)
    return w


# experts, identity, top, size, groups, kept: groups of one expert, one group, every group kept, every output chosen, identity
# experts only in the last group or a group of their own, a single expert, enough rows for each of the product kernels
ROUTED_SHAPES = [(5, 1, 2, 24, 3, 2), (6, 0, 1, 40, 1, 1), (3, 3, 3, 8, 6, 5), (4, 2, 4, 64, 3, 2), (8, 0, 3, 32, 4, 2), (1, 0, 1, 16, 1, 1),
                 (12, 2, 2, 64, 2, 1), (2, 2, 4, 16, 2, 2), (16, 16, 4, 8, 8, 3)]


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", ROUTED_SHAPES)
def test_routed_feed_forward_alone(device, dtype, shape):
    """The chosen experts themselves are checked, not only the sum: a correction that is left out, groups that are not
    formed over experts and identity experts together, or scores that are renormalised would pass a loose bar at random
    weights.  Rows whose choice is a close call are left out in bfloat16."""
    dt = getattr(torch, dtype)
    D = 64
    mlp = moe(*shape)
    weights = routed_weights(D, mlp, seed=20)
    part = routed_part(D, mlp, weights, device, dt)
    for T in (1, 7, 90, 300):
        h = randn(T, D, seed=5 + T)
        margins = []
        want = plain.routed_feed_forward(h.to(F64), as64(weights), "", mlp, margins)
        chosen, share, _ = plain.route(h.to(F64), as64(weights), "", mlp["router"])
        ctx = simple_ctx(device, dt)
        logits = ctx.ops.linear(h.to(device=device, dtype=dt), part.router_weight, None, out_float32=True)
        got_chosen, got_share = ctx.ops.route_top(logits, part.top, 1.0, correction=part.router_correction, groups=(part.groups, part.keep))
        sure = margins[0] > (1e-5 if dtype == "float32" else 2e-2)
        if not bool(sure.any()):
            continue
        assert torch.equal(got_chosen.cpu().long()[sure], chosen[sure]), f"experts chosen {shape} rows {T}"
        assert (got_share.cpu().double()[sure] - share[sure]).abs().max() < (1e-5 if dtype == "float32" else 2e-2)
        got = part.forward(ctx, h.to(device=device, dtype=dt))
        close(got.float().cpu()[sure], want[sure], dtype, f"routed {shape} rows {T}")


def test_a_correction_and_groups_change_the_choice():
    """The oracle itself: a correction moves the choice and leaves the weights; with groups the second-best expert of all can
    lose to a worse one of a kept group; a negative choice score still beats an expert of a dropped group."""
    D = 8
    w = {"router": torch.zeros(6, D, dtype=F64), "correction": torch.zeros(6, dtype=F64)}
    h = torch.ones(1, D, dtype=F64)
    w["router"][:, 0] = torch.tensor([3.0, 0.0, 0.5, 2.9, 1.0, 0.2])
    router = {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 1}}
    chosen, share, _ = plain.route(h, w, "", router)
    assert chosen.tolist() == [[0, 1]]                      # group (0, 1) holds the best score; expert 3 is out although second
    flat = dict(router, groups={"count": 1, "keep": 1})
    assert plain.route(h, w, "", flat)[0].tolist() == [[0, 3]]
    w["correction"][:] = torch.tensor([-2.0, 0.0, 0.0, 0.0, 0.0, 0.0])
    chosen2, share2, _ = plain.route(h, w, "", router)
    assert chosen2.tolist() == [[3, 2]] and torch.allclose(share2[0, 0], torch.softmax(w["router"][:, 0], 0)[3])
    w["correction"][:] = -5.0                                # every choice score negative: still chosen from the best group
    assert plain.route(h, w, "", router)[0].tolist() == [[0, 1]]
    got, got_share = kernel_refs.route_top((h @ w["router"].T).float(), 2, 1.0, correction=w["correction"].float(), groups=(3, 1))
    assert got.tolist() == [[0, 1]] and torch.allclose(got_share.double(), torch.softmax(w["router"][:, 0], 0)[[0, 1]][None], atol=1e-6)


# ---- kernels alone (GPU) ---------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pairs", ["halves", "interleaved"])
@pytest.mark.parametrize("shape", [(4, 2, 16, 24, 32, 8, True, True), (8, 2, 64, 64, 64, 64, True, True), (3, 3, 40, 8, 48, 0, False, True),
                                   (2, 1, 128, 128, 128, 2, True, False), (5, 1, 8, 12, 16, 8, False, False)])
def test_preparation_with_norms_over_whole_projections(dtype, pairs, shape):
    from flexengine_b200 import ops
    heads, kv_heads, dim, vdim, head, rot, normed, turned = shape
    dt = getattr(torch, dtype)
    T, page, pages = 23, 8, 6
    C = (heads + kv_heads) * dim + kv_heads * vdim
    projected = randn(T, C + 5, seed=1).to(device="cuda:0", dtype=dt)
    qw = (1.0 + randn(heads * dim, seed=2, scale=0.2)).cuda() if normed else None
    kw = (1.0 + randn(kv_heads * dim, seed=3, scale=0.2)).cuda() if normed else None
    positions = torch.arange(100, 100 + T, dtype=torch.int32, device="cuda:0")
    inv = torch.pow(torch.tensor(300.0), -2.0 * torch.arange(rot // 2) / max(rot, 1)).float().cuda() if rot else None
    vinv = torch.pow(torch.tensor(300.0), -2.0 * torch.arange(vdim // 2) / vdim).float().cuda() if turned else None
    slots = torch.randperm(page * pages)[:T].to(torch.int32).cuda()
    slots[5] = -1
    outs = []
    for provider in (ops, kernel_refs):
        kc = torch.zeros(pages, kv_heads, page, head, dtype=dt, device="cuda:0")
        vc = torch.zeros_like(kc)
        q = provider.qkv_norm_rope_cache(projected[:, :C + 5], qw, kw, 1e-5, positions, inv, rot, pairs, vinv, slots, kc, vc, heads, kv_heads,
                                         dim, vdim, head, page)
        back = provider.unrotate_heads(q.view(T, heads, head)[:, :, :].contiguous().view(T, heads * head), positions,
                                       vinv if vinv is not None else torch.ones(vdim // 2, device="cuda:0"), heads, head, vdim, pairs, scale=0.5)
        outs.append((q.float(), kc.float(), vc.float(), back.float()))
    bar = 1e-5 if dtype == "float32" else 2e-2
    for a, b, what in zip(outs[0], outs[1], ("queries", "keys", "values", "turned back")):
        assert (a - b).abs().max() <= bar * max(1.0, float(b.abs().max())), what


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(4, 2, 32, 8), (8, 2, 64, 16), (6, 6, 16, 16), (16, 1, 128, 16), (3, 1, 48, 4), (12, 3, 64, 16)])
@pytest.mark.parametrize("lengths", [[(0, 70)], [(299, 1), (37, 1), (1, 1)], [(40, 33), (130, 1), (0, 2), (15, 300)], [(1000, 1)] * 3, [(0, 1100)]])
def test_sigmoid_weights_in_every_attention_kernel(dtype, shape, lengths):
    """Decode steps (clustered and split), portions, mixed steps: the CUDA kernels against the reference, with biases far
    enough apart that a head reading another head's bias shows."""
    from flexengine_b200 import ops
    nq, nkv, d, page = shape
    dt = getattr(torch, dtype)
    dev = "cuda:0"
    gen = torch.Generator().manual_seed(5)
    R = len(lengths)
    starts, counts = [s for s, _ in lengths], [n for _, n in lengths]
    T = sum(counts)
    most = max(s + n for s, n in lengths)
    per = -(-most // page)
    pages = R * per + 3
    table = torch.randperm(pages, generator=gen)[:R * per].view(R, per).to(torch.int32).to(dev)
    kc = (torch.randn(pages, nkv, page, d, generator=gen) * 0.7).to(device=dev, dtype=dt)
    vc = torch.randn(pages, nkv, page, d, generator=gen).to(device=dev, dtype=dt)
    q = torch.randn(T, nq * d + 8, generator=gen).to(device=dev, dtype=dt)[:, :nq * d + 8]
    cu = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32, device=dev)
    ctx = types.SimpleNamespace(cu_q=cu, q_start=torch.tensor(starts, dtype=torch.int32, device=dev),
                                token_request=torch.repeat_interleave(torch.arange(R, dtype=torch.int32), torch.tensor(counts)).to(dev),
                                max_q_len=max(counts), max_ctx_len=most, host_lengths=counts, host_starts=starts)
    bias = (torch.arange(nq, dtype=torch.float32) * 0.9 - 4.0).to(dev)
    scale = d ** -0.5
    want = kernel_refs.paged_attention(q, kc, vc, table, ctx, nq, nkv, d, page, scale, 0, weights="sigmoid", head_bias=bias)
    runs = {"as the step would choose": lambda: ops.paged_attention(q, kc, vc, table, ctx, nq, nkv, d, page, scale, 0, weights="sigmoid",
                                                                     head_bias=bias)}
    if dtype == "bfloat16":
        # every tensor-core kernel by name: splits merged in a cluster and by a second kernel, both prefill kernels, split keys
        common = (q, q.stride(0), kc, vc, table, ctx.cu_q, ctx.q_start)
        if max(counts) == 1 and nq // nkv <= 16:
            for splits in (1, 3, 8):
                runs[f"cluster of {splits}"] = lambda splits=splits: ops.paged_decode_cluster(
                    *common, R, nq, nkv, d, page, scale, 0, splits, sigmoid=True, head_bias=bias)
            for splits in (1, 5, 40):
                runs[f"{splits} splits and a merge"] = lambda splits=splits: ops.paged_decode_mma(
                    *common, R, nq, nkv, d, page, scale, 0, splits, sigmoid=True, head_bias=bias)
        runs["mma.sync portions"] = lambda: ops.paged_prefill_mma(*common, T, R, max(counts), nq, nkv, d, page, scale, 0, sigmoid=True,
                                                                  head_bias=bias)
        if d in (64, 128):
            for splits in (1, 4):
                runs[f"tcgen05 portions, keys split {splits} ways"] = lambda splits=splits: ops.paged_prefill_tcgen05(
                    *common, T, R, max(counts), nq, nkv, d, page, scale, 0, splits=splits, sigmoid=True, head_bias=bias)
    for what, run in runs.items():
        got = run()
        err = (got.float() - want.float()).abs().max()
        assert float(err) <= (2e-4 if dtype == "float32" else 3e-2) * max(1.0, float(want.float().abs().max())), f"{what}: error {float(err):.3e}"
    ops.check_status(dev)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,K,N", [(1, 128, 72), (8, 256, 520), (1100, 1024, 520), (2048, 1536, 1000), (37, 96, 40)])
def test_squared_relu_in_the_products_epilogues(rows, K, N):
    """The weight-streaming kernel (a handful of rows), the tcgen05 kernel (a prompt's worth) and the product with the
    activation kernel behind it give the same rows."""
    from flexengine_b200 import ops
    x = randn(rows, K, seed=1).to(device="cuda:0", dtype=torch.bfloat16)
    w = randn(N, K, seed=2, scale=K ** -0.5).to(device="cuda:0", dtype=torch.bfloat16)
    got = ops.linear_activated(x, w, "relu2")
    want = kernel_refs.linear_activated(x, w, "relu2")
    assert (got.float() - want.float()).abs().max() <= 2e-2 * max(1.0, float(want.float().abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("T,D,F,experts,identity,top", [(700, 1024, 1024, 4, 2, 2), (1500, 1024, 1536, 3, 0, 1), (300, 256, 128, 6, 3, 3)])
def test_experts_without_a_gate_on_the_grouped_products(T, D, F, experts, identity, top):
    """Enough rows and wide enough experts for the grouped tcgen05 product (and one shape for the pipelined tiles), with choices
    that name experts which return their input: those pairs have no row in the sorted order."""
    from flexengine_b200 import ops
    gen = torch.Generator().manual_seed(3)
    h = randn(T, D, seed=4).to(device="cuda:0", dtype=torch.bfloat16)
    up = randn(experts, F, D, seed=5, scale=D ** -0.5).to(device="cuda:0", dtype=torch.bfloat16)
    down = randn(experts, D, F, seed=6, scale=F ** -0.5).to(device="cuda:0", dtype=torch.bfloat16)
    chosen = torch.stack([torch.randperm(experts + identity, generator=gen)[:top] for _ in range(T)]).to(torch.int32).cuda()
    weights = torch.rand(T, top, generator=gen).cuda()
    got = ops.routed_experts(h, chosen, weights, up, down, activation="relu2", identity=identity)
    want = kernel_refs.routed_experts(h, chosen, weights, up, down, activation="relu2", identity=identity)
    assert (got.float() - want.float()).abs().max() <= 3e-2 * max(1.0, float(want.float().abs().max()))
    ops.check_status("cuda:0")


# ---- whole models -------------------------------------------------------------------------------------------------------
def scenario(kind, requests, rng):
    if kind == "whole":
        return helpers.steps_whole(requests)
    if kind == "last_decoded":
        return helpers.steps_last_decoded(requests, tail=12)
    if kind == "portions":
        return helpers.steps_portions(requests, rng)
    doubled = dict(requests)
    doubled.update({rid + "x": ids[::-1] for rid, ids in requests.items()})     # more requests than seats: seats are used again
    return helpers.steps_mixed(doubled, rng, live=4)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("kind", ["whole", "last_decoded", "portions", "mixed"])
@pytest.mark.parametrize("name", ["U", "V", "W"])
def test_model_against_plain(model_dirs, name, kind, device, dtype):
    rng = random.Random(5)
    steps = scenario(kind, requests_for(name), rng)
    page = PAGE[name]
    pages = helpers.peak_pages(steps, page) + (0 if kind == "mixed" else 1)         # just enough: pages are used again
    runner = make_runner(model_dirs[name], dtype, device, pages, page, seats=4)
    results = helpers.run_steps(runner, steps)
    assert runner.cache.used_pages == 0 and len(runner.cache.free_state_slots) == 4
    fed = {}
    for entries, _ in steps:
        for rid, toks, _w in entries:
            fed.setdefault(rid, []).extend(toks)
    compare(model_dirs[name], results, fed, dtype, f"{name}/{kind}/{dtype}")
    if device != "cpu":
        ops_for(device).check_status(device)


def test_the_stream_after_every_layer_against_plain(model_dirs):
    """The residual stream after every layer, with what is pending put in: the plain implementation's, layer by layer."""
    for name in ("U", "W"):
        ids = requests_for(name)["r1"]
        cfg, weights = plain.read_model_folder(model_dirs[name])
        after = []
        plain.forward_logits(cfg, weights, ids, after)
        _cfg, plan, model = load_model(model_dirs[name], "float32", "cpu")
        cache = CacheManager(plan.cache_groups, 8, 16, 1, torch.float32, "cpu")
        runner = ModelRunner(model, cache, ops=kernel_refs)
        cache.reserve("a", len(ids))
        ctx = runner.build_context([StepEntry("a", ids, [])])
        residual = model.embedding.forward(ctx)
        pending = None
        assert len(plan.run) == len(after)
        for at, entry in enumerate(plan.run):
            pending = model.blocks[entry.layer].forward(ctx, residual, pending, entry)
            settled = residual.double() + plain.rms_norm(pending.y.double(), pending.eps, pending.weight.double())
            assert (settled - after[at]).abs().max() < 2e-5 * float(after[at].abs().max()), f"{name}: layer {at}"


STACKS = {
    "one attention layer without a feed-forward": config(50, 32, 1e-5, 1.0, [(attention(2, 1, 16, 16, 4), None)]),
    "a chain of layers that all read the first one's latents": config(97, 48, 1e-5, 0.5, [
        (latent(2, 8, 8, 8, 24, 12), dense(32)),
        (latent(3, 4, 8, 12, 24, 8, kv_from=0), None),
        (latent(1, 16, 8, 16, 24, 20, kv_from=0), moe(2, 2, 2, 16, groups=2, keep=1)),
        (latent(2, 8, 8, 4, 24, 12, kv_from=0), dense(40))]),
    "two makers of latents, each with a reader": config(64, 40, 1e-6, 4.0, [
        (latent(2, 8, 4, 8, 12, 8), None),
        (latent(2, 16, 8, 8, 56, 8), moe(3, 1, 2, 16, groups=4, keep=3)),
        (latent(1, 8, 4, 16, 12, 16, kv_from=0), dense(24)),
        (attention(5, 5, 8, 8, 8), None),
        (latent(4, 4, 8, 4, 56, 4, kv_from=1), None)]),
}


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("stack", list(STACKS))
def test_stacks_of_other_shapes(tmp_path, stack, device, dtype):
    cfg = STACKS[stack]
    write_random_model(cfg, str(tmp_path), seed=3)
    ids = helpers.random_prompt(random.Random(1), 45, cfg["vocab"])
    runner = make_runner(str(tmp_path), dtype, device, 8, 8)
    got = [runner.step([StepEntry("a", ids[:20], list(range(20)))]), runner.step([StepEntry("a", ids[20:44], list(range(24)))]),
           runner.step([StepEntry("a", ids[44:], [0])])]
    rows = torch.cat([g.float().cpu() for g in got])
    if dtype == "float32":
        close(rows, plain_logits(str(tmp_path), ids), dtype, stack, bars=(3e-4, 0.0))
    else:
        as_rounding_allows(str(tmp_path), [(ids, list(range(len(ids))), rows)], stack)
    runner.finish("a")
    runner.cache.assert_invariants()


@pytest.mark.parametrize("device,dtype", CASES)
def test_together_and_alone(model_dirs, device, dtype):
    """Unequal requests in one batch against each alone: the same logits (to rounding in bfloat16)."""
    name = "U"
    requests = requests_for(name, seed=9)
    together = make_runner(model_dirs[name], dtype, device, 16, PAGE[name])
    logits = together.step([StepEntry(rid, ids, [len(ids) - 1]) for rid, ids in requests.items()][:4])
    for row, (rid, ids) in enumerate(list(requests.items())[:4]):
        alone = make_runner(model_dirs[name], dtype, device, 8, PAGE[name])
        close(logits[row:row + 1], alone.step([StepEntry(rid, ids, [len(ids) - 1])]), dtype, rid)


@pytest.mark.parametrize("device,dtype", CASES)
def test_first_tokens_and_long_decoding(model_dirs, device, dtype):
    """A prompt of one token, then 150 tokens decoded one by one beside a neighbour that arrives later and leaves: every row
    against the whole sequence.  Pages fill and are given back, the values turn further with every token."""
    name = "U"
    rng = random.Random(12)
    ids = helpers.random_prompt(rng, 151, CONFIGS[name]["vocab"])
    other = helpers.random_prompt(rng, 60, CONFIGS[name]["vocab"])
    runner = make_runner(model_dirs[name], dtype, device, 16, PAGE[name], seats=2)
    rows, other_rows = [], []
    for p in range(len(ids)):
        entries = [StepEntry("long", ids[p:p + 1], [0])]
        q = p - 40
        if 0 <= q < len(other):
            entries.append(StepEntry("other", other[q:q + 1], [0]))
        logits = runner.step(entries)
        rows.append(logits[0].float().cpu())
        if len(entries) == 2:
            other_rows.append(logits[1].float().cpu())
        if q == len(other) - 1:
            runner.finish("other")
        runner.cache.assert_invariants()
    for got, seq, what in ((rows, ids, "long decoding"), (other_rows, other, "the neighbour")):
        if dtype == "float32":
            close(torch.stack(got), plain_logits(model_dirs[name], seq), dtype, what, bars=(3e-4, 0.0))
        else:
            as_rounding_allows(model_dirs[name], [(seq, list(range(len(seq))), torch.stack(got))], what)


# ---- generation through the engine ----------------------------------------------------------------------------------
def greedy(model_dir, prompt, count):
    cfg, weights = plain.read_model_folder(model_dir)
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(plain.forward_logits(cfg, weights, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(model_dirs, device, graphs):
    if graphs and device == "cpu":
        pytest.skip("CUDA graphs need a CUDA device")
    name = "V"
    rng = random.Random(1)
    prompts = [helpers.random_prompt(rng, n, CONFIGS[name]["vocab"]) for n in (5, 17, 33, 1, 40, 9)]
    cfg = EngineConfig(model=model_dirs[name], device=device, dtype="float32", max_model_len=128, max_num_seqs=3,
                       max_num_batched_tokens=24, prefill_chunk_size=8, kv_block_size=PAGE[name], kv_num_blocks=48,
                       max_output_tokens=16, scheduler_policy="decode_first", cuda_graph=graphs, overlap_steps=device != "cpu")
    engine = Engine.from_model_dir(model_dirs[name], cfg, ops=ops_for(device))
    outputs = engine.generate(prompts, max_tokens=6)
    for prompt, out in zip(prompts, outputs):
        assert out.token_ids == greedy(model_dirs[name], prompt, 6)
    assert engine.cache.used_pages == 0


@pytest.mark.gpu
def test_trace_replay_program(model_dirs, tmp_path):
    """``bin/trace_run`` as a user starts it: steps on standard input, logits in files."""
    name = "U"
    ids = requests_for(name)["r1"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[20:], "want": [len(ids) - 21]}, {"id": "b", "tokens": ids[:3], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": ids[3:5], "want": [1]}], "end": ["b"]}]
    program = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    want = plain_logits(model_dirs[name], ids)
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        done = subprocess.run([sys.executable, program, "--model", model_dirs[name], "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
        vocab = CONFIGS[name]["vocab"]
        rows = [np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, vocab) for n in range(3)]
        got = torch.from_numpy(np.concatenate(rows))
        if dtype == "float32":
            close(got, want[[0, 19, len(ids) - 1, 4]], dtype, "trace_run float32", bars=(3e-4, 0.0))
        else:
            as_rounding_allows(model_dirs[name], [(ids, [0, 19, len(ids) - 1, 4], got)], "trace_run bfloat16")
