"""The Fedutar decoder in the engine against the plain implementation (``plain_fedutar``): each mechanism alone (a branch
that ends in a norm of its own, the softmax side with normed queries and keys, a query temperature and element gates, the
retention side, both side by side, the dense feed-forward with biases, the routed one, the pass junction, the squashed
head), whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages and seats used
again, a far key among hundreds, memory of the retention state over hundreds of tokens, the edges of the query temperature's
steps, the first tokens, long decoding, other sizes (no repeated span, a span that starts at the first layer or ends at the
last, one head, all experts chosen, one expert chosen, no rotation, part of a head rotated, value and key sizes that
differ), and greedy generation through the engine's entry point.

Everything runs on the CPU with the reference kernels handed to the engine (host logic: plan, cache groups, state
seats, metadata) and, marked ``gpu``, with the CUDA kernels in float32 and bfloat16.  float32 is compared row by row with
the float64 oracle.  bfloat16 through a whole model is measured against what rounding alone does (``as_rounding_allows``).
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
import plain_fedutar as plain
from flexengine_b200.cache import CacheManager
from flexengine_b200.config import ConfigError, EngineConfig, resolve
from flexengine_b200.engine import ModelRunner, StepEntry
from flexengine_b200.engine.runtime import Engine
from flexengine_b200.parts import CacheGroupSpec, PartSpec, RunEntry, build_part
from flexengine_b200.parts.norm import PostNormed
from flexengine_b200.weights import load_model, write_random_model

DEVICES = [pytest.param("cpu", id="cpu"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
CASES = [pytest.param("cpu", "float32", id="cpu-float32"),
         pytest.param("cuda:0", "float32", id="gpu-float32", marks=pytest.mark.gpu),
         pytest.param("cuda:0", "bfloat16", id="gpu-bfloat16", marks=pytest.mark.gpu)]
F64 = torch.float64


def left_side(heads, kv_heads, dim, vdim, scale=None, temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def right_side(heads, dim, vdim, decay, rot_dims=0, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return m


def parallel(left, right, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def config(vocab, width, eps, scale, layers, loop=None, logit_scale=1.0, softcap=0.0):
    cfg = {"architecture": "Fedutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "logit_scale": logit_scale, "logit_softcap": softcap, "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# P: a span that starts at the first layer and runs twice; value heads wider than key heads and the other way round; part of a
#    head rotated and none; a layer without a feed-forward; a temperature that steps every 5 positions and one at every position
# Q: no repeated span at all; one head on each side; as many key/value heads as query heads; all experts chosen in one layer
#    and one of five in another; sizes that are no powers of two; logits that are not squashed
# R: head size 64 on the softmax side (the fast attention kernels in bfloat16), groups of four query heads, a span that ends
#    at the last layer and runs three times, retention heads of 64 x 64
CONFIGS = {
    "P": config(211, 64, 1e-5, 3.0, [
        (parallel(left_side(4, 2, 16, 24, temp=(0.3, 5)), right_side(3, 16, 8, [0.9, 0.95, 0.99], 8, base=500.0), 1.2, 0.9), dense(96)),
        (parallel(left_side(2, 2, 8, 8), right_side(2, 24, 40, [0.5, 0.999]), 0.7, 1.3), moe(6, 2, 24, 1.5)),
        (parallel(left_side(3, 1, 32, 16, temp=(1.0, 1)), right_side(1, 12, 12, [0.97], 12), 1.0, 1.0), None)],
        loop=(0, 2, 2), logit_scale=1.5, softcap=20.0),
    "Q": config(301, 96, 3e-6, 1.0, [
        (parallel(left_side(1, 1, 48, 40), right_side(1, 40, 24, [0.98], 20, base=77.0), 1.0, 0.5), moe(3, 3, 40, 0.8)),
        (parallel(left_side(3, 3, 16, 16, temp=(0.7, 16)), right_side(5, 8, 12, [0.9, 0.92, 0.94, 0.96, 1.0], 8), 0.5, 2.0), dense(112)),
        (parallel(left_side(2, 1, 24, 40), right_side(2, 16, 16, [0.99, 0.995]), 1.0, 1.0), moe(5, 1, 56, 3.0))],
        logit_scale=0.5),
    "R": config(400, 128, 1e-6, 2.0, [
        (parallel(left_side(8, 2, 64, 64, temp=(0.5, 32)), right_side(2, 64, 64, [0.97, 0.999], 32, base=50000.0), 1.1, 1.2), dense(192)),
        (parallel(left_side(4, 4, 64, 32), right_side(4, 32, 48, [0.9, 0.95, 0.99, 0.995], 32), 1.0, 1.0), moe(8, 3, 64, 2.5)),
        (parallel(left_side(8, 2, 64, 64), right_side(2, 64, 64, [0.98, 0.99], 64), 0.9, 0.8), moe(4, 2, 32, 1.0))],
        loop=(1, 3, 3), logit_scale=2.0, softcap=15.0),
}
PAGE = {"P": 16, "Q": 8, "R": 16}
LENGTHS = {"P": [5, 33, 70, 1, 47], "Q": [2, 40, 77, 23], "R": [150, 64, 90]}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp(f"fedutar_{name}")
        write_random_model(cfg, str(d), seed=61 + i)
        out[name] = str(d)
    return out


def ops_for(device):
    if device == "cpu":
        return kernel_refs
    from flexengine_b200 import ops
    return ops


def make_runner(model_dir, dtype, device, pages, page, seats=4):
    _cfg, plan, model = load_model(model_dir, dtype, device)
    cache = CacheManager(plan.cache_groups, pages, page, seats, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], device)
    return ModelRunner(model, cache, ops=ops_for(device))


def plain_logits(model_dir, ids):
    cfg, weights = plain.read_model_folder(model_dir)
    return plain.forward_logits(cfg, weights, ids)


def close(got, want, dtype, what, bars=(1e-4, 6e-2)):
    """Every row within 1e-4 (float32) or 6e-2 (bfloat16) of its own spread, with a tenth of the overall spread as the
    floor."""
    assert got.shape == want.shape, what
    err = row_errors(got.reshape(-1, want.shape[-1]), want.reshape(-1, want.shape[-1]))
    bar = bars[0] if dtype == "float32" else bars[1]
    worst = int(err.argmax())
    assert float(err[worst]) <= bar, f"{what}: row {worst} is off by {float(err[worst]):.3e} of its spread (bar {bar:.0e})"


def row_errors(got, want):
    """Per row: the largest difference over the row's spread (a tenth of the overall spread as the floor)."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape and torch.isfinite(got).all()
    floor = max(0.1 * float(want.std()), 1e-3)
    return (got - want).abs().max(dim=-1).values / torch.clamp(want.std(dim=-1), min=floor)


def as_rounding_allows(model_dir, pairs, what):
    """bfloat16 through a whole model.  Small random models of this design turn rounding into large differences: every
    sublayer's output is brought to unit size by a norm of its own, a retention head whose sum nearly cancels is divided by
    its own small size, and a router's close call changes a token's experts and, through the state, the tokens after it.
    So the measure is what rounding alone does: the same sequences through the reference kernels in bfloat16 (whole prompts,
    on the CPU), both against the float64 oracle.  ``pairs``: [(ids, positions, rows from the device)].  The device's
    median and ninth-decile row errors may be twice the reference kernels' and 0.03 / 0.06 more."""
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
            # through all runs of all layers and a head that multiplies, rounding alone reaches 1e-4 of a row's spread
            close(got, plain_logits(model_dir, ids), dtype, f"{what} request {rid}", bars=(3e-4, 0.0))
        pairs.append((ids, rows, got))
    if dtype != "float32":
        as_rounding_allows(model_dir, pairs, what)


def requests_for(name, seed=3):
    rng = random.Random(seed)
    return {f"r{i}": helpers.random_prompt(rng, n, CONFIGS[name]["vocab"]) for i, n in enumerate(LENGTHS[name])}


# ---- configuration and plan ---------------------------------------------------------------------------------------------
def test_plan_of_parts_and_cache_groups():
    _typed, plan = resolve(CONFIGS["P"])
    # layers 0 and 1 run twice in a row, then layer 2; every run has cache and state of its own; a pass begins with the junction
    assert [e.layer for e in plan.run] == [0, 1, 0, 1, 2]
    assert [e.before for e in plan.run] == [0, -1, 0, -1, -1]
    assert len(plan.junctions) == 1 and plan.junctions[0].kind == "reinject"
    places = [(e.cache_group, e.cache_slot) + e.more[0] for e in plan.run]
    assert len(set((g, s) for g, s, _, _ in places)) == 5 and len(set((g, s) for _, _, g, s in places)) == 5
    groups = {g.name: g for g in plan.cache_groups}
    # head size of the pages: the larger of key and value size, in steps of 16
    assert (groups["attention_2x32"].kind, groups["attention_2x32"].slots) == ("full", 2)
    assert groups["attention_2x16"].slots == 2 and groups["attention_1x32"].slots == 1
    assert groups["retention_state_384"].state_shape == (3 * 16 * 8,) and groups["retention_state_384"].state_dtype == "float32"
    assert groups["retention_state_1920"].slots == 2 and groups["retention_state_144"].slots == 1
    assert [layer.feed_forward.kind if layer.feed_forward else None for layer in plan.layers] == ["gated_mlp", "routed_experts", None]
    assert all(layer.block == "sandwich" for layer in plan.layers)
    left = dict(plan.layers[0].mixer.params["sides"][0][1].params)
    assert (left["qk_norm"], left["norm_weights"], left["gate"], left["temp_coef"], left["temp_every"]) == (True, True, "element", 0.3, 5)
    assert dict(plan.layers[1].mixer.params["sides"][0][1].params)["temp_coef"] == 0.0
    # no repeated span: no junction, every layer once
    _typed, plan = resolve(CONFIGS["Q"])
    assert [e.layer for e in plan.run] == [0, 1, 2] and not plan.junctions and all(e.before == -1 for e in plan.run)
    # a span that ends at the last layer and runs three times
    _typed, plan = resolve(CONFIGS["R"])
    assert [e.layer for e in plan.run] == [0, 1, 2, 1, 2, 1, 2] and [e.before for e in plan.run] == [-1, 0, -1, 0, -1, 0, -1]


def test_configuration_errors_are_named():
    def broken(change):
        cfg = json.loads(json.dumps(CONFIGS["P"]))
        change(cfg)
        return cfg
    with pytest.raises(ConfigError, match="unknown mixer type"):
        resolve(broken(lambda c: c["layers"][1].update(type="serial")))
    with pytest.raises(ConfigError, match="decay"):
        resolve(broken(lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.9])))
    with pytest.raises(ConfigError, match="loop"):
        resolve(broken(lambda c: c["loop"].update(stop=4)))
    with pytest.raises(ConfigError, match="rot.dims"):
        resolve(broken(lambda c: c["layers"][0]["mixer"]["right"]["rot"].update(dims=7)))
    with pytest.raises(ConfigError, match="unknown mlp kind"):
        resolve(broken(lambda c: c["layers"][0]["mlp"].update(kind="sparse")))
    with pytest.raises(ConfigError, match="experts"):
        resolve(broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=7)))
    with pytest.raises(ConfigError, match="scale"):
        resolve(broken(lambda c: c["layers"][0]["mixer"]["left"].pop("scale")))


def test_tensors_of_absent_parts_are_ignored_and_others_are_not(tmp_path):
    """A checkpoint may bring the second pair of norms of a layer without a feed-forward; a tensor that belongs to nothing is
    refused by name."""
    from flexengine_b200.weights.safetensors_io import CheckpointReader, write_safetensors
    cfg = CONFIGS["P"]
    write_random_model(cfg, str(tmp_path), seed=5)
    reader = CheckpointReader(str(tmp_path))
    tensors = {name: reader.read(name).clone() for name in reader.names()}
    reader.close()
    path = os.path.join(str(tmp_path), "model.safetensors")

    def write():
        write_safetensors(path, [(n, tuple(t.shape), t.dtype) for n, t in tensors.items()], lambda name: tensors[name])
    tensors["l2.norm2"] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    tensors["l2.norm2b"] = torch.ones(cfg["width"], dtype=torch.bfloat16)
    write()
    load_model(str(tmp_path), "float32", "cpu")
    tensors["l2.mix.middle.q"] = torch.ones(4, 4, dtype=torch.bfloat16)
    write()
    with pytest.raises(Exception, match="l2.mix.middle.q"):
        load_model(str(tmp_path), "float32", "cpu")


# ---- each mechanism alone -----------------------------------------------------------------------------------------
def step_context(device, dtype, cache, entries, ops):
    runner = ModelRunner.__new__(ModelRunner)                # only build_context is used
    runner.cache, runner.ops, runner.device = cache, ops, cache.device
    runner._ring, runner._ring_at, runner.h2d_bytes = [], 0, 0
    runner.model = types.SimpleNamespace(dtype=dtype)
    return runner.build_context([StepEntry(rid, [0] * n, []) for rid, n in entries])


def drive(run, group_specs, h, cuts, device, dtype, page=4, seats=2, pages=96):
    """``run(ctx, rows)`` over a cache of its own, the sequence cut into ``cuts`` portions; a second request runs in between
    and ends, so that its seat and pages are used again."""
    ops = ops_for(device)
    cache = CacheManager(group_specs, pages, page, seats, dtype, device)
    outs, fed = [], 0
    for n in cuts:
        cache.reserve("r", fed + n)
        ctx = step_context(device, dtype, cache, [("r", n)], ops)
        outs.append(run(ctx, h[fed:fed + n].to(device=device, dtype=dtype).contiguous()).float().cpu())
        cache.commit("r", n)
        fed += n
        if fed == cuts[0]:                                   # a neighbour that comes and goes
            cache.reserve("other", 7)
            ctx = step_context(device, dtype, cache, [("other", 7)], ops)
            run(ctx, torch.randn(7, h.shape[1]).to(device=device, dtype=dtype))
            cache.commit("other", 7)
            cache.free("other")
    cache.assert_invariants()
    return torch.cat(outs)


def bind_by_checkpoint_names(part, weights, names, device, dtype):
    tensors = {}
    for local, (shape, kind) in part.parameter_shapes().items():
        source = torch.cat([weights[n].reshape(-1, *weights[n].shape[1:]) for n in names[local]])
        held = torch.float32 if kind in ("vector", "float32") else dtype
        tensors[local] = source.reshape(shape).to(device=device, dtype=held).contiguous()
    part.bind(tensors)


def bf16_exact(t):
    return t.to(torch.bfloat16).float()


def randn(*shape, seed, scale=1.0):
    return bf16_exact(torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale)


def as64(weights):
    return {k: v.to(F64) for k, v in weights.items()}


def simple_ctx(device, dt):
    return types.SimpleNamespace(ops=ops_for(device), dtype=dt)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("width", [40, 97, 192])
@pytest.mark.parametrize("with_bias", [False, True])
def test_branch_through_a_norm_of_its_own(device, dtype, width, with_bias):
    """x <- x + w_b (y + b) / rms(y + b), then the next norm of the sum, in one kernel: all rows in place, chosen rows without
    writing, the branch in float32 and in the compute dtype, with and without a bias still to add."""
    dt = getattr(torch, dtype)
    T, D, eps = 11, width, 1e-5
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(1))
    y = randn(T, D, seed=2, scale=3.0)
    bias = randn(D, seed=3) if with_bias else None
    w_branch, w_next = randn(D, seed=4) + 1.0, randn(D, seed=5) + 1.0
    inner = y.to(F64) + (bias.to(F64) if with_bias else 0.0)
    new = x.to(F64) + plain.rms_norm(inner, eps, w_branch.to(F64))
    want = plain.rms_norm(new, eps, w_next.to(F64))
    norm_branch = build_part("norm", PartSpec("rmsnorm", {"hidden_size": D, "eps": eps}))
    norm_next = build_part("norm", PartSpec("rmsnorm", {"hidden_size": D, "eps": eps}))
    norm_branch.bind({"weight": w_branch.to(device)})
    norm_next.bind({"weight": w_next.to(device)})
    ctx = simple_ctx(device, dt)
    for held in (torch.float32, dt):
        pending = norm_branch.after(y.to(device=device, dtype=held), None if bias is None else bias.to(device))
        assert isinstance(pending, PostNormed)
        stream = x.clone().to(device)
        rows = torch.tensor([9, 0, 4], dtype=torch.int32, device=device)
        some = norm_next.forward(ctx, stream, pending, rows=rows)
        assert torch.equal(stream.cpu(), x)
        close(some, want[rows.long().cpu()], dtype, "chosen rows", bars=(2e-5, 3e-2))
        got = norm_next.forward(ctx, stream, pending)
        close(got, want, dtype, "all rows", bars=(2e-5, 3e-2))
        assert (stream.double().cpu() - new).abs().max() < 1e-5 * float(new.abs().max())


def softmax_weights(D, m, seed):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"q": randn(H * d, D, seed=seed, scale=D ** -0.5), "k": randn(G * d, D, seed=seed + 1, scale=D ** -0.5),
            "v": randn(G * dv, D, seed=seed + 2, scale=D ** -0.5), "g": randn(H * dv, D, seed=seed + 3, scale=D ** -0.5),
            "o": randn(D, H * dv, seed=seed + 4, scale=(H * dv) ** -0.5),
            "q.norm": randn(d, seed=seed + 5, scale=0.3) + 1.0, "k.norm": randn(d, seed=seed + 6, scale=0.3) + 1.0}


SOFTMAX_NAMES = {"qkvg.weight": ["q", "k", "v", "g"], "o.weight": ["o"], "q_norm.weight": ["q.norm"], "k_norm.weight": ["k.norm"]}


def softmax_spec(D, m, eps=1e-5):
    temp = m.get("q_temp") or {"coef": 0.0, "every": 1}
    return PartSpec("gated_attention", {
        "hidden_size": D, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
        "qk_norm": True, "norm_weights": True, "eps": eps, "temp_coef": temp["coef"], "temp_every": temp["every"], "gate": "element"})


def softmax_part(D, m, weights, device, dt, eps=1e-5):
    mixer = build_part("mixer", softmax_spec(D, m, eps))
    bind_by_checkpoint_names(mixer, weights, SOFTMAX_NAMES, device, dt)
    need = mixer.cache_need()
    return mixer, [CacheGroupSpec("rows", need["kind"], slots=1, kv_heads=need["kv_heads"], head_dim=need["head_dim"], window=need["window"])]


def run_mixer(mixer, more=()):
    return lambda ctx, rows: mixer.forward(ctx, rows, RunEntry(0, 0, 0, True, more=tuple(more)))


# heads, kv_heads, dim, vdim, temperature (coef, every): values wider and narrower than keys, one head, the head size of the
# fast kernels, groups of four, a temperature that steps at every position and one that never steps within the sequence
@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", [(4, 2, 16, 24, (0.3, 5)), (2, 1, 32, 16, None), (3, 3, 16, 16, (0.4, 1)), (8, 2, 64, 64, (0.5, 16)),
                                   (1, 1, 40, 8, (0.7, 1000)), (6, 3, 64, 128, (0.25, 7))])
def test_softmax_side_alone(device, dtype, shape):
    dt = getattr(torch, dtype)
    D, T = 48, 41
    m = left_side(*shape[:4], temp=shape[4])
    weights = softmax_weights(D, m, seed=10)
    mixer, specs = softmax_part(D, m, weights, device, dt)
    h = randn(T, D, seed=11)
    want = plain.softmax_attention(h.to(F64), as64(weights), "", m, 1e-5)
    for cuts in ([T], [1] * T, [7, 2, 19, 2, 1, 10], [2, 37, 2], [1, 1, 2, 1, 36]):
        close(drive(run_mixer(mixer), specs, h, cuts, device, dt), want, dtype, f"softmax side {shape} cut {cuts[:5]}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("decoded", [False, True])
def test_the_temperature_steps_where_it_should(device, dtype, decoded):
    """A strong temperature that steps every 7 positions; keys whose scores are sharp enough that a step taken one position
    early or late moves the output: positions 5, 6 (the first step: (p + 1) / 7 reaches 1 at p = 6), 12, 13 and 20 are decoded
    alone or stand at the start and the end of portions."""
    dt = getattr(torch, dtype)
    D, T = 32, 24
    m = left_side(2, 1, 16, 16, scale=1.5, temp=(3.0, 7))
    weights = softmax_weights(D, m, seed=40)
    mixer, specs = softmax_part(D, m, weights, device, dt)
    h = randn(T, D, seed=41)
    want = plain.softmax_attention(h.to(F64), as64(weights), "", m, 1e-5)
    # the oracle itself tells an early step from a right one at the edges
    for p, (a, b) in {5: (6, 7), 6: (7, 8), 12: (13, 14), 13: (14, 15)}.items():
        t_right = plain.query_temperature(torch.tensor([p]), 3.0, 7)
        t_early = plain.query_temperature(torch.tensor([p + 1]), 3.0, 7)
        assert (a // 7 == b // 7) == bool(torch.equal(t_right, t_early))
    cuts = [5, 1, 1, 5, 1, 1, 6, 1, 3] if decoded else [6, 7, 2, 5, 2, 2]
    close(drive(run_mixer(mixer), specs, h, cuts, device, dt), want, dtype, "temperature steps")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("decoded", [False, True])
def test_a_far_key_among_hundreds(device, dtype, decoded):
    """Queries and keys read channels 0..15 of the input, head by head the same; the key at position 3 of 700 has the direction
    of the last query behind a scale that lets it stand out: it decides the output through portions, pages and single tokens."""
    dt = getattr(torch, dtype)
    D, T = 32, 700
    m = left_side(4, 2, 16, 16, scale=6.0)
    weights = softmax_weights(D, m, seed=30)
    weights["q.norm"][:] = 1.0
    weights["k.norm"][:] = 1.0
    for name in ("q", "k"):
        weights[name][:] = 0.0
        for head in range(weights[name].shape[0] // 16):
            weights[name][head * 16:(head + 1) * 16, :16] = torch.eye(16)
    mixer, specs = softmax_part(D, m, weights, device, dt)
    h = randn(T, D, seed=31)
    direction = randn(16, seed=32)
    h[3, :16] = direction
    h[-1, :16] = direction
    want = plain.softmax_attention(h.to(F64), as64(weights), "", m, 1e-5)
    blind = h.clone()
    blind[3, :16] = -direction
    assert (plain.softmax_attention(blind.to(F64), as64(weights), "", m, 1e-5)[-1] - want[-1]).abs().max() > 0.2 * want[-1].abs().max()
    cuts = [300, 399, 1] if decoded else [2, 330, 366, 2]
    close(drive(run_mixer(mixer), specs, h, cuts, device, dt, page=16, pages=64), want, dtype, "far key")


def retention_weights(D, m, seed):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    return {"q": randn(H * d, D, seed=seed, scale=D ** -0.5), "k": randn(H * d, D, seed=seed + 1, scale=D ** -0.5),
            "v": randn(H * dv, D, seed=seed + 2, scale=D ** -0.5), "g": randn(H * dv, D, seed=seed + 3, scale=D ** -0.5),
            "o": randn(D, H * dv, seed=seed + 4, scale=(H * dv) ** -0.5)}


PLAIN_NAMES = {"qkvg.weight": ["q", "k", "v", "g"], "o.weight": ["o"]}


def retention_spec(D, m, eps=1e-5):
    rot = m.get("rot") or {"base": 10000.0, "dims": 0}
    return PartSpec("retention", {"hidden_size": D, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "decay": m["decay"],
                                  "rot_base": rot["base"], "rot_dims": rot["dims"], "eps": eps})


def retention_part(D, m, weights, device, dt, eps=1e-5):
    mixer = build_part("mixer", retention_spec(D, m, eps))
    bind_by_checkpoint_names(mixer, weights, PLAIN_NAMES, device, dt)
    need = mixer.cache_need()
    return mixer, [CacheGroupSpec("state", "state", slots=1, state_shape=need["state_shape"], state_dtype=need["state_dtype"])]


# heads, dim, vdim, decays, rot_dims: values narrower and wider than keys, no rotation, a whole head and part of a head rotated,
# one head, a decay of exactly 1 and a fast one, sizes that are no multiples of four or eight, a head of 128
@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", [(3, 16, 8, [0.9, 0.95, 0.99], 8), (2, 24, 40, [0.5, 0.999], 0), (1, 12, 12, [0.97], 12),
                                   (5, 8, 12, [0.9, 0.92, 0.94, 0.96, 1.0], 8), (2, 64, 64, [0.97, 0.999], 32), (6, 64, 16, [0.98] * 6, 48),
                                   (2, 20, 6, [0.8, 0.99], 10), (1, 128, 72, [0.995], 64), (3, 36, 130, [0.9, 0.99, 0.999], 36)])
def test_retention_alone(device, dtype, shape):
    """Whole, token by token and in portions down to two tokens: the state is carried by the seat, in float32."""
    dt = getattr(torch, dtype)
    D, T = 48, 45
    m = right_side(*shape[:4], rot_dims=shape[4], base=300.0)
    weights = retention_weights(D, m, seed=50)
    mixer, specs = retention_part(D, m, weights, device, dt)
    h = randn(T, D, seed=51)
    want = plain.retention(h.to(F64), as64(weights), "", m, 1e-5)
    for cuts in ([T], [1] * T, [7, 2, 19, 2, 1, 14], [2, 41, 2], [1, 1, 2, 1, 40]):
        close(drive(run_mixer(mixer), specs, h, cuts, device, dt), want, dtype, f"retention {shape} cut {cuts[:5]}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("cuts", [[700], [2, 330, 366, 2], [300, 380] + [1] * 20, [64, 64, 128, 256, 187, 1]])
def test_retention_remembers_over_hundreds_of_tokens(device, dtype, cuts):
    """Decays near 1 and one token whose key is far larger than the others': what it wrote into the state decides the output
    hundreds of tokens later, whereas under the fast decay of the third head it is gone.  A state that is lost, zeroed, decayed
    once too often or mixed up between seats shows at once; so do long portions (blocks of tokens on the device)."""
    dt = getattr(torch, dtype)
    D, T = 32, 700
    m = right_side(3, 16, 16, [1.0, 0.998, 0.9], rot_dims=8, base=100.0)
    weights = retention_weights(D, m, seed=60)
    weights["q"][:, 0] = 0.0
    weights["k"][:, 0] = bf16_exact(torch.full((3 * 16,), 2.0))              # channel 0 of the input drives every key entry
    mixer, specs = retention_part(D, m, weights, device, dt)
    h = randn(T, D, seed=61, scale=0.2)
    h[:, 0] = 0.0
    h[3, 0] = 8.0
    want = plain.retention(h.to(F64), as64(weights), "", m, 1e-5)
    silent = h.clone()
    silent[3, 0] = 0.0
    other = plain.retention(silent.to(F64), as64(weights), "", m, 1e-5)
    assert (other[-1] - want[-1]).abs().max() > 0.3 * want[-1].abs().max()
    # bfloat16: a head whose sum nearly cancels is divided by its own small size; a lost state would move every late row by far more
    close(drive(run_mixer(mixer), specs, h, cuts, device, dt, page=16, pages=64), want, dtype, "far memory", bars=(1e-4, 0.2))


@pytest.mark.parametrize("device,dtype", CASES)
def test_retention_over_a_portion_of_thousands_of_tokens(device, dtype):
    dt = getattr(torch, dtype)
    D, T = 16, 2300
    m = right_side(2, 16, 24, [0.999, 0.97], rot_dims=16, base=10000.0)
    weights = retention_weights(D, m, seed=70)
    mixer, specs = retention_part(D, m, weights, device, dt)
    h = randn(T, D, seed=71)
    want = plain.retention(h.to(F64), as64(weights), "", m, 1e-5)
    got = drive(run_mixer(mixer), specs, h, [2200, 98, 1, 1], device, dt, page=16, pages=160)
    close(got, want, dtype, "a long portion", bars=(1e-4, 0.1))


@pytest.mark.gpu
@pytest.mark.parametrize("value_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,decay", [(2, 64, 128, [0.97, 1.0]), (3, 24, 40, [0.5, 0.999, 0.9]), (1, 130, 72, [0.99]),
                                                   (2, 72, 200, [0.0, 0.98])])
def test_recurrence_in_blocks_of_tokens_against_the_walk(value_dtype, heads, dim, vdim, decay):
    """The kernels that sum blocks of tokens side by side and chain them, against the recurrence written out token by token:
    portions of one token, one token less and more than a block, several blocks and a ragged last one in ONE step; a seat that
    already holds a state, a fresh one, a request without a seat; key and value sizes that are no multiples of a tile; a decay
    of exactly one and of exactly zero."""
    import flexengine_b200.ops as ops
    device = "cuda:0"
    lengths = [1, 63, 64, 65, 333, 130]
    seats = [2, 0, -1, 5, 1, 4]
    T, per = sum(lengths), heads * dim * vdim
    g = torch.Generator().manual_seed(7)
    qk = torch.randn(T, 2 * heads * dim, generator=g) * dim ** -0.25
    projected = (torch.randn(T, heads * vdim + 9, generator=g)).to(getattr(torch, value_dtype))
    values = projected[:, 4:4 + heads * vdim]                                  # a view with a row stride of its own
    state = torch.randn(6, per + 3, generator=g)
    w = torch.tensor(decay, dtype=torch.float32)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
    slots = torch.tensor(seats, dtype=torch.int32)
    want_state = state.clone()
    want = kernel_refs.retention_scan(qk, values, w, want_state, slots, cu, heads, dim, vdim)
    dev = [t.to(device) for t in (qk, projected, w, state, slots, cu)]
    got_state = dev[3]
    got = ops.retention_scan(dev[0], dev[1][:, 4:4 + heads * vdim], dev[2], got_state, dev[4], dev[5], heads, dim, vdim, max_q_len=max(lengths))
    scale = want.abs().max()
    assert (got.cpu() - want).abs().max() <= 2e-5 * scale
    assert (got_state.cpu() - want_state).abs().max() <= 2e-5 * want_state.abs().max()
    # and the walk itself, which a step of short portions takes
    walked_state = state.to(device)
    walked = ops.retention_scan(dev[0], dev[1][:, 4:4 + heads * vdim], dev[2], walked_state, dev[4], dev[5], heads, dim, vdim, max_q_len=1)
    assert (walked.cpu() - want).abs().max() <= 2e-5 * scale and (walked_state.cpu() - want_state).abs().max() <= 2e-5 * want_state.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,decay,rot", [(2, 64, 128, [0.97, 1.0], 32), (3, 24, 40, [0.5, 0.999, 0.9], 24), (1, 130, 72, [0.99], 0),
                                                      (2, 10, 300, [0.0, 0.98], 4), (5, 8, 6, [0.9] * 5, 8)])
def test_one_token_a_request_in_one_kernel(dtype, heads, dim, vdim, decay, rot):
    """The decode kernel (rotation, recurrence, head norm, gate) against the three reference operations one after the other:
    kept and absent seats, rows and destination inside wider buffers, sizes that are multiples of nothing, an output scale."""
    import flexengine_b200.ops as ops
    device, dt = "cuda:0", getattr(torch, dtype)
    R, per, inner = 7, heads * dim * vdim, heads * vdim
    g = torch.Generator().manual_seed(9)
    projected = (torch.randn(R, 2 * heads * dim + 2 * inner + 5, generator=g) * 0.7).to(dt)
    state = torch.randn(9, per + 2, generator=g)
    seats = torch.tensor([3, -1, 0, 8, 5, -1, 1], dtype=torch.int32)
    positions = torch.tensor([0, 1, 77, 1000, 12345, 3, 64], dtype=torch.int32)
    w = torch.tensor(decay, dtype=torch.float32)
    inv_freq = None
    if rot:
        inv_freq = torch.pow(torch.tensor(10000.0, dtype=F64), -2.0 * torch.arange(rot // 2, dtype=F64) / rot).float()
    want_state = state.clone()
    want = kernel_refs.retention_decode(projected, heads, dim, vdim, positions, inv_freq, rot, dim ** -0.5, w, want_state, seats, 1e-6,
                                        torch.float32 if dtype == "float32" else dt, scale=1.3)
    wide = torch.zeros(R, inner + 11, dtype=dt, device=device)
    got_state = state.to(device)
    ops.retention_decode(projected.to(device), heads, dim, vdim, positions.to(device), None if inv_freq is None else inv_freq.to(device), rot,
                         dim ** -0.5, w.to(device), got_state, seats.to(device), 1e-6, dt, scale=1.3, into=wide[:, 3:3 + inner])
    assert (got_state.cpu() - want_state).abs().max() <= 2e-6 * want_state.abs().max()
    bar = 2e-5 if dtype == "float32" else 1.6e-2
    assert (wide[:, 3:3 + inner].float().cpu() - want.float()).abs().max() <= bar * want.float().abs().max()
    assert float(wide[:, :3].abs().max()) == 0.0 and float(wide[:, 3 + inner:].abs().max()) == 0.0


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", [((4, 2, 16, 24, (0.3, 5)), (3, 16, 8, [0.9, 0.95, 0.99], 8), 1.2, 0.9),
                                   ((1, 1, 48, 40, None), (1, 40, 24, [0.98], 20), 1.0, 0.5),
                                   ((8, 2, 64, 64, (0.5, 32)), (2, 64, 64, [0.97, 0.999], 32), 0.0, 1.0),
                                   ((4, 4, 64, 32, None), (4, 32, 48, [0.9, 0.95, 0.99, 0.995], 32), 1.1, 0.0)])
def test_two_mixers_side_by_side(device, dtype, shape):
    """One product for both sides' projections, one for both outputs: against the weighted sum of the two mixers, also with
    a weight of zero on either side."""
    dt = getattr(torch, dtype)
    D, T = 56, 37
    left, right = left_side(*shape[0][:4], temp=shape[0][4]), right_side(*shape[1][:4], rot_dims=shape[1][4], base=500.0)
    m = parallel(left, right, shape[2], shape[3])["mixer"]
    weights = {"left." + k: v for k, v in softmax_weights(D, left, seed=80).items()}
    weights.update({"right." + k: v for k, v in retention_weights(D, right, seed=90).items()})
    mixer = build_part("mixer", PartSpec("parallel", {"hidden_size": D, "sides": (
        ("left", softmax_spec(D, left), shape[2]), ("right", retention_spec(D, right), shape[3]))}))
    names = {f"left.{k}": [f"left.{n}" for n in v] for k, v in SOFTMAX_NAMES.items()}
    names.update({f"right.{k}": [f"right.{n}" for n in v] for k, v in PLAIN_NAMES.items()})
    bind_by_checkpoint_names(mixer, weights, names, device, dt)
    needs = mixer.cache_need()
    specs = [CacheGroupSpec("rows", needs[0]["kind"], slots=1, kv_heads=needs[0]["kv_heads"], head_dim=needs[0]["head_dim"], window=needs[0]["window"]),
             CacheGroupSpec("state", "state", slots=1, state_shape=needs[1]["state_shape"], state_dtype=needs[1]["state_dtype"])]
    h = randn(T, D, seed=99)
    want = plain.parallel_mixer(h.to(F64), as64(weights), "", m, 1e-5)
    for cuts in ([T], [30] + [1] * 7, [7, 2, 19, 2, 1, 6]):
        close(drive(run_mixer(mixer, more=((1, 0),)), specs, h, cuts, device, dt), want, dtype, f"side by side cut {cuts[:4]}")


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("sizes", [(48, 72), (40, 100), (64, 256)])
def test_dense_feed_forward_with_biases_alone(device, dtype, sizes):
    dt = getattr(torch, dtype)
    D, F = sizes
    T = 13
    weights = {"gate": randn(F, D, seed=1, scale=D ** -0.5), "up": randn(F, D, seed=2, scale=D ** -0.5), "down": randn(D, F, seed=3, scale=F ** -0.5),
               "gate.b": randn(F, seed=4), "up.b": randn(F, seed=5), "down.b": randn(D, seed=6)}
    part = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": F, "activation": "silu", "bias": True}))
    bind_by_checkpoint_names(part, weights, {"gate_up.weight": ["gate", "up"], "gate_up.bias": ["gate.b", "up.b"], "down.weight": ["down"],
                                             "down.bias": ["down.b"]}, device, dt)
    h = randn(T, D, seed=7, scale=2.0)
    ctx = simple_ctx(device, dt)
    want = plain.dense_feed_forward(h.to(F64), as64(weights), "")
    for rows in (T, 1):
        got = part.forward(ctx, h[:rows].to(device=device, dtype=dt).contiguous())
        close(got, want[:rows], dtype, f"dense feed-forward, {rows} rows", bars=(2e-5, 4e-2))
        # the last bias left to the norm that follows: rows in float32 and the bias beside them
        late, bias = part.forward(ctx, h[:rows].to(device=device, dtype=dt).contiguous(), defer_bias=True)
        assert late.dtype == torch.float32
        close(late + bias, want[:rows], dtype, "bias deferred", bars=(2e-5, 4e-2))


# experts, top, size, limit: all experts chosen, one chosen, a limit that cuts most products and one that cuts none
@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("shape", [(6, 2, 24, 1.5), (3, 3, 40, 0.8), (5, 1, 56, 3.0), (16, 4, 64, 0.3), (8, 3, 32, 100.0), (1, 1, 16, 1.0)])
def test_routed_feed_forward_alone(device, dtype, shape):
    """The largest logits are chosen, the weights are the softmax over the chosen; gate products cut off above the limit, up
    products on both sides.  Router logits apart by design: row t prefers experts t, t + 1, ... in steps of 0.5."""
    dt = getattr(torch, dtype)
    E, top, F, limit = shape
    D, T = 48, 29
    weights = {"router": torch.zeros(E, D)}
    for e in range(E):
        weights.update({f"e{e}.gate": randn(F, D, seed=10 + 3 * e, scale=2 * D ** -0.5), f"e{e}.up": randn(F, D, seed=11 + 3 * e, scale=2 * D ** -0.5),
                        f"e{e}.down": randn(D, F, seed=12 + 3 * e, scale=F ** -0.5)})
        weights["router"][e, e] = 1.0                                         # channel e of the input is expert e's logit
    part = build_part("feed_forward", PartSpec("routed_experts", {"hidden_size": D, "experts": E, "top": top, "expert_size": F,
                                                                  "router": "softmax_chosen", "activation": "clamped", "limit": limit}))
    names = {"router.weight": ["router"], "experts.gate_up.weight": [f"e{e}.{w}" for e in range(E) for w in ("gate", "up")],
             "experts.down.weight": [f"e{e}.down" for e in range(E)]}
    bind_by_checkpoint_names(part, weights, names, device, dt)
    h = randn(T, D, seed=8)
    for t in range(T):
        for e in range(E):
            h[t, e] = -0.5 * ((e - t) % E)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": F, "limit": limit}}
    gaps = []
    want = plain.routed_feed_forward(h.to(F64), as64(weights), "", mlp, gaps)
    assert not gaps or float(gaps[0].min()) > 0.4
    ctx = simple_ctx(device, dt)
    for rows in (T, 1, 3):
        got = part.forward(ctx, h[:rows].to(device=device, dtype=dt).contiguous())
        close(got, want[:rows], dtype, f"routed feed-forward {shape}, {rows} rows", bars=(2e-5, 5e-2))


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("width", [40, 66])
def test_pass_junction_alone(device, dtype, width):
    """x <- W [x; x0] after what the block before left pending is settled; the origin is not touched."""
    from flexengine_b200.parts.junction import Reinject
    dt = getattr(torch, dtype)
    D, T, eps = width, 9, 1e-5
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(1))
    x0 = torch.randn(T, D, generator=torch.Generator().manual_seed(2))
    y, w_branch, w = randn(T, D, seed=3), randn(D, seed=4) + 1.0, randn(D, 2 * D, seed=5, scale=(2 * D) ** -0.5)
    part = build_part("junction", PartSpec("reinject", {"hidden_size": D}))
    assert isinstance(part, Reinject)
    part.bind({"weight": w.to(device=device, dtype=dt)})
    ctx = simple_ctx(device, dt)
    for pending in (None, PostNormed(y.to(device), w_branch.to(device), eps)):
        settled = x.to(F64) if pending is None else x.to(F64) + plain.rms_norm(y.to(F64), eps, w_branch.to(F64))
        want = torch.cat([settled, x0.to(F64)], dim=-1) @ w.to(F64).T
        origin = x0.clone().to(device)
        got = part.forward(ctx, x.clone().to(device), pending, origin)
        assert got.dtype == torch.float32 and torch.equal(origin.cpu(), x0)
        close(got, want, dtype, "junction", bars=(2e-5, 3e-2))


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("scale,cap", [(2.0, 30.0), (0.5, 0.0), (1.0, 2.0), (7.0, 1.0)])
def test_squashed_head_alone(device, dtype, scale, cap):
    dt = getattr(torch, dtype)
    V, D, T = 131, 40, 6
    w, h = randn(V, D, seed=1), randn(T, D, seed=2)
    head = build_part("head", PartSpec("linear", {"vocab_size": V, "hidden_size": D, "scale": scale, "softcap": cap}))
    head.bind({"weight": w.to(device=device, dtype=dt)})
    logits = h.to(F64) @ w.to(F64).T * scale
    want = cap * torch.tanh(logits / cap) if cap else logits
    got = head.forward(simple_ctx(device, dt), h.to(device=device, dtype=dt))
    assert got.dtype == torch.float32
    close(got, want, dtype, "head", bars=(2e-5, 3e-2))


# ---- the whole model under every way of cutting the work ---------------------------------------------------------------
def scenario(kind, requests, rng):
    if kind == "whole":
        return helpers.steps_whole(requests)
    if kind == "last_decoded":
        return helpers.steps_last_decoded(requests, tail=20)
    if kind == "portions":
        return helpers.steps_portions(requests, rng, sizes=(24, 7, 2, 13, 2, 31, 3, 64, 5))
    doubled = dict(requests)
    doubled.update({rid + "x": ids[::-1] for rid, ids in requests.items()})     # more requests than seats: seats are used again
    return helpers.steps_mixed(doubled, rng, live=4)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("kind", ["whole", "last_decoded", "portions", "mixed"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
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
    """The residual stream after every run of a layer, with what is pending put in: the plain implementation's, run by run."""
    for name in ("P", "R"):
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
        origin, pending = residual.clone(), None
        assert len(plan.run) == len(after)
        for at, entry in enumerate(plan.run):
            if entry.before >= 0:
                residual, pending = model.junctions[entry.before].forward(ctx, residual, pending, origin), None
            pending = model.blocks[entry.layer].forward(ctx, residual, pending, entry)
            settled = residual.double() + plain.rms_norm(pending.y.double() + (0.0 if pending.bias is None else pending.bias.double()),
                                                         pending.eps, pending.weight.double())
            assert (settled - after[at]).abs().max() < 2e-5 * float(after[at].abs().max()), f"{name}: run {at}"


STACKS = {
    "one layer that is the whole repeated span": config(50, 32, 1e-5, 1.0, [
        (parallel(left_side(2, 1, 16, 16), right_side(2, 8, 8, [0.9, 0.99], 4)), None)], loop=(0, 1, 3)),
    "a span that runs once": config(97, 48, 1e-5, 0.5, [
        (parallel(left_side(2, 2, 16, 8, temp=(0.2, 3)), right_side(1, 16, 32, [0.95])), dense(32)),
        (parallel(left_side(3, 1, 8, 24), right_side(4, 8, 4, [0.5, 0.9, 0.99, 1.0], 8), 2.0, 0.1), moe(4, 4, 16, 0.5))], loop=(1, 2, 1)),
    "every layer without a feed-forward": config(64, 40, 1e-6, 4.0, [
        (parallel(left_side(5, 5, 8, 8), right_side(2, 16, 16, [0.9, 0.8], 16)), None),
        (parallel(left_side(1, 1, 24, 16, temp=(2.0, 2)), right_side(1, 8, 40, [0.99], 2)), None)], loop=(0, 2, 2), logit_scale=3.0, softcap=5.0),
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
    name = "P"
    requests = requests_for(name, seed=9)
    together = make_runner(model_dirs[name], dtype, device, 16, PAGE[name])
    logits = together.step([StepEntry(rid, ids, [len(ids) - 1]) for rid, ids in requests.items()][:4])
    for row, (rid, ids) in enumerate(list(requests.items())[:4]):
        alone = make_runner(model_dirs[name], dtype, device, 8, PAGE[name])
        close(logits[row:row + 1], alone.step([StepEntry(rid, ids, [len(ids) - 1])]), dtype, rid)


@pytest.mark.parametrize("device,dtype", CASES)
def test_first_tokens_and_long_decoding(model_dirs, device, dtype):
    """A prompt of one token, then 150 tokens decoded one by one beside a neighbour that arrives later and leaves: every row
    against the whole sequence.  The temperature steps 30 times, pages fill and the states of all passes are carried."""
    name = "P"
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
    name = "Q"
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
    name = "P"
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
