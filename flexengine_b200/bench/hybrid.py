"""``--workload fuvozen|fuvuvik|fedutar|rikolix``: prefill and decode throughput of one of these designs at a few sizes that resemble a
real model's layers (random weights), beside the closest existing model at equal width, depth and vocabulary (a Qwen2
decoder; for Fedutar the Fuvozen design, which also has a recurrence with a matrix state and routed experts; for Rikolix the
Fuvozen design too, which also has attention over a cached latent, routed experts and a dense feed-forward without a gate), and, at one size, an
operation-by-operation table of both: time, the bytes and flops of the work, and how far each operation is from the
roofline of the measured peaks (time / max(bytes / copy rate, flops / bf16 rate)).

Prefill is one 2,048-token prompt in one step; decode is batch 8 at 2,048 cached tokens, replayed from a CUDA graph.
The table times every call of the kernel provider with CUDA events around it (a synchronize on both sides), in a
prefill step and in a decode step run kernel by kernel.
"""
from __future__ import annotations

import json

from .clocks import ClockSampler, load_peaks
from .timing import Timer

PROMPT, CONTEXT, PAGE, BATCH = 2048, 4096, 16, 8


def fuvozen_config(width, layers, vocab, heads, experts=8, top=2):
    """Alternating layers: the recurrence beside a dense feed-forward, then latent attention beside routed experts.
    Recurrent heads of 64; attention heads of 64 + 64 rotated over a latent of 64 (a cached row of 128)."""
    stack = []
    for i in range(layers):
        if i % 2 == 0:
            stack.append({"type": "wkv", "mixer": {"heads": width // 64, "dim": 64}, "mlp": {"kind": "dense", "ff": 4 * width}})
        else:
            stack.append({"type": "latent_attention",
                          "mixer": {"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 64, "kv_rank": 64, "mask": {"size": 1024},
                                    "rot": {"base": 10000.0, "dims": 64}, "scale": 128 ** -0.5},
                          "mlp": {"kind": "moe", "expert": {"ff": width}, "router": {"experts": experts, "top": top, "scale": 1.0},
                                  "shared": {"ff": width}}})
    return {"architecture": "Fuvozen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 2},
            "embedding": {"bigram": {"buckets": 100003, "mul_prev": 31, "mul_cur": 7}}, "layers": stack}


def fuvuvik_config(width, layers, vocab, heads):
    """Layers in turns of four: attention with convolutions of four taps, two minGRU recurrences of 1.5 x width, attention in
    chunks of 1,024 with a sink; heads of 128 in groups of four, half of a head rotated in the first kind; two residual
    streams; a gated feed-forward of 2 x width, which with the two residual gates of a layer holds the 8 width^2 of the
    Qwen2 decoder's feed-forward beside it."""
    stack = []
    for i in range(layers):
        turn = i % 4
        if turn == 0:
            mixer = {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "conv": 4,
                                                    "rot": {"base": 10000.0, "dims": 64}, "scale": 128 ** -0.5}}
        elif turn == 3:
            mixer = {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128,
                                                      "mask": {"size": 1024}, "rot": {"base": 500000.0, "dims": 128}, "scale": 128 ** -0.5}}
        else:
            mixer = {"type": "mingru", "mixer": {"width": width * 3 // 2}}
        stack.append(dict(mixer, mlp={"kind": "dense", "ff": 2 * width}))
    return {"architecture": "Fuvuvik", "vocab": vocab, "width": width, "streams": 2, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": stack}


def fedutar_config(width, layers, vocab, heads):
    """``layers`` runs of a layer: the first two layers run twice in a row (a junction before each pass), the others once.
    Every layer has softmax attention (heads of 128 in groups of four, a query temperature that steps every 512 positions)
    beside retention (width / 128 heads of 64 x 128, half of a head rotated); feed-forwards in turns: dense of 2.5 x width
    with biases, then 8 experts of 1.25 x width of which a token uses 2.  A layer run multiplies a token by about
    15 width^2 weights, as a Fuvozen layer does on average."""
    distinct = max(2, layers - 2)
    r_heads = max(1, width // 128)
    stack = []
    for i in range(distinct):
        mixer = {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                          "q_temp": {"coef": 0.1, "every": 512}},
                 "right": {"heads": r_heads, "dim": 64, "vdim": 128, "decay": [1.0 - 2.0 ** -(5 + h % 6) for h in range(r_heads)],
                           "rot": {"base": 10000.0, "dims": 32}},
                 "left_scale": 1.0, "right_scale": 1.0}
        mlp = {"kind": "dense", "ff": width * 5 // 2} if i % 2 == 0 else \
            {"kind": "moe", "expert": {"ff": width * 5 // 4, "limit": 7.0}, "router": {"experts": 8, "top": 2}}
        stack.append({"type": "parallel", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Fedutar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "logit_softcap": 30.0, "loop": {"start": 0, "stop": 2, "times": 2}, "layers": stack}


def rikolix_config(width, layers, vocab, heads):
    """Layers in turns of four: sigmoid attention (heads of 128 in groups of four, half of a head rotated, values that turn)
    beside a dense feed-forward of 4 x width; latent attention that makes its latents (heads of 64 + 64 rotated over a latent
    of 64, a cached row of 128 as in the Fuvozen model beside it; queries through a latent of width / 2) beside 8 experts of
    ``width`` and 2 that return their input, in two groups of which one is kept, two chosen; latent attention that reads
    those latents beside a dense feed-forward; latent attention of its own beside experts again."""
    stack = []
    latent = {"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 64, "kv_rank": 64, "q_rank": width // 2,
              "rot": {"base": 10000.0, "dims": 64}, "scale": 128 ** -0.5}
    moe = {"kind": "moe", "expert": {"ff": width}, "router": {"experts": 8, "identity": 2, "top": 2, "groups": {"count": 2, "keep": 1}}}
    for i in range(layers):
        turn = i % 4
        if turn == 0:
            stack.append({"type": "attention",
                          "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                    "rot": {"base": 500000.0, "dims": 64}},
                          "mlp": {"kind": "dense", "ff": 4 * width}})
        elif turn == 2:
            stack.append({"type": "latent_attention", "mixer": dict(latent, kv_from=i - 1), "mlp": {"kind": "dense", "ff": 4 * width}})
        else:
            stack.append({"type": "latent_attention", "mixer": dict(latent), "mlp": moe})
    return {"architecture": "Rikolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": stack}


DESIGNS = {"fuvozen": ("Fuvozen", fuvozen_config), "fuvuvik": ("Fuvuvik", fuvuvik_config), "fedutar": ("Fedutar", fedutar_config),
           "rikolix": ("Rikolix", rikolix_config)}


def qwen2_config(width, layers, vocab, heads):
    """The closest existing model at equal size: grouped-query attention with heads of 128 and a SwiGLU feed-forward
    whose three matrices hold what a Fuvozen layer's feed-forward uses per token on average (about 8 width^2)."""
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=layers, hidden_size=width,
                num_attention_heads=heads, num_key_value_heads=max(1, heads // 4), head_dim=128,
                intermediate_size=width * 8 // 3 // 256 * 256, vocab_size=vocab, rope_theta=1000000.0, rms_norm_eps=1e-6,
                max_position_embeddings=32768, tie_word_embeddings=True, use_sliding_window=False, hidden_act="silu", eos_token_id=None)


# the model a design is measured beside (default: the Qwen2 decoder)
BESIDE = {"fedutar": ("fuvozen", "Fuvozen", fuvozen_config), "rikolix": ("fuvozen", "Fuvozen", fuvozen_config)}

SIZES = {"1k": (1024, 8, 32000, 8), "2k": (2048, 8, 32000, 16), "4k": (4096, 4, 32000, 32)}


class TimedOps:
    """A kernel provider that forwards to ``ops`` and keeps, per operation, the device time of its calls (CUDA events,
    a synchronize on both sides) and the bytes of the tensors that go in and come out."""

    def __init__(self, ops, torch):
        self._ops, self._torch = ops, torch
        self.rows = {}

    def __getattr__(self, name):
        if name == "native_layers_usable":             # every operation on its own: no layer as one call
            raise AttributeError(name)
        target = getattr(self._ops, name)
        if not callable(target) or isinstance(target, type) or name in ("check_status", "status_word", "sm_count", "scratch"):
            return target
        torch = self._torch

        def timed(*args, **kwargs):
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = target(*args, **kwargs)
            end.record()
            torch.cuda.synchronize()
            tensors = [a for a in list(args) + list(kwargs.values()) if torch.is_tensor(a)]
            tensors += [o for o in (out if isinstance(out, (tuple, list)) else [out]) if torch.is_tensor(o)]
            seen, nbytes = set(), 0
            for t in tensors:
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    nbytes += t.numel() * t.element_size()
            flops = 0.0
            if name in ("linear", "linear_swiglu", "linear_gated", "linear_activated") and len(args) >= 2:
                flops = 2.0 * args[0].shape[0] * args[1].shape[0] * args[1].shape[1]
            elif name == "batched_linear":
                flops = 2.0 * args[0].shape[0] * args[0].shape[1] * args[0].shape[2] * args[1].shape[1]
            elif name == "routed_experts":
                pairs = args[1].numel()
                if kwargs.get("activation") == "relu2":           # experts without a gate: one matrix up, one down
                    flops = 2.0 * pairs * 2 * args[3].shape[1] * args[3].shape[2]
                else:
                    flops = 2.0 * pairs * 3 * (args[3].shape[1] // 2) * args[3].shape[2]
                used = min(args[3].shape[0], pairs)
                nbytes = nbytes - (args[3].numel() + args[4].numel()) * 2 * (1 - used / args[3].shape[0])
            elif name in ("paged_attention",):
                ctx, nq, d = args[4], args[5], args[7]
                window = args[10]                 # w > 0: the last w keys; -c < 0: the keys of the query's chunk of c positions
                sees = lambda p: (min(p + 1, window) if window > 0 else (p % -window + 1 if window < 0 else p + 1))
                pairs = 0
                for s, n in zip(ctx.host_starts, ctx.host_lengths):
                    if window < 0:
                        pairs += sum(sees(p) for p in range(s, s + n))
                    else:
                        pairs += (sees(s) + sees(s + n - 1)) * n / 2.0
                flops = 4.0 * nq * d * pairs
                page, kv = args[8], args[6]
                reach = abs(window)
                keys = sum(min(s + n, (reach + n) if reach else s + n) for s, n in zip(ctx.host_starts, ctx.host_lengths))
                nbytes = args[0].numel() * 2 + 2 * args[0].shape[0] * nq * d + keys * kv * d * 2 * (1 if args[1].data_ptr() == args[2].data_ptr() else 2)
            elif name == "wkv_recurrence":
                flops = 6.0 * args[0].shape[0] * args[9] * args[10] * args[10]
                nbytes = args[0].numel() * (3 * args[0].element_size() + 8) + 2 * 4 * (args[8].numel() - 1) * args[9] * args[10] * args[10]
            elif name == "retention_scan":
                # per token and head: the state's update and its product with the query; the state of a request read and written once
                heads, d, dv = args[6], args[7], args[8]
                tokens, requests = args[0].shape[0], args[5].numel() - 1
                flops = 4.0 * tokens * heads * d * dv
                nbytes = tokens * (2 * heads * d * 4 + heads * dv * (args[1].element_size() + 4)) + 2 * 4 * requests * heads * d * dv
            elif name == "stream_rmsnorm":
                # the streams are read, and written back when a sublayer's output goes in; its output and gate are read
                update = kwargs.get("update")
                streams = args[0].numel() * 4
                nbytes = streams * (2 if update is not None and kwargs.get("rows") is None else 1) + (out.numel() * out.element_size())
                if update is not None:
                    nbytes += update.y.numel() * update.y.element_size() * 2
                if kwargs.get("rows") is not None:
                    nbytes = nbytes * kwargs["rows"].numel() / max(1, args[0].shape[1])
            shapes = "x".join(str(tuple(a.shape)) for a in args[:2] if torch.is_tensor(a)) if name in ("linear", "linear_swiglu", "linear_gated", "linear_activated", "batched_linear") else ""
            row = self.rows.setdefault(f"{name} {shapes}".strip(), [0, 0.0, 0.0, 0.0])
            row[0] += 1
            row[1] += start.elapsed_time(end) * 1e3
            row[2] += nbytes
            row[3] += flops
            return out
        return timed

    def call_floor_us(self, repeats: int = 20) -> float:
        """What the timing itself costs a call: the device time between the events around a kernel that does next to nothing
        (an activation of two numbers), taken the same way.  An operation's time in the table includes it."""
        torch = self._torch
        tiny = torch.zeros((1, 2), dtype=torch.bfloat16, device="cuda")
        times = []
        for _ in range(repeats):
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            self._ops.gated_activation(tiny, 1, "silu")
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end) * 1e3)
        return round(sorted(times)[len(times) // 2], 1)

    def table(self, peaks):
        hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
        out = []
        for name, (calls, us, nbytes, flops) in sorted(self.rows.items(), key=lambda kv: -kv[1][1]):
            floor = max(nbytes / hbm, flops / tensor) * 1e6
            out.append({"op": name, "calls": calls, "us": round(us, 1), "mbytes": round(nbytes / 1e6, 1), "gflop": round(flops / 1e9, 1),
                        "roofline_us": round(floor, 1), "times_roofline": round(us / floor, 1) if floor > 0 else None})
        return out


def run(args) -> int:
    import torch
    from .. import ops
    from ..cache import CacheManager
    from ..engine import ModelRunner, StepEntry
    from ..weights import random_model

    dev = "cuda:0"
    peaks, peak_source = load_peaks(args.peaks)
    sampler = ClockSampler().start()
    timer = Timer(ops)
    gen = torch.Generator().manual_seed(1)
    results, tables = {}, {}
    sizes = [args.size] if getattr(args, "size", None) else list(SIZES)
    design, design_config = DESIGNS[args.workload]
    key = args.workload
    other, other_name, other_config = BESIDE.get(key, ("qwen2", "Qwen2", qwen2_config))

    def measure(cfg, vocab, provider=None, steps=args.steps, warmup=max(args.warmup, 3)):
        _typed, plan, model = random_model(cfg, seed=0, dtype="bfloat16", device=dev)
        cache = CacheManager(plan.cache_groups, (BATCH + 1) * CONTEXT // PAGE, PAGE, BATCH + 1, torch.bfloat16, dev)
        runner = ModelRunner(model, cache, ops=provider)
        prompt = torch.randint(0, vocab, (PROMPT,), generator=gen).tolist()

        def prefill_once(i):
            runner.step([StepEntry(f"p{i}", prompt, [PROMPT - 1])])
            runner.finish(f"p{i}")
        if provider is not None:                        # the table: one prefill step and one decode step, kernel by kernel
            prefill_once(-1)
            provider.rows.clear()
            prefill_once(0)
            prefill_table = provider.table(peaks)
            rids = [f"d{i}" for i in range(BATCH)]
            for rid in rids:
                runner.step([StepEntry(rid, prompt, [])])
            runner.step([StepEntry(rid, [1], [0]) for rid in rids])
            provider.rows.clear()
            runner.step([StepEntry(rid, [2], [0]) for rid in rids])
            return {"prefill": prefill_table, "decode": provider.table(peaks), "call_floor_us": provider.call_floor_us()}
        for w in range(3):
            prefill_once(-1 - w)
        prefill_ms, _ = timer.timed(prefill_once, 5)
        runner.enable_decode_graphs(BATCH, CONTEXT)
        rids = [f"d{i}" for i in range(BATCH)]
        for rid in rids:
            runner.step([StepEntry(rid, prompt, [])])
        feed = torch.randint(0, vocab, (warmup + steps, BATCH), generator=gen).tolist()

        def one(i, base=0):
            runner.step([StepEntry(rid, [feed[base + i][j]], [0]) for j, rid in enumerate(rids)])
        for w in range(warmup):
            one(w)
        ms, launches = timer.timed(lambda i: one(i, warmup), steps)
        ops.check_status(dev)
        weights = model.weight_bytes()
        del runner, cache, model
        torch.cuda.empty_cache()
        return {"prefill_tokens_per_s": round(PROMPT / (prefill_ms / 1e3)), "prefill_ms": round(prefill_ms, 2),
                "decode_tokens_per_s": round(BATCH / (ms / 1e3)), "decode_ms_per_step": round(ms, 3), "weight_gbytes": round(weights / 1e9, 2),
                "launches": launches}

    launches = 0
    for name in sizes:
        width, layers, vocab, heads = SIZES[name]
        results[name] = {key: measure(design_config(width, layers, vocab, heads), vocab),
                         other: measure(other_config(width, layers, vocab, heads), vocab)}
        launches += results[name][key].pop("launches") + results[name][other].pop("launches")
    if args.kernels:
        width, layers, vocab, heads = SIZES[sizes[-1] if getattr(args, "size", None) else "2k"]
        # as many layers as show every kind of layer the design has
        tables[key] = measure(design_config(width, 2 if key == "fuvozen" else 4, vocab, heads), vocab, TimedOps(ops, torch))
        tables[other] = measure(other_config(width, 2, vocab, heads), vocab, TimedOps(ops, torch))
    sampler.stop()
    first = results[sizes[0]][key]
    line = {"metric": f"decode tokens/s ({design} design, size {sizes[0]}, batch {BATCH}, {PROMPT}-token prompts)",
            "value": first["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": first["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: random token ids, random weights", "impl": "ours",
            "config": {"model": f"{design} beside {other_name} at equal width, depth and vocabulary", "sizes": {k: list(v) for k, v in SIZES.items() if k in sizes},
                       "global_batch": BATCH, "seq_len": CONTEXT, "prompt_len": PROMPT, "kv_page": PAGE, "parallelism": "single GPU",
                       "peaks": peak_source},
            "sizes": results, "gpu_launches": launches, "clocks": sampler.summary(timer.windows)}
    if tables:
        line["operations"] = tables
    print(json.dumps(line))
    return 0
