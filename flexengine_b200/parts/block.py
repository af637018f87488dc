"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

"prenorm" is the reference's decoder layer (src/flexengine/inference/models/qwen2.py:97-130):
    x = x + mixer(norm_in(x));  x = x + feed_forward(norm_post(x)).
The residual stream is float32.  A branch output is not added at once: it is handed on
as ``pending`` and added inside the next norm kernel (fused residual add + norm).
"""
from __future__ import annotations

import inspect

import torch

from .base import build_part, register_block


def _accepts(function, name: str) -> bool:
    """Whether ``function`` names the parameter (looked up once per function)."""
    cache = _accepts.__dict__.setdefault("seen", {})
    key = (getattr(function, "__func__", function), name)
    if key not in cache:
        cache[key] = name in inspect.signature(function).parameters
    return cache[key]


class PreNormBlock:
    part_names = ("input_norm", "mixer", "post_mixer_norm", "feed_forward")
    takes_prenormed = True          # ``pending`` may be rows on their way through this block's input norm

    def __init__(self, layer_spec):
        self.input_norm = build_part("norm", layer_spec.norm)
        self.post_mixer_norm = build_part("norm", layer_spec.norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward)

    def parts(self) -> dict:
        return {name: getattr(self, name) for name in self.part_names}

    def forward(self, ctx, residual, pending, entry, next_norm=None, next_reads=None):
        """``next_norm``: the norm that will read the residual after this block (the next block's input norm), when
        the model knows it: the feed-forward may then begin it (see ``parts.base``, "a norm that follows").
        ``next_reads``: the matrix the next block streams first."""
        if getattr(ctx.ops, "native_layers_usable", None) is not None and ctx.ops.native_layers_usable(ctx):
            done = self._native_forward(ctx, residual, pending, entry)
            if done is not None:
                return done
        h = self._normed(self.input_norm, ctx, residual, pending, self.mixer)
        mixed = self._branch(self.mixer, (ctx, h, entry), ctx, residual, self.post_mixer_norm, self.feed_forward.reads_first())
        h = self._normed(self.post_mixer_norm, ctx, residual, mixed, self.feed_forward)
        return self._branch(self.feed_forward, (ctx, h), ctx, residual, next_norm, next_reads)

    def _native_forward(self, ctx, residual, pending, entry):
        """The whole layer as one call into the kernel library (a step of more than a handful of tokens, outside graph
        capture), when its parts are the ones that call is written for; None otherwise."""
        ops = ctx.ops
        layer = self.__dict__.get("_native")
        if layer is None:
            layer = self._native = self._native_layer(ctx) or False
        group = ctx.groups[entry.cache_group]
        if (layer is False or (pending is not None and not torch.is_tensor(pending)) or group.kind not in ("full", "window")
                or group.storage.dtype != torch.bfloat16):
            return None
        steps = ctx.__dict__.setdefault("_native_steps", {})
        step_key = (entry.cache_group, entry.write_cache, layer.hidden, layer.nq, layer.nkv, layer.d, layer.intermediate, layer.window)
        step = steps.get(step_key)
        if step is None:
            step = steps[step_key] = ops.native_step(ctx, group, layer, residual, entry.write_cache)
        # two buffers take turns: a layer's output is the next layer's pending input
        outs = ctx.__dict__.setdefault("_native_outs", [])
        if not outs:
            outs.extend(torch.empty((residual.shape[0], layer.hidden), dtype=torch.bfloat16, device=residual.device) for _ in range(2))
        out = outs[0] if pending is not outs[0] else outs[1]
        k_cache, v_cache = group.kv_slot(entry.cache_slot)
        return out if ops.layer_forward(layer, step, k_cache, v_cache, pending, out) else None

    def _native_layer(self, ctx):
        from .attention import AttentionMixer
        from .feed_forward import SwiGLU
        from .norm import RMSNorm
        from .position import RotaryHalfSplit
        m, f = self.mixer, self.feed_forward
        if not (type(m) is AttentionMixer and type(f) is SwiGLU and type(self.input_norm) is RMSNorm
                and type(self.post_mixer_norm) is RMSNorm and type(m.position) is RotaryHalfSplit and not m.has_out_bias
                and self.input_norm.eps == self.post_mixer_norm.eps):
            return None
        ops = ctx.ops
        if not ops.NativeLayer.fits(m.qkv_weight, m.out_weight, f.gate_up_weight, f.down_weight):
            return None
        inv_freq, rot = m.position.rotary_table(ctx.device)
        return ops.NativeLayer(self.input_norm.weight, self.post_mixer_norm.weight, self.input_norm.eps, m.qkv_weight, m.qkv_bias,
                               m.out_weight, f.gate_up_weight, f.down_weight, inv_freq, rot, m.num_heads, m.num_kv_heads,
                               m.head_dim, m.scale, m.window)

    @staticmethod
    def _normed(norm, ctx, residual, pending, reader):
        """The input of ``reader``: ``pending`` added to the residual and normalised, or, when the part before has
        begun this very norm already, the rows it left (materialised for a reader that does not take them)."""
        if getattr(pending, "weight", None) is not None and hasattr(pending, "materialize"):
            if pending.weight is not norm.weight:
                raise RuntimeError("a part began a norm that is not the one that follows it")
            return pending if getattr(reader, "takes_prenormed", False) else pending.materialize()
        # the norm is told which matrix comes next: in a decode step it starts that matrix into L2 meanwhile
        return _norm(norm, ctx, residual, pending, reader.reads_first())

    @staticmethod
    def _branch(part, args, ctx, residual, norm_after, upcoming=None):
        follow = None
        if norm_after is not None and _accepts(part.forward, "follow"):
            follow = norm_after.following(ctx, residual)
        if follow is None:
            return part.forward(*args)
        if upcoming is not None and _accepts(part.forward, "upcoming"):
            return part.forward(*args, follow=follow, upcoming=upcoming)
        return part.forward(*args, follow=follow)


def _norm(norm, ctx, residual, delta, upcoming):
    """A norm of another kind need not know the hint: it is passed only to a ``forward`` that names it."""
    if upcoming is not None and _accepts(norm.forward, "upcoming"):
        return norm.forward(ctx, residual, delta, upcoming=upcoming)
    return norm.forward(ctx, residual, delta)


class DepthWeights:
    """The learned weights with which a layer blends all streams so far; a part, so that it is bound by name."""

    def __init__(self, count: int):
        self.count = int(count)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.count,), "vector")}

    def bind(self, tensors: dict) -> None:
        from .base import Part
        Part.bind(self, tensors)

    def reads_first(self):
        return None


class ParallelDepthAverageBlock:
    """One norm whose output feeds mixer and feed-forward side by side, then a learned average over depth:
        h = norm(x);  X_{i+1} = x + (mixer(h) + feed_forward(h));  x <- sum_{j=0..i+1} a_j X_j,
    with X_0 the embedding's output and i = ``depth`` the layer's place in the stack (``block_params``).  The X_j of a
    step are kept in one float32 tensor [layers + 1, T, width] that the first layer makes; sum and average are
    float32 and one kernel.  A layer may have no feed-forward."""
    part_names = ("norm", "mixer", "feed_forward", "depth_average")

    def __init__(self, layer_spec):
        params = dict(layer_spec.block_params)
        self.depth, self.total = int(params["depth"]), int(params["total"])
        self.norm = build_part("norm", layer_spec.norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward) if layer_spec.feed_forward is not None else None
        self.depth_average = DepthWeights(self.depth + 2)

    def parts(self) -> dict:
        return {name: getattr(self, name) for name in self.part_names if getattr(self, name) is not None}

    def forward(self, ctx, residual, pending, entry):
        h = self.norm.forward(ctx, residual, pending)
        mixed = self.mixer.forward(ctx, h, entry)
        fed = self.feed_forward.forward(ctx, h) if self.feed_forward is not None else None
        if self.depth == 0 or "stream_history" not in ctx.__dict__:
            ctx.__dict__["stream_history"] = torch.empty((self.total + 1,) + tuple(residual.shape), dtype=torch.float32,
                                                         device=residual.device)
        ctx.ops.depth_average(ctx.__dict__["stream_history"], residual, mixed, fed, self.depth_average.weight, self.depth)
        return None


class HyperGatedBlock:
    """A layer over S residual streams x [S, T, width] (float32).  Sublayer q (1: the mixer, 2: the feed-forward, if
    the layer has one):
        h = norm_q(sum_s read_q[s] x_s);  y = sublayer(h) * sigmoid(W_rg h + b_rg);
        x_t <- sum_s mix_q[s, t] x_s + write_q[t] * y      (every stream from the old ones)
    and the mixer reads h blended with the row of the token before (``TokenShift``), the gate the rows as they are.
    A sublayer's y is not put into the streams at once: it is handed on as ``pending`` and the kernel of the norm that
    reads the streams next does it (the next sublayer's, the next layer's, or the model's final norm)."""

    def __init__(self, layer_spec):
        from .streams import HyperConnection, ResidualGate, TokenShift
        params = dict(layer_spec.block_params)
        streams, width = int(params["streams"]), int(params["hidden_size"])
        self.norm1 = build_part("norm", layer_spec.norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.hc1, self.rg1 = HyperConnection(streams), ResidualGate(width)
        self.shift = TokenShift(width, params["shift_group"], params["shift_slot"])
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward) if layer_spec.feed_forward is not None else None
        self.part_names = ("norm1", "hc1", "rg1", "shift", "mixer")
        if self.feed_forward is not None:
            self.norm2 = build_part("norm", layer_spec.norm)
            self.hc2, self.rg2 = HyperConnection(streams), ResidualGate(width)
            self.part_names += ("norm2", "hc2", "rg2", "feed_forward")

    def parts(self) -> dict:
        return {name: getattr(self, name) for name in self.part_names}

    def forward(self, ctx, residual, pending, entry):
        from .streams import StreamUpdate
        shift = self.shift.within_norm(ctx)
        if shift is not None:                       # a decode step: norm and token shift are one kernel
            h, shifted = self.norm1.forward(ctx, residual, pending, read=self.hc1.read, shift=shift)
        else:
            h = self.norm1.forward(ctx, residual, pending, read=self.hc1.read)
            shifted = self.shift.forward(ctx, h)
        gate = self.rg1.logits(ctx, h)
        y = self.mixer.forward(ctx, shifted, entry)
        pending = StreamUpdate(y, gate, self.rg1.bias, self.hc1.mix, self.hc1.write)
        if self.feed_forward is None:
            return pending
        h = self.norm2.forward(ctx, residual, pending, read=self.hc2.read)
        gate = self.rg2.logits(ctx, h)
        y = self.feed_forward.forward(ctx, h)
        return StreamUpdate(y, gate, self.rg2.bias, self.hc2.mix, self.hc2.write)


class SandwichBlock:
    """Norms on both sides of every sublayer:
        x <- x + norm1b(mixer(norm1(x)));  x <- x + norm2b(feed_forward(norm2(x)))   (the second where the layer has one).
    A sublayer's output is not normed and added at once: it is handed on as ``pending`` (``PostNormed``), and the kernel
    of the norm that reads the stream next norms it, adds it and norms the sum (the next sublayer's, the next layer's,
    a junction's, or the model's final norm)."""

    def __init__(self, layer_spec):
        self.norm1 = build_part("norm", layer_spec.norm)
        self.norm1b = build_part("norm", layer_spec.norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward) if layer_spec.feed_forward is not None else None
        self.part_names = ("norm1", "mixer", "norm1b")
        if self.feed_forward is not None:
            self.norm2 = build_part("norm", layer_spec.norm)
            self.norm2b = build_part("norm", layer_spec.norm)
            self.part_names += ("norm2", "feed_forward", "norm2b")

    def parts(self) -> dict:
        return {name: getattr(self, name) for name in self.part_names}

    @staticmethod
    def _post(norm, out):
        """A sublayer may return (rows, bias still to add): the norm's kernel adds it."""
        return norm.after(*out) if isinstance(out, tuple) else norm.after(out)

    def forward(self, ctx, residual, pending, entry):
        h = self.norm1.forward(ctx, residual, pending)
        pending = self._post(self.norm1b, self.mixer.forward(ctx, h, entry))
        if self.feed_forward is None:
            return pending
        h = self.norm2.forward(ctx, residual, pending)
        if _accepts(self.feed_forward.forward, "defer_bias"):
            return self._post(self.norm2b, self.feed_forward.forward(ctx, h, defer_bias=True))
        return self._post(self.norm2b, self.feed_forward.forward(ctx, h))


register_block("prenorm", PreNormBlock)
register_block("sandwich", SandwichBlock)
register_block("hyper_gated", HyperGatedBlock)
register_block("parallel_depth_average", ParallelDepthAverageBlock)
