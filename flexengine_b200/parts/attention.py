"""Causal grouped-query attention over the paged cache.

q = h Wq^T + bq, k, v likewise; rotary encoding of q and k; k, v written to the
request's pages before the scores are taken, so that a portion sees itself; key t is
visible to the query at absolute position p iff t <= p (and t > p - window for a
window group); softmax in float32; query head h reads key/value head h // (nq/nkv);
output projection (src/flexengine/inference/models/qwen2.py:98-129,
src/flexengine/inference/attention/paged.py:18-70).
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, build_part, register_mixer
from .spec import PartSpec


class AttentionMixer(Mixer):
    takes_prenormed = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec | dict | None = None, qkv_bias: bool = True, out_bias: bool = False,
                 window: int = 0, scale: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("Invalid GQA head ratio")
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise ValueError(f"head_dim={head_dim}: the attention kernels take head sizes in steps of 16 from 16 to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = \
            int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.has_qkv_bias, self.has_out_bias, self.window = bool(qkv_bias), bool(out_bias), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        if position is None:
            position = PartSpec("none")
        if isinstance(position, dict):
            position = PartSpec(position["kind"], position.get("params", {}))
        self.position = build_part("position", position)
        self.qkv_weight = self.qkv_bias = self.out_weight = self.out_bias = None      # bound by local name

    @property
    def qkv_width(self) -> int:
        return (self.num_heads + 2 * self.num_kv_heads) * self.head_dim

    def parameter_shapes(self) -> dict:
        shapes = {"qkv.weight": ((self.qkv_width, self.hidden_size), "matrix"),
                  "out.weight": ((self.hidden_size, self.num_heads * self.head_dim), "matrix")}
        if self.has_qkv_bias:
            shapes["qkv.bias"] = ((self.qkv_width,), "vector")
        if self.has_out_bias:
            shapes["out.bias"] = ((self.hidden_size,), "vector")
        return shapes

    def reads_first(self):
        return self.qkv_weight

    def cache_need(self):
        return {"kind": "window" if self.window > 0 else "full", "kv_heads": self.num_kv_heads,
                "head_dim": self.head_dim, "window": self.window}

    def forward(self, ctx, h, entry, follow=None, upcoming=None):
        ops = ctx.ops
        group = ctx.groups[entry.cache_group]
        k_cache, v_cache = group.kv_slot(entry.cache_slot)
        slot_mapping = group.slot_mapping if entry.write_cache else None
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        if self.position.applies_itself:
            # an encoding of its own: projection and bias, the encoding on the query and key heads in place,
            # then the keys and values to their cache slots
            qkv = ops.linear(h, self.qkv_weight, self.qkv_bias)
            self.position.apply(ctx, qkv[:, :nq * d].view(-1, nq, d), qkv[:, nq * d:(nq + nkv) * d].view(-1, nkv, d))
            ops.qkv_bias_rope_cache(qkv, None, ctx.positions, None, 0, slot_mapping, k_cache, v_cache, nq, nkv, d,
                                    group.page_size)
        else:
            # projection, bias, rotation and the cache write are one operation (one kernel in decode); a
            # run entry that only reads another entry's cache passes no slot mapping, so nothing is written
            inv_freq, rot = self.position.rotary_table(h.device) or (None, 0)
            qkv = ops.qkv_projection(h, self.qkv_weight, self.qkv_bias, ctx.positions, inv_freq, rot, slot_mapping,
                                     k_cache, v_cache, nq, nkv, d, group.page_size)
        out = ops.paged_attention(qkv, k_cache, v_cache, group.block_table, ctx, self.num_heads,
                                  self.num_kv_heads, self.head_dim, group.page_size, self.scale, self.window,
                                  upcoming=self.out_weight)
        if follow is not None:
            return ops.linear(out, self.out_weight, self.out_bias, follow=follow, upcoming=upcoming)
        return ops.linear(out, self.out_weight, self.out_bias)


class GatedAttentionMixer(Mixer):
    """Grouped-query attention with the options some designs add, each a parameter:

    ``conv`` > 0: a causal convolution of that many taps over time on every channel of the projected q, k and v
    (y_t = sum_j w[:, j] u_(t - conv + 1 + j), zeros before the sequence's start), before everything else; the last
    conv - 1 projected rows of a request are kept in a state slot (``conv_group``, ``conv_slot``).
    ``rot_dims``: the first that many entries of every query and key head turn by position * rot_base^(-2i/rot_dims),
    entry i paired with i + rot_dims/2; the rest pass unchanged.
    ``qk_norm``: queries and keys are then divided by their root mean square over the head (eps inside the root).
    ``mask``: "full" (every earlier key), "window" (the last ``mask_size`` keys) or "chunk" (the earlier keys of the
    query's own chunk of ``mask_size`` positions, counted from position 0 of the sequence).
    ``norm_weights``: the unit norm becomes an RMS norm with a weight of ``dim`` numbers, one for the queries and one for
    the keys, shared by their heads.
    ``temp_coef``, ``temp_every``: a query temperature: the query at position p is multiplied (after its norm) by
    1 + temp_coef * ln(floor((p + 1) / temp_every) + 1); 0 for none.
    ``sink``: 1 is added to the softmax's denominator, as if every query also saw a key of score 0 and value 0.
    ``gate`` "head": every head's output is multiplied by sigmoid(w_g,h . x), x the rows the projections read; "element":
    every entry of the concatenated heads by the sigmoid of its own projection of x (``heads * vdim`` gate rows).  The value size may differ
    from the query/key size: the cache and the attention kernels run at ``head`` = the larger, in steps of 16, the
    smaller padded with zeros (scores and outputs are the same).  ``gate`` "none": the heads go to the output projection as
    they are.  No biases.
    ``norm_scope`` "all" (with ``norm_weights``): instead of a norm per head, the whole query projection (all heads at once)
    goes through one RMS norm with a weight of ``heads * dim`` numbers, and the whole key projection through one with
    ``kv_heads * dim``; this norm comes BEFORE the rotation.
    ``rot_pairs`` "interleaved": entry 2i turns with 2i + 1 instead of i with i + rot_dims/2.
    ``rotate_values``: the value of position j turns by j over all ``vdim`` entries (pairs laid out as ``rot_pairs`` says,
    pair m by j * rot_base^(-2m/vdim)) before it is cached, and a head's output at position i is turned back by i.
    ``weights`` "sigmoid": the weight of a visible key is sigmoid(score * scale + b_head) with a learned number per head
    (``score_bias``), not normalised over the keys.

    q, k, v and the head gates are one product; convolution, rotation, unit norm and the cache write are one kernel;
    angles, norms, scores and softmax are float32."""

    MASKS = ("full", "window", "chunk")
    GATES = ("head", "element", "none")
    NORM_SCOPES = ("head", "all")
    ROT_PAIRS = ("halves", "interleaved")
    WEIGHTS = ("softmax", "sigmoid")

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, rot_base: float = 10000.0,
                 rot_dims: int = 0, conv: int = 0, qk_norm: bool = False, eps: float = 1e-6, mask: str = "full", mask_size: int = 0,
                 sink: bool = False, conv_group: int = -1, conv_slot: int = -1, norm_weights: bool = False, temp_coef: float = 0.0,
                 temp_every: int = 1, gate: str = "head", norm_scope: str = "head", rot_pairs: str = "halves", rotate_values: bool = False,
                 weights: str = "softmax"):
        if heads % kv_heads:
            raise ValueError("Invalid GQA head ratio")
        if mask not in self.MASKS or (mask != "full" and mask_size <= 0):
            raise ValueError(f"mask {mask!r} of size {mask_size}: known masks are {', '.join(self.MASKS)}; all but 'full' need a size")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError("rot_dims must be even and at most dim")
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.vdim = int(hidden_size), int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.rot_base, self.rot_dims, self.conv = float(scale), float(rot_base), int(rot_dims), int(conv)
        self.qk_norm, self.eps, self.mask, self.mask_size, self.sink = bool(qk_norm), float(eps), mask, int(mask_size), bool(sink)
        self.conv_group, self.conv_slot = int(conv_group), int(conv_slot)
        self.norm_weights, self.temp_coef, self.temp_every, self.gate = bool(norm_weights), float(temp_coef), int(temp_every), gate
        if gate not in self.GATES:
            raise ValueError(f"gate {gate!r}: known gates are {', '.join(self.GATES)}")
        if self.norm_weights and not self.qk_norm:
            raise ValueError("norm weights need the query/key norm")
        if norm_scope not in self.NORM_SCOPES or rot_pairs not in self.ROT_PAIRS or weights not in self.WEIGHTS:
            raise ValueError(f"norm_scope {norm_scope!r} / rot_pairs {rot_pairs!r} / weights {weights!r}: known are "
                             f"{self.NORM_SCOPES}, {self.ROT_PAIRS} and {self.WEIGHTS}")
        self.norm_scope, self.rot_pairs, self.rotate_values, self.weights = norm_scope, rot_pairs, bool(rotate_values), weights
        # what the second preparation kernel does (a norm over the whole projection, neighbouring pairs, turned values) and
        # what only the first one does (convolutions, a norm per head, the query temperature) do not meet in one layer
        self.wide_prepare = norm_scope == "all" or rot_pairs == "interleaved" or self.rotate_values
        if self.wide_prepare and (self.conv > 0 or self.temp_coef != 0.0 or (self.qk_norm and norm_scope == "head")):
            raise ValueError("a norm over the whole projection, neighbouring rotation pairs or turned values go with neither a "
                             "convolution, nor a norm per head, nor a query temperature")
        if norm_scope == "all" and not self.norm_weights:
            raise ValueError("the norm over the whole projection has weights")
        if self.rotate_values and self.vdim % 2:
            raise ValueError("values turn in pairs: vdim must be even")
        if weights == "sigmoid" and self.sink:
            raise ValueError("a sink belongs to a softmax")
        self.score_bias = None
        self._inv_freq_v = {}
        if self.temp_every < 1:
            raise ValueError("temp_every must be positive")
        self.q_norm_weight = self.k_norm_weight = None
        if self.conv > 1 and self.conv_group < 0:
            raise ValueError("a convolution of more than one tap needs a state slot for its history")
        self.head = -(-max(self.dim, self.vdim) // 16) * 16
        if self.head > 1024:
            raise ValueError(f"head size {self.head}: the attention kernels take up to 1024")
        self.qkvg_weight = self.conv_weight = self.o_weight = None
        self._conv_by_tap = None
        self._inv_freq = {}

    @property
    def channels(self) -> int:
        return (self.heads + self.kv_heads) * self.dim + self.kv_heads * self.vdim

    @property
    def gate_width(self) -> int:
        return {"head": self.heads, "element": self.heads * self.vdim, "none": 0}[self.gate]

    @property
    def input_width(self) -> int:
        """Rows of the one matrix that holds all projections of the mixer's input."""
        return self.channels + self.gate_width

    @property
    def inner_width(self) -> int:
        """Columns of the output projection."""
        return self.heads * self.vdim

    def parameter_shapes(self) -> dict:
        shapes = {"qkvg.weight": ((self.input_width, self.hidden_size), "matrix"),
                  "o.weight": ((self.hidden_size, self.inner_width), "matrix")}
        if self.conv > 0:
            shapes["conv.weight"] = ((self.channels, self.conv), "vector")
        if self.norm_weights:
            every = self.norm_scope == "all"
            shapes["q_norm.weight"] = ((self.heads * self.dim if every else self.dim,), "vector")
            shapes["k_norm.weight"] = ((self.kv_heads * self.dim if every else self.dim,), "vector")
        if self.weights == "sigmoid":
            shapes["score_bias"] = ((self.heads,), "vector")
        return shapes

    def bind(self, tensors: dict) -> None:
        super().bind(tensors)
        # the table tap by tap, [taps, channels]: the kernel's lanes then read neighbouring numbers
        self._conv_by_tap = self.conv_weight.t().contiguous() if self.conv > 0 else None

    def reads_first(self):
        return self.qkvg_weight

    def cache_need(self):
        return {"kind": self.mask, "kv_heads": self.kv_heads, "head_dim": self.head, "window": self.mask_size}

    def inverse_frequencies(self, device):
        key = str(device)
        if key not in self._inv_freq:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            table = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / max(self.rot_dims, 1))
            self._inv_freq[key] = table.to(torch.float32).to(device).contiguous()
        return self._inv_freq[key]

    def value_inverse_frequencies(self, device):
        """The values' rotation: pair m of ``vdim`` / 2 turns by position * rot_base^(-2m/vdim)."""
        key = str(device)
        if key not in self._inv_freq_v:
            m = torch.arange(self.vdim // 2, dtype=torch.float64)
            table = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * m / self.vdim)
            self._inv_freq_v[key] = table.to(torch.float32).to(device).contiguous()
        return self._inv_freq_v[key]

    def forward(self, ctx, h, entry):
        projected = ctx.ops.linear(h, self.qkvg_weight)                      # [T, channels + gates]
        return ctx.ops.linear(self.mix(ctx, projected, entry), self.o_weight)

    def mix(self, ctx, projected, entry, out=None, scale=1.0):
        """Everything between the input projections and the output projection: ``projected`` [T, >= input_width] (any
        row stride) -> the gated heads [T, inner_width], times ``scale``, into ``out`` where given (a view of a wider
        buffer: a mixer that stands beside another one shares its products with it)."""
        ops = ctx.ops
        group = ctx.groups[entry.cache_group]
        k_cache, v_cache = group.kv_slot(entry.cache_slot)
        slot_mapping = group.slot_mapping if entry.write_cache else None
        history = ctx.groups[self.conv_group].state(self.conv_slot) if self.conv > 1 else None
        more = {}
        if self.norm_weights:
            more.update(q_weight=self.q_norm_weight, k_weight=self.k_norm_weight)
        if self.temp_coef != 0.0:
            more.update(temp=(self.temp_coef, self.temp_every))
        turned = self.value_inverse_frequencies(projected.device) if self.rotate_values else None
        if self.wide_prepare:
            queries = ops.qkv_norm_rope_cache(
                projected, self.q_norm_weight, self.k_norm_weight, self.eps, ctx.positions,
                self.inverse_frequencies(projected.device) if self.rot_dims else None, self.rot_dims, self.rot_pairs, turned,
                slot_mapping, k_cache, v_cache, self.heads, self.kv_heads, self.dim, self.vdim, self.head, group.page_size)
        else:
            queries = ops.qkv_conv_rope_norm_cache(
                projected, self._conv_by_tap, history, self.conv, ctx.state_slots, ctx.cu_q, ctx.token_request, ctx.positions,
                self.inverse_frequencies(projected.device) if self.rot_dims else None, self.rot_dims, self.qk_norm, self.eps, slot_mapping,
                k_cache, v_cache, self.heads, self.kv_heads, self.dim, self.vdim, self.head, group.page_size, **more)
        # one int says what a query sees: 0 every earlier key, w > 0 the last w, -c < 0 its own chunk of c positions
        visibility = {"full": 0, "window": self.mask_size, "chunk": -self.mask_size}[self.mask]
        if self.weights == "sigmoid":
            mixed = ops.paged_attention(queries, k_cache, v_cache, group.block_table, ctx, self.heads, self.kv_heads, self.head,
                                        group.page_size, self.scale, visibility, weights="sigmoid", head_bias=self.score_bias)
        else:
            mixed = ops.paged_attention(queries, k_cache, v_cache, group.block_table, ctx, self.heads, self.kv_heads, self.head,
                                        group.page_size, self.scale, visibility, sink=self.sink)
        head = self.head
        if self.rotate_values:
            # every head's sum turned back by the query's position; the padding of the kernels' head size goes on the way
            if self.gate == "none":
                return ops.unrotate_heads(mixed, ctx.positions, turned, self.heads, head, self.vdim, self.rot_pairs, scale=scale, out=out)
            mixed, head = ops.unrotate_heads(mixed, ctx.positions, turned, self.heads, head, self.vdim, self.rot_pairs), self.vdim
        elif self.gate == "none":
            rows = mixed if head == self.vdim else mixed.view(-1, self.heads, head)[:, :, :self.vdim].reshape(-1, self.inner_width)
            if out is None and scale == 1.0:
                return rows
            rows = rows if scale == 1.0 else rows * scale
            if out is None:
                return rows
            out.copy_(rows)
            return out
        if self.gate == "head" and out is None and scale == 1.0:
            return ops.head_gate(mixed, projected, self.channels, self.heads, head, self.vdim)
        return ops.head_gate(mixed, projected, self.channels, self.heads, head, self.vdim, per_element=self.gate == "element",
                             scale=scale, out=out)


register_mixer("attention", AttentionMixer)
register_mixer("gated_attention", GatedAttentionMixer)
