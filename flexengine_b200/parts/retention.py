"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.

q, k = W_q h, W_k h in heads of ``dim``; v = W_v h in heads of ``vdim``.  The first ``rot_dims`` entries of every query
and key head turn by position * rot_base^(-2i/rot_dims), entry i paired with i + rot_dims/2; the keys are then multiplied
by dim^(-1/2).  Per head, with state S [dim, vdim]:
    S_t = decay_h S_(t-1) + k_t v_t^T ;   o_t = S_t^T q_t .
Each head's o is divided by its root mean square (no weight), the heads are concatenated, multiplied by silu(W_g h) and
projected.  S of a request lives in a state slot of the cache manager in float32, zero at admission; angles, the rotated
queries and keys, the decay, the recurrence and the head norm are float32 whatever the compute dtype.  The four
projections are one product.
"""
from __future__ import annotations

import torch

from .base import Mixer, register_mixer


class RetentionMixer(Mixer):
    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, decay, rot_base: float = 10000.0, rot_dims: int = 0,
                 eps: float = 1e-6):
        self.hidden_size, self.heads, self.dim, self.vdim = int(hidden_size), int(heads), int(dim), int(vdim)
        self.decay = tuple(float(x) for x in decay)
        if len(self.decay) != self.heads:
            raise ValueError("one decay per head")
        self.rot_base, self.rot_dims, self.eps = float(rot_base), int(rot_dims), float(eps)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.dim:
            raise ValueError("rot_dims must be even and at most dim")
        self.qkvg_weight = self.o_weight = None
        self._tables = {}

    @property
    def input_width(self) -> int:
        return 2 * self.heads * self.dim + 2 * self.heads * self.vdim

    @property
    def inner_width(self) -> int:
        return self.heads * self.vdim

    def parameter_shapes(self) -> dict:
        return {"qkvg.weight": ((self.input_width, self.hidden_size), "matrix"),
                "o.weight": ((self.hidden_size, self.inner_width), "matrix")}

    def reads_first(self):
        return self.qkvg_weight

    @property
    def state_elements(self) -> int:
        return self.heads * self.dim * self.vdim

    def cache_need(self):
        return {"kind": "state", "state_shape": (self.state_elements,), "state_dtype": "float32"}

    def tables(self, device):
        """(inverse frequencies [rot_dims / 2] or None, decay [heads]) as float32 on ``device``, rounded once from float64."""
        key = str(device)
        if key not in self._tables:
            inv_freq = None
            if self.rot_dims:
                i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
                inv_freq = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / self.rot_dims)
                inv_freq = inv_freq.to(torch.float32).to(device).contiguous()
            self._tables[key] = (inv_freq, torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device))
        return self._tables[key]

    def forward(self, ctx, h, entry):
        projected = ctx.ops.linear(h, self.qkvg_weight)
        return ctx.ops.linear(self.mix(ctx, projected, entry), self.o_weight)

    def mix(self, ctx, projected, entry, out=None, scale=1.0):
        """``projected`` [T, >= input_width] = q | k | v | g (any row stride) -> the normed, gated heads [T, inner_width],
        times ``scale``, into ``out`` where given."""
        ops = ctx.ops
        H, d, dv = self.heads, self.dim, self.vdim
        state = ctx.groups[entry.cache_group].state(entry.cache_slot)        # [seats, H d dv] float32
        inv_freq, decay = self.tables(projected.device)
        if ctx.max_q_len == 1:
            # a step of one token a request: rotation, recurrence, head norm and gate in one kernel
            return ops.retention_decode(projected, H, d, dv, ctx.positions, inv_freq, self.rot_dims, d ** -0.5, decay, state,
                                        ctx.state_slots, self.eps, ctx.dtype, scale=scale, into=out)
        # queries and keys, rotated, the keys scaled: float32 from here on
        qk = ops.rotate_heads(projected, 2 * H, d, ctx.positions, inv_freq, self.rot_dims, ((H, 1.0), (H, d ** -0.5)))
        values = projected[:, 2 * H * d:2 * H * d + H * dv]
        o = ops.retention_scan(qk, values, decay, state, ctx.state_slots, ctx.cu_q, H, d, dv, max_q_len=ctx.max_q_len)
        gates = projected[:, 2 * H * d + H * dv:2 * H * d + 2 * H * dv]
        return ops.head_rmsnorm_gate(o, None, gates, self.eps, H, ctx.dtype, scale=scale, into=out)


register_mixer("retention", RetentionMixer)
