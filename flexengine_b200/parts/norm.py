"""RMSNorm fused with the residual add.

y = w * (x * rsqrt(mean(x^2) + eps)), statistics and product in float32
(src/flexengine/inference/kernels/rmsnorm.py:24-32; called at
src/flexengine/inference/models/qwen2.py:67-71,97,130,134).  The residual stream is
float32; the pending branch output is added in the same kernel.
"""
from __future__ import annotations

import torch

from .base import Norm, register_norm


class PostNormed:
    """A branch's output on its way into the residual stream through a norm of its own: the stream receives
    w * (y + bias) / sqrt(mean((y + bias)^2) + eps).  The kernel of the norm that reads the stream next does it (the
    ``pending`` of this framework: a branch output is not added at once).  ``y`` is float32 or in the compute dtype,
    ``bias`` (float32, may be None) what the branch's last product has yet to add."""
    __slots__ = ("y", "weight", "eps", "bias")

    def __init__(self, y, weight, eps, bias=None):
        self.y, self.weight, self.eps, self.bias = y, weight, float(eps), bias


class RMSNorm(Norm):
    """``unit_offset``: the checkpoint stores the weight around zero and the norm multiplies by (1 + w).  The sum is taken
    once, in float32, when the weights are bound; the kernels see a plain weight."""

    def __init__(self, hidden_size: int, eps: float, unit_offset: bool = False):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.unit_offset = bool(unit_offset)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.hidden_size,), "vector")}

    def bind(self, tensors: dict) -> None:
        super().bind(tensors)
        if self.unit_offset:
            self.weight = self.weight.to(torch.float32) + 1.0

    def forward(self, ctx, residual, delta, rows=None, upcoming=None):
        if isinstance(delta, PostNormed):
            # the branch before ends in a norm of its own (a layer with norms on both sides of a sublayer): one kernel
            # norms the branch's output, adds it to the stream and norms the sum
            return ctx.ops.add_rmsnorm(residual, delta.y, self.weight, self.eps, ctx.dtype, rows,
                                       post=(delta.weight, delta.eps, delta.bias))
        return ctx.ops.add_rmsnorm(residual, delta, self.weight, self.eps, ctx.dtype, rows, upcoming=upcoming)

    def after(self, y, bias=None) -> PostNormed:
        """``y`` on its way through this norm into the residual stream (this norm follows a sublayer)."""
        return PostNormed(y, self.weight, self.eps, bias)

    def following(self, ctx, residual):
        # a decode step in bfloat16 on kernels that can: the product before this norm adds to the residual and
        # starts the norm, the product after it finishes it
        ops = ctx.ops
        if (getattr(ops, "FUSES_RESIDUAL_NORM", False) and ctx.dtype == torch.bfloat16
                and ctx.num_tokens <= ops.FUSED_NORM_MAX_ROWS and type(self).forward is RMSNorm.forward):
            return (residual, self.weight, self.eps)
        return None


class GroupRMSNorm(Norm):
    """RMSNorm in groups: a row is cut into ``groups`` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps); the whole is then multiplied by the weight.  One group is the plain norm."""

    def __init__(self, hidden_size: int, eps: float, groups: int = 1):
        self.hidden_size, self.eps, self.groups = int(hidden_size), float(eps), int(groups)
        if self.groups < 1 or self.hidden_size % self.groups:
            raise ValueError("the number of norm groups must divide the width")
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.hidden_size,), "vector")}

    def forward(self, ctx, residual, delta, rows=None):
        return ctx.ops.add_group_rmsnorm(residual, delta, self.weight, self.eps, self.groups, ctx.dtype, rows)


class StreamRMSNorm(Norm):
    """RMSNorm of a learned sum of several residual streams: u = sum_s read[s] x_s over the streams x [S, T, hidden]
    (``read`` None: the plain sum), y = w * u * rsqrt(mean(u^2) + eps), all float32.  What the sublayer before left
    (``delta``: an object with ``y``, ``gate``, ``gate_bias``, ``mix`` and ``write``) is put into the streams first, in
    the same kernel: x_t <- sum_s mix[s, t] x_s + write[t] * y * sigmoid(gate + gate_bias), every stream from the old
    ones.  With ``rows`` only those rows are read and nothing is written back."""

    def __init__(self, hidden_size: int, eps: float, streams: int):
        self.hidden_size, self.eps, self.streams = int(hidden_size), float(eps), int(streams)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.hidden_size,), "vector")}

    def forward(self, ctx, residual, delta, rows=None, read=None, shift=None):
        """``shift`` = (mu, kept rows, state slots) in a step of one token a request: the token shift of the normed rows is
        done in the same kernel, and (rows, shifted rows) come back."""
        if shift is not None:
            return ctx.ops.stream_rmsnorm(residual, read, self.weight, self.eps, ctx.dtype, update=delta, rows=rows, shift=shift)
        return ctx.ops.stream_rmsnorm(residual, read, self.weight, self.eps, ctx.dtype, update=delta, rows=rows)


register_norm("rmsnorm", RMSNorm)
register_norm("stream_rmsnorm", StreamRMSNorm)
register_norm("group_rmsnorm", GroupRMSNorm)
