"""Junctions: parts that rewrite the residual stream between two layers.

``reinject``: x <- W [x; x0], x0 the embedding's output of the same tokens and W [width, 2 width] (x's columns first).  A
design that runs a span of its layers several times puts one before every pass, so that the input stays in sight.  What
the block before left pending is settled into the stream by the kernel that lays [x; x0] out for the product; the
product's float32 result is the new stream.
"""
from __future__ import annotations

from .base import Junction, register_junction


class Reinject(Junction):
    def __init__(self, hidden_size: int):
        self.hidden_size = int(hidden_size)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.hidden_size, 2 * self.hidden_size), "matrix")}

    def reads_first(self):
        return self.weight

    def forward(self, ctx, residual, pending, origin):
        post = None if pending is None else (pending.weight, pending.eps, pending.bias)
        both = ctx.ops.residual_concat(residual, None if pending is None else pending.y, origin, ctx.dtype, post=post)
        return ctx.ops.linear(both, self.weight, None, out_float32=True)


register_junction("reinject", Reinject)
