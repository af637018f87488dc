"""Vocabulary head: float32 logits of the rows that are wanted.

logits = x_last lm_head.weight^T, no bias (src/flexengine/inference/models/qwen2.py:131-136); tied
embeddings bind ``weight`` to the embedding table's storage.  A design may multiply the logits by a constant and
squash them: logits <- softcap * tanh(logits * scale / softcap) (``softcap`` 0: not squashed).
"""
from __future__ import annotations

from .base import Head, register_head


class LinearHead(Head):
    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, softcap: float = 0.0):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale, self.softcap = float(scale), float(softcap)
        self.weight = None

    def parameter_shapes(self) -> dict:
        return {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def forward(self, ctx, h):
        logits = ctx.ops.linear(h, self.weight, None, out_float32=True)
        if self.scale != 1.0 or self.softcap > 0.0:
            ctx.ops.scale_softcap(logits, self.scale, self.softcap)         # in place, float32
        return logits


register_head("linear", LinearHead)
