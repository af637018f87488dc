"""Several mixers side by side: all read the same rows, and the result is a weighted sum of theirs.

    out = sum_i scale_i * mixer_i(h)

Each side is a mixer of its own kind with its own cache group and slot (a run entry names the first side's place in
``cache_group``/``cache_slot`` and the others' in ``more``).  A side is a mixer that can work between shared products: it
has ``input_width``, ``inner_width`` and ``mix(ctx, projected, entry, out, scale)`` besides ``qkvg.weight`` and
``o.weight``.  The sides' input projections are ONE product, their gated rows are written side by side (each times its
scale), and their output projections are one product over the concatenated rows, so that the weighted sum costs nothing.
The sides keep their parameters' names, behind the side's name (``left.qkvg.weight``); when the tensors are bound, the
matrices are laid out side by side once and the sides' own matrices become views of that storage.
"""
from __future__ import annotations

import torch

from .base import Mixer, build_part, register_mixer
from .spec import PartSpec


class ParallelMixer(Mixer):
    def __init__(self, hidden_size: int, sides):
        """``sides``: [(name, PartSpec or {"kind", "params"}, scale)]."""
        self.hidden_size = int(hidden_size)
        self.names, self.sides, self.scales = [], [], []
        for name, spec, scale in sides:
            if isinstance(spec, dict):
                spec = PartSpec(spec["kind"], spec.get("params", {}))
            self.names.append(str(name))
            self.sides.append(build_part("mixer", spec))
            self.scales.append(float(scale))
        if len(set(self.names)) != len(self.names) or not self.sides:
            raise ValueError("the sides of a parallel mixer need names of their own")
        if not all(hasattr(s, "mix") and hasattr(s, "input_width") and hasattr(s, "inner_width") for s in self.sides):
            raise ValueError("the sides of a parallel mixer are mixers that can work between shared products (input_width, "
                             "inner_width, mix)")
        self.in_weight = self.o_weight = None

    def parameter_shapes(self) -> dict:
        return {f"{name}.{local}": what for name, side in zip(self.names, self.sides) for local, what in side.parameter_shapes().items()}

    def bind(self, tensors: dict) -> None:
        want = self.parameter_shapes()
        missing, extra = sorted(set(want) - set(tensors)), sorted(set(tensors) - set(want))
        if missing or extra:
            raise ValueError(f"ParallelMixer: missing {missing}, unexpected {extra}")
        for name, side in zip(self.names, self.sides):
            side.bind({k[len(name) + 1:]: t for k, t in tensors.items() if k.startswith(name + ".")})
        # one matrix for all input projections, one for all output projections; the sides see views of them
        self.in_weight = torch.cat([s.qkvg_weight for s in self.sides], dim=0).contiguous()
        self.o_weight = torch.cat([s.o_weight for s in self.sides], dim=1).contiguous()
        row = col = 0
        for s in self.sides:
            s.qkvg_weight = self.in_weight[row:row + s.input_width]
            s.o_weight = self.o_weight[:, col:col + s.inner_width]
            row, col = row + s.input_width, col + s.inner_width
        for name, side in zip(self.names, self.sides):
            for local in side.parameter_shapes():
                setattr(self, f"{name}.{local}".replace(".", "_"), getattr(side, local.replace(".", "_")))

    def reads_first(self):
        return self.in_weight

    def cache_need(self):
        return [side.cache_need() for side in self.sides]

    def forward(self, ctx, h, entry):
        ops = ctx.ops
        projected = ops.linear(h, self.in_weight)                            # [T, every side's projections]
        inner = sum(s.inner_width for s in self.sides)
        rows = torch.empty((projected.shape[0], inner), dtype=ctx.dtype, device=projected.device)
        row = col = 0
        for i, (side, scale) in enumerate(zip(self.sides, self.scales)):
            side.mix(ctx, projected[:, row:row + side.input_width], entry.place(i), out=rows[:, col:col + side.inner_width], scale=scale)
            row, col = row + side.input_width, col + side.inner_width
        # the weighted sum of the sides is the product over their concatenated rows; it stays float32 on its way to a norm
        return ops.linear(rows, self.o_weight, None, out_float32=True)


register_mixer("parallel", ParallelMixer)
