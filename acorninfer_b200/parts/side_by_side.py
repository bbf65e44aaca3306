"""Two mixers side by side on the same input: ``left_scale * left(h) + right_scale * right(h)``.

Both mixers are built from their own specs (any registered kinds whose last step is an output
projection: they offer ``inner(x, inputs, cache, out_scale)``, the rows that projection reads, and
``w_o``).  The two projections are one matrix product over the concatenated rows, ``[left rows | right
rows] [W_o,left | W_o,right]^T``: the sum of the two results is taken in the product's float32
accumulator, and each side's scale is applied in float32 where its rows are rounded.

Cache: one side may keep keys and values in pages, and either side per-request state; the states lie
one after the other in the request's slot (``state_base`` tells a side where its part starts).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, BuildContext, CacheNeeds, Mixer, PartSpec, StateNeeds, build_part


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    adds_residual = True

    def __init__(self, ctx: BuildContext, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0):
        self.ctx = ctx
        self.sides = [(left.prefix, build_part(MIXERS, left, ctx)), (right.prefix, build_part(MIXERS, right, ctx))]
        self.scales = (float(left_scale), float(right_scale))
        for _, m in self.sides:
            if not hasattr(m, "inner"):
                raise ValueError(f"{type(m).__name__} cannot stand beside another mixer: it offers no rows before an "
                                 "output projection ('inner')")
        self.graph_safe = all(getattr(m, "graph_safe", False) for _, m in self.sides)
        self.w_o = None

    def tensor_specs(self):
        return {prefix + rel: spec for prefix, m in self.sides for rel, spec in m.tensor_specs().items()}

    def bind(self, tensors):
        for prefix, m in self.sides:
            m.bind({rel: tensors[prefix + rel] for rel in m.tensor_specs() if prefix + rel in tensors})
        ws = [m.w_o for _, m in self.sides]
        dtype = ws[0].dtype if ws[0].dtype == ws[1].dtype else torch.float32
        self.widths = [w.shape[1] for w in ws]
        self.w_o = torch.cat([w.to(dtype) for w in ws], dim=1).contiguous()

    def step_arrays(self):
        out = {}
        for _, m in self.sides:
            out.update(m.step_arrays())
        return out

    def cache_needs(self):
        kv, size = None, 0
        for _, m in self.sides:
            needs = m.cache_needs()
            if needs.kv is not None:
                if kv is not None:
                    raise ValueError("only one of two mixers side by side may keep keys and values in pages")
                kv = needs.kv
            if needs.state is not None:
                if len(needs.state.shape) != 1 or needs.state.dtype not in (None, torch.float32):
                    raise ValueError("mixers side by side keep their state as one float32 vector each")
                m.state_base = size
                size += needs.state.shape[0]
        return CacheNeeds(kv=kv, state=StateNeeds((size,)) if size else None)

    def forward(self, x, inputs, cache, residual32=None):
        (_, left), (_, right) = self.sides
        rows = torch.empty((x.shape[0], sum(self.widths)), dtype=self.ctx.dtype, device=x.device)
        left.inner(x, inputs, cache, out_scale=self.scales[0], out=rows[:, :self.widths[0]])
        right.inner(x, inputs, cache, out_scale=self.scales[1], out=rows[:, self.widths[0]:])
        return ops.linear(rows, self.w_o, out_dtype=self.ctx.dtype, residual32=residual32)
