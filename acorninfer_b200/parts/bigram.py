"""Hashed bigram rows added to the token rows, as a stage after the token table.

``x[t] += table[(prev * mul_prev + cur * mul_cur) mod buckets]`` where ``prev`` is the token before
``t`` in its request; a request's first token takes the table's extra last row ``buckets``.  The token
before a step's first one is the request's state: one int32 per state slot, which the kernel reads
and then replaces by the step's last token, on the device (the ids of decoded tokens may exist there
only).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import STAGES, BuildContext, Stage, StateNeeds, TensorSpec


@STAGES.register("bigram_rows")
class BigramRows(Stage):
    graph_safe = True

    def __init__(self, ctx: BuildContext, width: int, buckets: int, mul_prev: int, mul_cur: int, tensor: str = "bigram"):
        self.ctx, self.width, self.buckets = ctx, width, int(buckets)
        self.mul_prev, self.mul_cur, self.tensor = int(mul_prev), int(mul_cur), tensor
        self.table = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.buckets + 1, self.width))}

    def bind(self, tensors):
        self.table = tensors[self.tensor].contiguous()

    def state_needs(self):
        return StateNeeds((), torch.int32)

    def forward(self, x, inputs):
        return ops.bigram_add(x, inputs.token_ids, inputs.token_row, inputs.row_start, inputs.row_pos, inputs.row_slot,
                              self.state, self.table, self.buckets, self.mul_prev, self.mul_cur)
