"""Token embedding and the output head.

The embedding gathers table rows into the float32 residual stream, adding the rows of an
additive position table in the same kernel. The head normalises only the rows whose logits
are wanted and multiplies them with the [V, D] table (`x @ table^T`); GPT-2 ties the two
tables (kelpie-models/kelpie_models/models/torch/gpt2.py:70,98-101).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Runtime
from .util import matrix


class TokenEmbedding:
    def __init__(self, table: torch.Tensor, rt: Runtime):
        self.table = matrix(table, rt)

    def forward(self, ctx, additive_table=None):
        return ops.embed(ctx.input_ids, self.table, ctx.positions, additive_table)


class Head:
    """logits[i] = norm(x[rows[i]]) @ table^T, float32."""

    def __init__(self, norm, table: torch.Tensor, compute_dtype: torch.dtype):
        self.norm, self.table, self.compute_dtype = norm, table, compute_dtype

    def forward(self, x, rows):
        lazy = getattr(self.norm, "can_be_lazy", False)
        last = self.norm.forward(x, self.compute_dtype, rows=rows, lazy=True) if lazy else self.norm.forward(x, self.compute_dtype, rows=rows)
        return ops.linear(last, self.table, None, w_is_nk=True, out_dtype=torch.float32)
