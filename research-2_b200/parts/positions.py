"""Learned absolute positions: a table row per position, added to the token embedding.
Positions are given per row by the batch, not counted from the start of the step
(kelpie-models/kelpie_models/models/torch/gpt2.py:90; kelpie-core/src/scheduler.zig:1340-1343)."""

from __future__ import annotations

from .base import Runtime, register_positions
from .util import matrix


@register_positions("learned")
class LearnedPositions:
    """params: n_positions. weights: table [n_positions, D]."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.table = matrix(weights["table"], rt)
        if self.table.shape[0] != int(params["n_positions"]):
            raise ValueError(f"positions: table {tuple(self.table.shape)} has not {params['n_positions']} rows")

    def additive_table(self):
        return self.table

    def rotate(self, q, k, ctx) -> None:
        """Learned positions leave queries and keys alone."""
