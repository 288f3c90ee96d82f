"""LayerNorm with statistics in float32.
Reference: kelpie-models/kelpie_models/kernels/ops/layer_norm.py:21-23."""

from __future__ import annotations

from ..kernels import ops
from .base import Runtime, register_norm
from .util import vector


@register_norm("layer_norm")
class LayerNorm:
    """params: eps. weights: gamma, beta."""

    can_be_lazy = True

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.eps = float(params["eps"])
        self.gamma = vector(weights["gamma"], rt)
        self.beta = vector(weights["beta"], rt)

    def layer_norm_params(self):
        """(gain, shift, eps): for a kernel that normalises rows itself."""
        return self.gamma, self.beta, self.eps

    def forward(self, x, out_dtype, rows=None, lazy: bool = False):
        """Normalised rows in out_dtype. With `lazy` the result is an `ops.NormedRows` that a
        following `ops.linear` may compute inside its own kernel."""
        if lazy:
            return ops.NormedRows(x, self.gamma, self.beta, self.eps, out_dtype, rows=rows)
        return ops.layer_norm(x, self.gamma, self.beta, self.eps, out_dtype, rows=rows)
