"""The dense feed-forward: act(h @ w_in + b_in) @ w_out + b_out, added to the residual stream.
Reference: kelpie-models/kelpie_models/models/torch/gpt2.py:94-96."""

from __future__ import annotations

from ..kernels import ops
from .base import Runtime, register_feed_forward
from .util import matrix, vector


@register_feed_forward("mlp")
class DenseMLP:
    """params: activation ("gelu_new" | "gelu"). weights: w_in [D, F], b_in, w_out [F, D], b_out,
    both matrices stored [in, out]; the inner width F is the weights' own."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.activation = params["activation"]
        if self.activation not in ops.ACTIVATIONS or self.activation in (None, "none"):
            raise ValueError(f"mlp: unknown activation {self.activation!r}")
        self.w_in = matrix(weights["w_in"], rt)
        self.b_in = vector(weights["b_in"], rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.b_out = vector(weights["b_out"], rt)
        if self.w_in.shape[1] != self.w_out.shape[0] or self.w_in.shape[0] != self.w_out.shape[1]:
            raise ValueError(f"mlp: w_in {tuple(self.w_in.shape)} and w_out {tuple(self.w_out.shape)} do not fit")

    takes_lazy_norm = True  # the input goes straight into ops.linear

    def matrices(self):
        """The weight matrices in the order in which forward() uses them."""
        return [self.w_in, self.w_out]

    def resident_mlp(self) -> dict:
        return {"w_fc": self.w_in, "b_fc": self.b_in, "w_pr": self.w_out, "b_pr": self.b_out, "act": self.activation,
                "width": self.w_in.shape[0], "inner": self.w_in.shape[1]}

    def forward(self, h, residual, ctx):
        return ops.mlp(h, self.w_in, self.b_in, self.activation, self.w_out, self.b_out, residual=residual)
