"""Arrangements of norms, a mixer and a feed-forward around the float32 residual stream."""

from __future__ import annotations

from .base import register_block


@register_block("pre_norm")
class PreNormBlock:
    """x + mixer(norm_1 x), then x + feed_forward(norm_2 x); both additions happen in the
    epilogue of each part's last matrix product
    (kelpie-models/kelpie_models/models/torch/gpt2.py:91-97)."""

    def __init__(self, norm_1, mixer, norm_2, feed_forward, compute_dtype):
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self.compute_dtype = compute_dtype

    def forward(self, x, ctx, cache=None, state=None, writes_cache: bool = True):
        h = self._normed(self.norm_1, x, self.mixer)
        x = self.mixer.forward(h, x, ctx, cache, state, writes_cache)
        h = self._normed(self.norm_2, x, self.feed_forward)
        return self.feed_forward.forward(h, x, ctx)

    def resident_layer(self) -> dict | None:
        """What the one-kernel form of a decode step (parts/resident.py) needs to know of this layer, or
        None if one of its parts is not of a kind that the kernel is written for."""
        asks = (getattr(self.norm_1, "layer_norm_params", None), getattr(self.mixer, "resident_attention", None),
                getattr(self.norm_2, "layer_norm_params", None), getattr(self.feed_forward, "resident_mlp", None))
        if any(ask is None for ask in asks):
            return None
        n1, attention, n2, mlp = (ask() for ask in asks)
        if attention is None or mlp is None or attention["width"] != mlp["width"]:
            return None
        return {**attention, **mlp, "ln1_g": n1[0], "ln1_b": n1[1], "eps1": n1[2], "ln2_g": n2[0], "ln2_b": n2[1], "eps2": n2[2]}

    def _normed(self, norm, x, consumer):
        """A part that says `takes_lazy_norm` gets the norm unevaluated and may fuse it into its
        first matrix product; any other part gets a tensor."""
        if getattr(consumer, "takes_lazy_norm", False) and getattr(norm, "can_be_lazy", False):
            return norm.forward(x, self.compute_dtype, lazy=True)
        return norm.forward(x, self.compute_dtype)
