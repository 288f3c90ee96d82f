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

    def _normed(self, norm, x, consumer):
        """A part that says `takes_lazy_norm` gets the norm unevaluated and may fuse it into its
        first matrix product; any other part gets a tensor."""
        if getattr(consumer, "takes_lazy_norm", False) and getattr(norm, "can_be_lazy", False):
            return norm.forward(x, self.compute_dtype, lazy=True)
        return norm.forward(x, self.compute_dtype)
