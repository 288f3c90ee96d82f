"""Multi-head (or grouped) causal attention over the paged cache.

Formulas of the reference (kelpie-models/kelpie_models/models/torch/gpt2.py:104-131 and
kernels/ops/paged_attention.py): one fused projection to q, k, v (in that order along the
output), keys and values written to the cache before attention reads it, scores scaled by
`scale`, causal mask (and a window when `window` > 0), softmax and P.V in float32, then the
output projection, whose epilogue adds the residual stream.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import MemberSpec, Runtime, register_mixer
from .util import matrix, vector


@register_mixer("attention")
class PagedAttention:
    """params: n_heads, n_kv_heads, head_dim, scale, window (0 = none).
    weights: w_qkv [D, (n_heads + 2 n_kv_heads) * head_dim] stored [in, out], b_qkv,
    w_out [n_heads * head_dim, D] stored [in, out], b_out."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = int(params.get("window", 0))
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"attention: n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv_heads}")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"attention: head sizes come in steps of 16 from 16 to 256, got {self.head_dim}")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.w_qkv = matrix(weights["w_qkv"], rt)
        self.b_qkv = vector(weights["b_qkv"], rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.b_out = vector(weights["b_out"], rt)
        if self.w_qkv.shape[1] != self.q_width + 2 * self.kv_width or self.w_out.shape[0] != self.q_width:
            raise ValueError(f"attention: weights {tuple(self.w_qkv.shape)} / {tuple(self.w_out.shape)} do not fit "
                             f"{self.n_heads} heads, {self.n_kv_heads} kv heads of {self.head_dim}")
        self.rotary = None  # a positions part that changes q and k may be attached by the model

    def matrices(self):
        """The weight matrices in the order in which forward() uses them."""
        return [self.w_qkv, self.w_out]

    @property
    def cache_spec(self) -> MemberSpec:
        return MemberSpec(self.n_kv_heads, self.head_dim, self.window)

    state_spec = None
    capturable = True  # nothing here depends on the batch's contents, only on its shape
    takes_lazy_norm = True  # the input goes straight into ops.linear

    def resident_attention(self) -> dict | None:
        """For the one-kernel form of a decode step; None while a positions part rotates q and k."""
        if self.rotary is not None or self.w_out.shape[1] != self.w_qkv.shape[0]:
            return None
        return {"w_qkv": self.w_qkv, "b_qkv": self.b_qkv, "w_out": self.w_out, "b_out": self.b_out, "n_heads": self.n_heads,
                "n_kv_heads": self.n_kv_heads, "head_dim": self.head_dim, "scale": self.scale, "window": self.window,
                "width": self.w_qkv.shape[0]}

    def forward(self, h, residual, ctx, cache, state=None, writes_cache: bool = True):
        in_cache = False
        if writes_cache and not ctx.decode_only and self.rotary is None:
            # keys and values leave the product's epilogue for their cache slots (where that kernel takes the shape)
            qkv, in_cache = ops.linear(h, self.w_qkv, self.b_qkv, kv=ops.kv_scatter(
                ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride, cache.page_size, cache.n_pages,
                self.q_width, self.kv_width, self.head_dim))
        else:
            qkv = ops.linear(h, self.w_qkv, self.b_qkv)
        q = qkv[:, : self.q_width]
        k = qkv[:, self.q_width: self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if self.rotary is not None:
            self.rotary.rotate(q, k, ctx)
        if writes_cache and ctx.decode_only:
            mixed = ops.decode_attention_fused(
                q, k, v, ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride, cache.page_size,
                cache.n_pages, ctx.block_tables[cache.group], ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads,
                self.n_kv_heads, self.head_dim, self.scale, self.window, ctx.max_context)
            if mixed is not None:
                return ops.linear(mixed, self.w_out, self.b_out, residual=residual)
        if writes_cache and not in_cache:
            ops.kv_write(k, v, cache.k, cache.v, ctx.slot_mapping[cache.group], self.n_kv_heads, self.head_dim,
                         cache.page_size, cache.page_stride, cache.n_pages)
        mixed = ops.paged_attention(
            q, cache.k, cache.v, cache.page_stride, cache.page_size, cache.n_pages, ctx.block_tables[cache.group],
            ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
            self.window, decode_only=ctx.decode_only, max_context=ctx.max_context, q_start=ctx.q_start,
            n_tiles=ctx.n_attention_tiles)
        return ops.linear(mixed, self.w_out, self.b_out, residual=residual)
