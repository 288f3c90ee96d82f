"""What a layer is made of, and how a part is found by its kind.

A model is put together from five kinds of part, each of which takes its sizes and constants
as parameters and knows nothing about the model it is in:

  mixer          mixes information across positions; may keep a per-token cache (keys and
                 values in pages), a per-request state of fixed size, or both
  feed_forward   position-wise (dense here; routed experts would be another kind)
  norm           normalises rows
  positions      tells the model where a token is: added to the embedding, or applied to
                 queries and keys inside a mixer
  block          arranges norms, a mixer and a feed-forward around the residual stream

Interfaces (duck-typed; `parts/attention.py`, `mlp.py`, `norm.py`, `positions.py`, `block.py`
are the GPT-2 ones):

  Mixer.cache_spec        -> MemberSpec | None     per-token cache need of this layer
  Mixer.state_spec        -> StateSpec | None      per-request state need of this layer
  Mixer.forward(h, residual, ctx, cache, state, writes_cache) -> new residual [T, D] float32
  FeedForward.forward(h, residual, ctx)            -> new residual [T, D] float32
  Norm.forward(x, out_dtype, rows=None)            -> normalised rows in out_dtype
  Positions.additive_table() -> Tensor | None      rows added to the token embedding
  Positions.rotate(q, k, ctx)                      in-place change of queries and keys (or no-op)
  Block.forward(x, ctx, cache, state, writes_cache) -> x

The residual stream `x` is float32 in every mode; `h` has the compute dtype. Each kind has a
registry from a name to a constructor `cls(params: dict, weights: dict, rt: Runtime)`; a
LayerSpec names the parts of one layer, so different layers of one model may use different ones.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..cache.arena import MemberSpec

__all__ = [
    "LayerSpec", "MemberSpec", "PartSpec", "Runtime", "StateSpec", "build_part", "register_block",
    "register_feed_forward", "register_mixer", "register_norm", "register_positions", "registry",
]


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one tensor row of this shape per request slot."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class Runtime:
    device: torch.device
    dtype: torch.dtype  # the compute dtype of activations and matrices: bfloat16 or float32


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict)
    weights: dict = field(default_factory=dict)  # the part's weight name -> checkpoint tensor name


@dataclass(frozen=True)
class LayerSpec:
    block: str  # arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    norm_1: PartSpec
    norm_2: PartSpec


_REGISTRIES: dict[str, dict[str, Callable[..., Any]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "positions": {}, "block": {},
}


def registry(family: str) -> dict[str, Callable[..., Any]]:
    return _REGISTRIES[family]


def _register(family: str, kind: str):
    def deco(cls):
        _REGISTRIES[family][kind] = cls
        return cls

    return deco


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feed_forward(kind: str):
    return _register("feed_forward", kind)


def register_norm(kind: str):
    return _register("norm", kind)


def register_positions(kind: str):
    return _register("positions", kind)


def register_block(kind: str):
    return _register("block", kind)


def build_part(family: str, spec: PartSpec, tensors: dict[str, torch.Tensor], rt: Runtime):
    """Construct the part that `spec` names, handing it its own weights under its own names."""
    try:
        cls = _REGISTRIES[family][spec.kind]
    except KeyError:
        raise KeyError(
            f"no {family} of kind {spec.kind!r}; registered: {sorted(_REGISTRIES[family])}"
        ) from None
    weights = {own: tensors[name] for own, name in spec.weights.items()}
    return cls(spec.params, weights, rt)
