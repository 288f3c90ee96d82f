from . import attention, block, embedding, mlp, norm, positions  # noqa: F401  (registers the parts)
from .base import (
    LayerSpec, MemberSpec, PartSpec, Runtime, StateSpec, build_part, register_block, register_feed_forward,
    register_mixer, register_norm, register_positions, registry,
)

__all__ = [
    "LayerSpec", "MemberSpec", "PartSpec", "Runtime", "StateSpec", "build_part", "register_block",
    "register_feed_forward", "register_mixer", "register_norm", "register_positions", "registry",
]
