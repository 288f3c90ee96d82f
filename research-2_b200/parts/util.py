"""How parts hold their weights: matrices in the compute dtype, vectors in float32."""

from __future__ import annotations

import torch

from .base import Runtime


def matrix(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """A matrix or table on the device in the compute dtype (bfloat16 serving, or float32)."""
    return t.to(device=rt.device, dtype=rt.dtype).contiguous()


def vector(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """Biases and norm parameters stay float32: they enter sums that are kept in 32-bit."""
    return t.to(device=rt.device, dtype=torch.float32).contiguous()
