"""From a model folder to a model on the GPU."""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.registry import load_config
from ..parts import Runtime
from ..weights.loader import load_weights
from . import gpt2  # noqa: F401  (registers the architecture)

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def compute_dtype(name: str) -> torch.dtype:
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


def load_model(model_dir: str | Path, dtype: str = "bfloat16", device: str | torch.device = "cuda:0"):
    """config.json picks the architecture; weights are checked against its spec; the model is
    built on `device` with `dtype` as compute dtype. No CPU execution path exists."""
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"the engine runs on a CUDA device only, got {device}")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available: the engine has no CPU fallback")
    arch, cfg = load_config(model_dir)
    tensors = load_weights(model_dir, arch.weight_spec(cfg))
    return arch.build(cfg, tensors, Runtime(device, compute_dtype(dtype)))
