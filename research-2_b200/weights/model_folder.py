"""The random-weights mode: write a model folder from a configuration and a seed."""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.registry import Architecture
from .safetensors_io import write_file

STORE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def write_model_folder(  # noqa: PLR0913
    folder: str | Path, arch: Architecture, config, seed: int, store_dtype: str = "bfloat16",
    **init_options,
) -> Path:
    """Draw weights for `config` from `seed` and write config.json + model.safetensors.
    The draw is made in float32 on the CPU and then rounded to `store_dtype`."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    dtype = STORE_DTYPES[store_dtype]
    tensors = arch.random_weights(config, seed, **init_options)
    stored = {name: (t if t.dtype == torch.int32 else t.to(dtype)) for name, t in tensors.items()}
    data = arch.config_to_json(config)
    data["torch_dtype"] = store_dtype
    (folder / "config.json").write_text(json.dumps(data, indent=1) + "\n")
    write_file(folder / "model.safetensors", stored)
    return folder
