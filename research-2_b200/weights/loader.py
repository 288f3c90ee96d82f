"""Weights by tensor name, checked against what the architecture says it needs.

The reference looks each name up bare and then with a `transformer.` prefix, raises KeyError on
the first missing one and asserts two shapes (kelpie-models/kelpie_models/models/torch/gpt2.py:
157-188). Here every tensor is checked and ONE error lists all that is missing, unexpected or
of the wrong shape. Stored precision is kept: a bfloat16 tensor stays bfloat16, a 32-bit one
stays 32-bit, integer tables become int32; the model casts what its compute path needs.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, read_folder

FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16)
INT_DTYPES = (torch.int32, torch.int64, torch.uint8)


class WeightError(ValueError):
    """The checkpoint does not fit the configuration. `missing`, `unexpected` and `wrong`
    hold the details that the message lists."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong = list(wrong)


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple[int, ...]
    integer: bool = False


@dataclass(frozen=True)
class WeightSpec:
    tensors: tuple[TensorSpec, ...]
    prefixes: tuple[str, ...] = ("",)  # spellings tried in order, e.g. ("", "transformer.")
    ignorable: tuple[str, ...] = field(default=())  # regexes of names that may be present and are not read
    # (stored name, spec name): a tensor that may be stored beside the one it is tied to; it is
    # not read, but it must hold the same values, else the checkpoint is not the tied model it claims to be
    tied: tuple[tuple[str, str], ...] = field(default=())


def check_and_select(found: dict[str, torch.Tensor], spec: WeightSpec, where: str = "checkpoint") -> dict[str, torch.Tensor]:
    """Pick the spec's tensors out of `found` (bare names in the result) or raise WeightError."""
    missing: list[str] = []
    wrong: list[str] = []
    used: set[str] = set()
    out: dict[str, torch.Tensor] = {}
    for ts in spec.tensors:
        spellings = [p + ts.name for p in spec.prefixes]
        key = next((s for s in spellings if s in found), None)
        if key is None:
            missing.append(" or ".join(spellings))
            continue
        used.add(key)
        tensor = found[key]
        if tuple(tensor.shape) != tuple(ts.shape):
            wrong.append(f"{key}: expected shape {tuple(ts.shape)}, got {tuple(tensor.shape)}")
            continue
        if ts.integer:
            if tensor.dtype not in INT_DTYPES:
                wrong.append(f"{key}: expected an integer table, got {tensor.dtype}")
                continue
            tensor = tensor.to(torch.int32)
        else:
            if tensor.dtype not in FLOAT_DTYPES:
                wrong.append(f"{key}: expected a floating-point tensor, got {tensor.dtype}")
                continue
            if tensor.dtype == torch.float16:
                tensor = tensor.to(torch.bfloat16)
        out[ts.name] = tensor
    for alias, target in spec.tied:
        if alias not in found:
            continue
        used.add(alias)
        if target not in out:
            continue  # already reported as missing or wrong
        copy, kept = found[alias], out[target]
        if tuple(copy.shape) != tuple(kept.shape):
            wrong.append(f"{alias}: tied to {target} of shape {tuple(kept.shape)}, got {tuple(copy.shape)}")
        elif not torch.equal(copy.to(torch.float32), kept.to(torch.float32)):
            gap = float((copy.to(torch.float32) - kept.to(torch.float32)).abs().max())
            wrong.append(f"{alias}: tied to {target} but its values differ (max |difference| {gap:.3g}); "
                         f"an untied head is not supported")
    ignorable = [re.compile(p) for p in spec.ignorable]
    unexpected = sorted(
        name for name in found
        if name not in used and not any(rx.fullmatch(name) for rx in ignorable)
    )
    if missing or wrong or unexpected:
        parts = [f"{where} does not fit the configuration:"]
        if missing:
            parts.append(f"  missing ({len(missing)}): " + "; ".join(missing))
        if unexpected:
            parts.append(f"  unexpected ({len(unexpected)}): " + "; ".join(unexpected))
        if wrong:
            parts.append(f"  wrong ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(parts), missing, unexpected, wrong)
    return out


def load_weights(model_dir: str | Path, spec: WeightSpec) -> dict[str, torch.Tensor]:
    try:
        found = read_folder(model_dir)
    except SafetensorsError as err:
        raise WeightError(str(err)) from None
    return check_and_select(found, spec, where=str(model_dir))
