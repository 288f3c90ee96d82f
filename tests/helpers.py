"""Shared pieces of the tests: the two tiny configurations, model folders in temporary
directories, the plain implementation's logits, and the error budget."""

from __future__ import annotations

import functools
from pathlib import Path

import numpy as np
import torch

from tests.plain import gpt2_plain

# Two tiny GPT-2 configurations that differ in every size and option.
TINY_A = {
    "config": {
        "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
        "n_layer": 2, "n_embd": 64, "n_head": 4, "n_inner": 256, "vocab_size": 512, "n_positions": 128,
        "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5, "scale_attn_weights": True,
        "scale_attn_by_inverse_layer_idx": False, "tie_word_embeddings": True, "eos_token_id": 511,
    },
    "seed": 0, "std": 0.02, "store_dtype": "float32", "page_size": 16,
}
TINY_B = {
    "config": {
        "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
        "n_layer": 3, "n_embd": 96, "n_head": 3, "n_inner": 320, "vocab_size": 1031, "n_positions": 256,
        "activation_function": "gelu", "layer_norm_epsilon": 1e-6, "scale_attn_weights": True,
        "scale_attn_by_inverse_layer_idx": True, "tie_word_embeddings": True, "eos_token_id": None,
    },
    "seed": 2, "std": 0.05, "store_dtype": "bfloat16", "page_size": 8,
}
# Head size 64 (what the tcgen05 prefill attention and the 4-D tensor copies are built for) at a
# width, a hidden size and a vocabulary that are no power of two.
TINY_C = {
    "config": {
        "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
        "n_layer": 2, "n_embd": 192, "n_head": 3, "n_inner": 448, "vocab_size": 777, "n_positions": 512,
        "activation_function": "gelu_new", "layer_norm_epsilon": 3e-6, "scale_attn_weights": True,
        "scale_attn_by_inverse_layer_idx": True, "tie_word_embeddings": True, "eos_token_id": None,
    },
    "seed": 9, "std": 0.04, "store_dtype": "bfloat16", "page_size": 16,
}
TINY = {"a": TINY_A, "b": TINY_B, "c": TINY_C}


def make_model_dir(folder: Path, tiny: dict, std: float | None = None) -> Path:
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.models import gpt2  # noqa: F401
    from research_2_b200.weights import write_model_folder

    arch = architecture_of(tiny["config"])
    cfg = arch.parse_config(tiny["config"])
    return write_model_folder(folder, arch, cfg, tiny["seed"], tiny["store_dtype"], std=std or tiny["std"])


def random_tokens(seed: int, n: int, vocab: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


@functools.lru_cache(maxsize=64)
def _plain_cached(folder: str, ids: tuple, dtype_name: str) -> np.ndarray:
    dtype = {"float32": torch.float32, "float64": torch.float64}[dtype_name]
    w, cfg = gpt2_plain.read_model(folder, dtype)
    return gpt2_plain.forward(w, cfg, torch.tensor(ids)).numpy()


def plain_logits(folder, ids, dtype_name: str = "float32") -> np.ndarray:
    """Logits [T, V] of the plain implementation for one whole sequence."""
    return _plain_cached(str(folder), tuple(int(i) for i in ids), dtype_name)


FLOORS = {"float32": 2e-5, "bfloat16": 2e-2}


def budget(folder, ids, dtype_name: str) -> tuple[np.ndarray, float]:
    """(truth, allowed max-abs error): the reference's rule for grading a kernel,
    err <= max(2 * err_ref, floor * max|truth|) with truth in float64, err_ref the plain
    implementation's own float32 error, floors 2e-5 (float32) and 2e-2 (bfloat16)
    (kelpie-models/kelpie_models/bench/correctness.py:28-51; bench/compare.py:34-52)."""
    truth = plain_logits(folder, ids, "float64")
    err_ref = float(np.abs(plain_logits(folder, ids, "float32") - truth).max())
    return truth, max(2.0 * err_ref, FLOORS[dtype_name] * float(np.abs(truth).max()))


def assert_within_budget(got: np.ndarray, folder, ids, dtype_name: str, positions=None, what: str = "") -> None:
    truth, allowed = budget(folder, ids, dtype_name)
    if positions is not None:
        truth = truth[list(positions)]
    assert got.shape == truth.shape, (got.shape, truth.shape, what)
    err = np.abs(got.astype(np.float64) - truth)
    worst = float(err.max())
    if not worst <= allowed:
        row = int(np.unravel_index(err.argmax(), err.shape)[0])
        first_bad = int(np.argmax(err.max(axis=1) > allowed))
        pos = list(positions)[first_bad] if positions is not None else first_bad
        raise AssertionError(
            f"{what}: max |logit - truth| = {worst:.3e} > allowed {allowed:.3e} "
            f"(worst row {row}; first row over budget is at position {pos})"
        )
