"""Sampling is one kernel (csrc/kernels/sampling.cu) behind `kernels.ops.sample`; the per-request
parameters (temperature, top_k, seed: kelpie-engine/kelpie_engine/sdk/engine.py:284-305) travel in the
step batch, which the scheduler fills. `sampling_parameters` is the one place that turns a request's
options into what the kernel reads, for callers that build a batch by hand."""

from __future__ import annotations

SAMPLING_EPS = 1e-6  # below this a temperature means greedy (kelpie-core/src/request.zig:118-144)


def sampling_parameters(temperature: float, top_k: int, seed: int) -> tuple[float, int, int, int]:
    """(temperature, top_k, key0, key1) as the kernel reads them: greedy is (1.0, 1); the Philox
    key is the seed's low and high 32 bits."""
    if temperature < SAMPLING_EPS:
        temperature, top_k = 1.0, 1
    return float(temperature), int(top_k), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF


__all__ = ["SAMPLING_EPS", "sampling_parameters"]
