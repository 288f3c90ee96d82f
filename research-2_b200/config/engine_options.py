"""Options of the engine around a model: capacity, batching budget, precision.

Names and meanings follow the reference where it has them: `max_requests`, `max_seq_len`,
`num_slabs` (kelpie-models/kelpie_models/sdk/tiers.py:41-48), `max_batch_tokens`,
`max_batch_reqs`, `reserve_ratio`, `order` (kelpie-engine/kelpie_engine/sdk/engine.py:107-135),
`capture` (kelpie-models/kelpie_models/sdk/run.py:139-157). With one cache group a slab is one
page (kelpie-core/src/kv_pool.zig:24-25), so `num_slabs` counts the pages of each group's pool.
"""

from __future__ import annotations

from dataclasses import dataclass

from .registry import ConfigError

DTYPES = ("bfloat16", "float32")
ORDERS = ("running_first", "waiting_first")
MAX_BUDGET = 8192  # the reference's ceiling for both budgets (kelpie-core/src/c_api.zig:467-478)


@dataclass(frozen=True)
class EngineOptions:
    dtype: str = "bfloat16"
    max_requests: int = 8
    max_seq_len: int = 0  # 0 = the model's own maximum
    block_size: int = 16  # tokens per cache page
    num_slabs: int = 0  # pages per cache group; 0 = enough for max_requests full sequences
    max_batch_tokens: int = 1024
    max_batch_reqs: int = 0  # 0 = min(256, max_requests)
    chunk_size: int = 0  # most rows of a prompt portion that does not finish its prompt; 0 = the token budget decides
    reserve_ratio: float = 0.0
    order: str = "running_first"
    capture: bool | None = None  # CUDA graphs for decode-only steps; None = on for bfloat16
    seed: int = 0

    def validated(self, model_max_seq_len: int) -> "EngineOptions":
        if self.dtype not in DTYPES:
            raise ConfigError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        if self.order not in ORDERS:
            raise ConfigError(f"order must be one of {ORDERS}, got {self.order!r}")
        if self.max_requests < 1:
            raise ConfigError(f"max_requests must be >= 1, got {self.max_requests}")
        if self.block_size < 1:
            raise ConfigError(f"block_size must be >= 1, got {self.block_size}")
        max_seq = self.max_seq_len or model_max_seq_len
        if not 1 <= max_seq <= model_max_seq_len:
            raise ConfigError(
                f"max_seq_len must be in [1, {model_max_seq_len}] (the model's limit), got {max_seq}"
            )
        if not 1 <= self.max_batch_tokens <= MAX_BUDGET:
            raise ConfigError(f"max_batch_tokens must be in [1, {MAX_BUDGET}], got {self.max_batch_tokens}")
        reqs = self.max_batch_reqs or min(256, self.max_requests)
        if not 1 <= reqs <= MAX_BUDGET:
            raise ConfigError(f"max_batch_reqs must be in [1, {MAX_BUDGET}], got {reqs}")
        if not 0 <= self.chunk_size <= self.max_batch_tokens:
            raise ConfigError(f"chunk_size must be 0 or in [1, max_batch_tokens = {self.max_batch_tokens}], got {self.chunk_size}")
        if (self.chunk_size or self.max_batch_tokens) < self.block_size:
            raise ConfigError(
                f"max_batch_tokens and chunk_size must be at least block_size ({self.block_size}): a portion that does "
                f"not finish its prompt ends on a page boundary, so a smaller budget could never run a longer prompt")
        if not 0.0 <= self.reserve_ratio <= 1.0:
            raise ConfigError(f"reserve_ratio must be in [0, 1], got {self.reserve_ratio}")
        pages_per_seq = -(-max_seq // self.block_size)
        slabs = self.num_slabs or self.max_requests * pages_per_seq
        if slabs < 1:
            raise ConfigError(f"num_slabs must be >= 1, got {slabs}")
        capture = self.capture if self.capture is not None else self.dtype == "bfloat16"
        return EngineOptions(
            dtype=self.dtype, max_requests=self.max_requests, max_seq_len=max_seq,
            block_size=self.block_size, num_slabs=slabs, max_batch_tokens=self.max_batch_tokens,
            max_batch_reqs=reqs, chunk_size=self.chunk_size, reserve_ratio=self.reserve_ratio, order=self.order,
            capture=capture, seed=self.seed,
        )
