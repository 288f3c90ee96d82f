"""The step function: one batch of (request, its next tokens) in, logits at the wanted rows out.

It runs only the tokens it is given, as one batch, against the cache that earlier steps left,
and returns float32 logits [n_logit_rows, vocab]. It owns the cache memory (the arena and the
state tensors) and writes it in place; the cache manager and the scheduler own the indices.
Reference shape of this seam: `Step.forward(plan) -> logits`
(kelpie-models/kelpie_models/sdk/step.py:102-184), `to_device`
(kelpie-models/kelpie_models/sdk/device.py:124-149).
"""

from __future__ import annotations

import numpy as np
import torch

from ..cache.arena import KVArena, derive_groups
from ..cache.manager import GroupSpec
from .batch import BatchLayout, StepBatch


class StepContext:
    """What parts may read about the current step: the batch's arrays on the device (int32),
    and the same batch on the host for decisions that shape launches."""

    def __init__(self, host: StepBatch, dev: torch.Tensor):
        self.host = host
        self.n_tokens, self.n_entries, self.n_logit_rows = host.n_tokens, host.n_entries, host.n_logit_rows
        t, r, w = host.n_tokens, host.n_entries, host.n_logit_rows

        def view(name: str, count: int) -> torch.Tensor:
            at, _ = host.section(name)
            return dev[at: at + count]

        self.input_ids = view("input_ids", t)
        self.positions = view("positions", t)
        self.row_entry = view("row_entry", t)
        self.q_start = view("q_start", r + 1)
        self.seq_lens = view("seq_lens", r)
        self.state_slot = view("state_slot", r)
        self.fresh = view("fresh", r)
        self.logit_rows = view("logit_rows", w)
        at, _ = host.section("slot_mapping")
        self.slot_mapping = [dev[at + g * host.t_cap: at + g * host.t_cap + t] for g in range(len(host.block_tables))]
        at, _ = host.section("block_tables")
        self.block_tables = []
        for width in host.layout.table_widths:
            self.block_tables.append(dev[at: at + r * width].view(r, width))
            at += host.r_cap * width


class StepFunction:
    def __init__(self, model, page_size: int, num_pages: int, max_requests: int):
        self.model = model
        self.device = model.rt.device
        self.groups, self.member_group = derive_groups(model.cache_members, page_size, num_pages)
        self.arena = KVArena(model.cache_members, self.groups, self.member_group, model.rt.dtype, self.device)
        self.state_tensors = [
            torch.zeros((max_requests,) + tuple(spec.shape), dtype=spec.dtype, device=self.device)
            for spec in model.state_members
        ]
        self.max_requests = max_requests
        self.table_widths = tuple(-(-model.max_seq_len // g.page_size) for g in self.groups)
        self.launches = 0

    def cache_groups(self) -> list[GroupSpec]:
        return list(self.groups)

    def new_batch(self, n_tokens: int, n_entries: int, n_logit_rows: int, widths=None) -> StepBatch:
        layout = BatchLayout(n_tokens, n_entries, n_logit_rows, tuple(widths or self.table_widths))
        return StepBatch(layout, pinned=True)

    def upload(self, batch: StepBatch) -> StepContext:
        batch.pad()
        dev = torch.empty(batch.buf.shape[0], dtype=torch.int32, device=self.device)
        src = batch._pinned_tensor if batch._pinned_tensor is not None else torch.from_numpy(batch.buf)
        dev.copy_(src, non_blocking=True)
        return StepContext(batch, dev)

    def validate(self, batch: StepBatch) -> None:
        """Host-side bounds checks (there is no device-side sanitizer to lean on)."""
        batch.check()
        t = batch.n_tokens
        if t and (batch.input_ids[:t].min() < 0 or batch.input_ids[:t].max() >= self.model.vocab_size):
            raise ValueError(f"a token id lies outside the vocabulary [0, {self.model.vocab_size})")
        for g, spec in enumerate(self.groups):
            limit = (spec.num_pages + 1) * spec.page_size
            if t and (batch.slot_mapping[g, :t].min() < spec.page_size or batch.slot_mapping[g, :t].max() >= limit):
                raise ValueError(f"group {g}: a slot lies outside the pool or in the null page")
            table = batch.block_tables[g][: batch.n_entries]
            if table.size and (table.min() < 0 or table.max() > spec.num_pages):
                raise ValueError(f"group {g}: a block table names a page outside the pool")
        if t and batch.seq_lens[: batch.n_entries].max() > self.model.max_seq_len:
            raise ValueError("an entry reaches beyond max_seq_len")

    @torch.no_grad()
    def __call__(self, batch: StepBatch) -> torch.Tensor:
        if batch.n_tokens == 0:
            return torch.empty(0, self.model.vocab_size, dtype=torch.float32, device=self.device)
        self.validate(batch)
        with torch.cuda.device(self.device):
            ctx = self.upload(batch)
            logits = self.model.forward(ctx, self.arena.members, self.state_tensors)
        return logits[: batch.n_logit_rows]


def logit_rows_of_last(batch: StepBatch) -> np.ndarray:
    return batch.last_rows().astype(np.int32)
