"""The batch of one step: (request, its next tokens) entries, as flat int32 arrays.

An entry is `rows` tokens of one request at positions [start, start + rows): a portion of a
prompt, or one decoded token. All entries of a step run as one batch. The arrays are those of
the reference's plan (kelpie-core/include/kelpie.h:115-185; device form
kelpie-models/kelpie_models/sdk/device.py:26-78): per row `input_ids positions row_entry
slot_mapping[g]`, per entry `q_start seq_lens block_tables[g] state_slot fresh`, plus
`logit_rows`, the rows whose logits are wanted. They live in ONE buffer so that a step costs
one host-to-device copy. Capacities may exceed the counts; pads are inert by value: pad rows
have row_entry -1 and write the null page's slot 0, pad entries are empty.
"""

from __future__ import annotations

from dataclasses import dataclass

import ctypes as C

import numpy as np

_ALIGN = 4  # sections start on 16-byte boundaries


def _round(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


@dataclass(frozen=True)
class BatchLayout:
    t_cap: int
    r_cap: int
    w_cap: int
    table_widths: tuple[int, ...]

    def sections(self) -> dict[str, tuple[int, int]]:
        g = len(self.table_widths)
        sizes = [
            ("input_ids", self.t_cap), ("positions", self.t_cap), ("row_entry", self.t_cap),
            ("q_start", self.r_cap + 1), ("seq_lens", self.r_cap), ("state_slot", self.r_cap),
            ("fresh", self.r_cap), ("logit_rows", self.w_cap), ("temperature", self.w_cap), ("top_k", self.w_cap),
            ("key0", self.w_cap), ("key1", self.w_cap), ("sample_pos", self.w_cap), ("slot_mapping", g * self.t_cap),
            ("block_tables", self.r_cap * sum(self.table_widths)),
        ]
        out, at = {}, 0
        for name, size in sizes:
            out[name] = (at, size)
            at += _round(max(size, 1))
        out["_total"] = (0, at)
        return out


class StepBatch:
    """Host side of a batch. `buf` is one int32 array (pinned when a CUDA device is there)."""

    def __init__(self, layout: BatchLayout, pinned: bool = False):
        self.layout = layout
        self.t_cap, self.r_cap, self.w_cap = layout.t_cap, layout.r_cap, layout.w_cap
        self._sections = layout.sections()
        total = self._sections["_total"][1]
        self._pinned_tensor = None
        if pinned:
            import torch

            self._pinned_tensor = torch.zeros(total, dtype=torch.int32).pin_memory()
            self.buf = self._pinned_tensor.numpy()
        else:
            self.buf = np.zeros(total, dtype=np.int32)
        for name, (at, size) in self._sections.items():
            if not name.startswith("_"):
                setattr(self, name if name not in ("slot_mapping", "block_tables") else name + "_flat",
                        self.buf[at: at + size])
        g = len(layout.table_widths)
        self.slot_mapping = self.slot_mapping_flat.reshape(g, self.t_cap)
        self.block_tables = []
        at = 0
        for width in layout.table_widths:
            self.block_tables.append(self.block_tables_flat[at: at + self.r_cap * width].reshape(self.r_cap, width))
            at += self.r_cap * width
        # host-only facts about the entries
        self.entry_req = np.zeros(max(self.r_cap, 1), dtype=np.int32)
        self.entry_start = np.zeros(max(self.r_cap, 1), dtype=np.int32)
        self.entry_rows = np.zeros(max(self.r_cap, 1), dtype=np.int32)
        self.n_entries = 0
        self.n_tokens = 0
        self.n_logit_rows = 0
        self.trusted = False   # filled and padded natively by the scheduler: nothing left to pad or check
        self._native = None

    def native(self):
        """The batch's arrays as the native side's struct (made once: the buffer never moves)."""
        if self._native is None:
            from ..cache import _host

            n = _host.StepBatchC()
            n.t_cap, n.r_cap, n.w_cap = self.t_cap, self.r_cap, self.w_cap
            for name in ("input_ids", "positions", "row_entry", "q_start", "seq_lens", "state_slot", "fresh", "logit_rows",
                         "temperature", "top_k", "key0", "key1", "sample_pos"):
                setattr(n, name, getattr(self, name).ctypes.data)
            n.slot_mapping = self.slot_mapping_flat.ctypes.data
            n.block_tables = self.block_tables_flat.ctypes.data
            n.entry_req, n.entry_start, n.entry_rows = (a.ctypes.data for a in (self.entry_req, self.entry_start, self.entry_rows))
            self._native = n
        return self._native

    def section(self, name: str) -> tuple[int, int]:
        return self._sections[name]

    def set_entries(self, reqs, starts, token_lists) -> None:
        """Entries in batch order; `token_lists[i]` are entry i's tokens."""
        n = len(reqs)
        total = sum(len(t) for t in token_lists)
        if n > self.r_cap or total > self.t_cap:
            raise ValueError(f"batch of {n} entries / {total} rows exceeds its capacity {self.r_cap} / {self.t_cap}")
        self.n_entries, self.n_tokens = n, total
        self.trusted = False
        at = 0
        for i, (req, start, toks) in enumerate(zip(reqs, starts, token_lists)):
            if len(toks) < 1:
                raise ValueError(f"entry {i} (request {req}) has no tokens")
            self.entry_req[i], self.entry_start[i], self.entry_rows[i] = req, start, len(toks)
            self.input_ids[at: at + len(toks)] = toks
            at += len(toks)

    def set_logit_rows(self, rows) -> None:
        rows = np.asarray(rows, dtype=np.int32).reshape(-1)
        if len(rows) > self.w_cap:
            raise ValueError(f"{len(rows)} logit rows exceed the capacity {self.w_cap}")
        if len(rows) and (rows.min() < 0 or rows.max() >= self.n_tokens):
            raise ValueError(f"logit rows must lie in [0, {self.n_tokens})")
        self.n_logit_rows = len(rows)
        self.logit_rows[: len(rows)] = rows
        self.logit_rows[len(rows):] = 0

    def set_sampling(self, temperature, top_k, key0, key1, sample_pos) -> None:
        """Per logit row: temperature (> 0), top_k, the request's Philox key, and the position
        of the token that is drawn. Rows beyond the count are greedy and inert."""
        n = self.n_logit_rows
        self.temperature.view(np.float32)[:n] = np.asarray(temperature, dtype=np.float32)
        self.temperature.view(np.float32)[n:] = 1.0
        self.top_k[:n] = np.asarray(top_k, dtype=np.int32)
        self.top_k[n:] = 1
        self.key0[:n] = np.asarray(key0, dtype=np.uint32).view(np.int32)
        self.key1[:n] = np.asarray(key1, dtype=np.uint32).view(np.int32)
        self.sample_pos[:n] = np.asarray(sample_pos, dtype=np.int32)
        self.key0[n:] = 0
        self.key1[n:] = 0
        self.sample_pos[n:] = 0

    def last_rows(self) -> np.ndarray:
        """The last row of each entry (the reference's `last_rows`, sdk/device.py:130)."""
        return self.q_start[1: self.n_entries + 1] - 1

    def pad(self) -> None:
        """Make everything beyond the counts inert (call after the cache manager's fill)."""
        t, r = self.n_tokens, self.n_entries
        self.input_ids[t:] = 0
        self.positions[t:] = 0
        self.row_entry[t:] = -1
        self.slot_mapping[:, t:] = 0
        self.q_start[r + 1:] = t
        self.seq_lens[r:] = 0
        self.state_slot[r:] = 0
        self.fresh[r:] = 0
        for table in self.block_tables:
            table[r:] = 0

    def check(self, limits: "BatchLimits") -> None:
        """Host-side bounds checks of a batch that the caller filled (there is no device-side
        sanitizer to lean on), in one native pass over the rows: every row belongs to an entry of
        the batch and an entry's rows are its newest positions (the invariant that the reference
        asserts on the device, kernels/ops/paged_attention.py:143-157); token ids lie in the
        vocabulary; slots and block-table entries lie inside the pool; no entry reaches beyond
        the longest sequence."""
        from ..cache import _host

        where = C.c_int32(-1)
        code = _host.lib().r2_step_batch_check(C.byref(self.native()), self.n_tokens, self.n_entries, limits.vocab_size,
                                               limits.max_seq_len, limits.groups, limits.table_widths, limits.n_groups, C.byref(where))
        if code == 0:
            return
        if code == 1:
            raise AssertionError("a row names an entry outside the batch")
        if code == 2:
            raise AssertionError(f"entry {where.value}: rows are not its newest positions")
        raise ValueError({
            3: f"a token id lies outside the vocabulary [0, {limits.vocab_size})",
            4: f"group {where.value}: a slot lies outside the pool or in the null page",
            5: f"group {where.value}: a block table names a page outside the pool",
            6: "an entry reaches beyond max_seq_len",
        }[code])


class BatchLimits:
    """What a batch is checked against, in the native side's types (made once per step function)."""

    def __init__(self, vocab_size: int, max_seq_len: int, groups, table_widths):
        from ..cache import _host

        self.vocab_size, self.max_seq_len, self.n_groups = int(vocab_size), int(max_seq_len), len(groups)
        self.groups = (_host.GroupSpecC * len(groups))(*[_host.GroupSpecC(g.page_size, g.window, g.num_pages) for g in groups])
        self.table_widths = (C.c_int32 * len(groups))(*[int(w) for w in table_widths])


def batch_for(table_widths, n_tokens: int, n_entries: int, n_logit_rows: int, pinned: bool = False) -> StepBatch:
    return StepBatch(BatchLayout(n_tokens, n_entries, n_logit_rows, tuple(table_widths)), pinned=pinned)
