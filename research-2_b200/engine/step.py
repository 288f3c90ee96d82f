"""The step function: one batch of (request, its next tokens) in, logits at the wanted rows out.

It runs only the tokens it is given, as one batch, against the cache that earlier steps left,
and returns float32 logits [n_logit_rows, vocab]; `sample` turns them into one token per row
on the device. It owns the cache memory (the arena and the state tensors) and writes it in
place; the cache manager and the scheduler own the indices. Reference shape of this seam:
`Step.forward(plan) -> logits`, `Step.sample` (kelpie-models/kelpie_models/sdk/step.py:102-184),
`to_device` (kelpie-models/kelpie_models/sdk/device.py:124-149).

With `capture` on, a step runs as a CUDA graph per shape bucket: the batch is copied into the
graph's static buffer and the graph is replayed; forward pass and sampling are both inside it.
Decode-only batches (every entry one row) have a bucket per batch size, captured at first use,
as the reference captures its decode buckets (kelpie-models/kelpie_models/sdk/captured.py:8-17,
117-191). The reference keeps prefill eager; here a step with prompt portions has a bucket per
(rows rounded up to 128, entries rounded up), captured when a shape comes a second time, since
a step of some hundred launches of a few microseconds each is otherwise bound by the host.
Everything beyond a batch's own counts is inert padding (rows of no entry, entries of no rows),
so what a graph computes for the real rows does not depend on its capacity.
"""

from __future__ import annotations

import numpy as np
import torch

from ..cache.arena import KVArena, derive_groups
from ..cache.manager import GroupSpec
from ..kernels import ops
from .batch import BatchLayout, BatchLimits, StepBatch


class StepContext:
    """What parts may read about the current step: the batch's arrays on the device (int32),
    and the same batch on the host for decisions that shape launches. `counts` are the sizes
    the kernels run at: the batch's own, or its capacities inside a CUDA graph."""

    def __init__(self, host: StepBatch, dev: torch.Tensor, counts: tuple[int, int, int] | None = None):
        self.host = host
        t, r, w = counts or (host.n_tokens, host.n_entries, host.n_logit_rows)
        self.n_tokens, self.n_entries, self.n_logit_rows = t, r, w
        self.captured = counts is not None
        # shape facts that choose kernels: inside a graph every row is an entry of its own and
        # contexts may reach the whole table; outside, the host batch says what is there
        if self.captured:
            self.decode_only = bool(r == t)
            self.max_context = host.max_context_bound
            self.n_attention_tiles = 0 if self.decode_only else t // 64 + r  # each entry may end in a partial tile
        else:
            self.decode_only = bool(r == t and r > 0)
            self.max_context = int(host.seq_lens[:r].max()) if r else 0
            rows = host.q_start[1: r + 1] - host.q_start[:r]
            self.n_attention_tiles = int(((rows + 63) // 64).sum())  # 64-row tiles, entry by entry

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
        self.temperature = view("temperature", w).view(torch.float32)
        self.top_k = view("top_k", w)
        self.key0 = view("key0", w)
        self.key1 = view("key1", w)
        self.sample_pos = view("sample_pos", w)
        at, _ = host.section("slot_mapping")
        self.slot_mapping = [dev[at + g * host.t_cap: at + g * host.t_cap + t] for g in range(len(host.block_tables))]
        at, _ = host.section("block_tables")
        self.block_tables = []
        for width in host.layout.table_widths:
            self.block_tables.append(dev[at: at + r * width].view(r, width))
            at += host.r_cap * width


def _bucket(n: int) -> int:
    """Powers of two up to 8, then multiples of 8."""
    b = 1
    while b < n and b < 8:
        b *= 2
    return b if n <= 8 else -(-n // 8) * 8


class StepGraph:
    """Forward pass + sampling of a batch of up to `t_cap` rows in up to `r_cap` entries (one
    logit row per entry), as one CUDA graph. t_cap == r_cap is the decode-only form. The graph
    begins with the copy of the pinned host batch to the device and ends with the copy of the
    sampled tokens into pinned host memory, so that a step is one graph launch and one wait."""

    def __init__(self, step_fn: "StepFunction", t_cap: int, r_cap: int):
        self.cap = r_cap
        self.device = step_fn.device
        self.host = StepBatch(BatchLayout(t_cap, r_cap, r_cap, step_fn.table_widths), pinned=True)
        self.host.max_context_bound = step_fn.model.max_seq_len
        self.host.pad()
        self.host.set_logit_rows([])
        self.host.set_sampling([], [], [], [], [])
        self.dev = torch.zeros(self.host.buf.shape[0], dtype=torch.int32, device=step_fn.device)
        self.dev.copy_(self.host._pinned_tensor)
        self.ctx = StepContext(self.host, self.dev, counts=(t_cap, r_cap, r_cap))
        self.tokens_host = torch.zeros(r_cap, dtype=torch.int32).pin_memory()
        self.tokens_host_np = self.tokens_host.numpy()
        # the device's error word travels to the host with the tokens: a kernel's time-out is seen at no extra cost
        self.error_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.error_host_np = self.error_host.numpy()
        self.error_word = ops.error_word(self.device)
        self.done = torch.cuda.Event()   # recorded after every replay: the batch is consumed, the tokens are on the host
        side = torch.cuda.Stream(device=step_fn.device)
        side.wait_stream(torch.cuda.current_stream(step_fn.device))
        with torch.cuda.stream(side):  # inert warm-up: every row is a pad row
            for _ in range(2):
                step_fn.sample(step_fn.forward(self.ctx), self.ctx)
        torch.cuda.current_stream(step_fn.device).wait_stream(side)
        torch.cuda.synchronize(step_fn.device)
        try:
            self._capture(step_fn)
        except RuntimeError as first:
            # a driver that cannot record programmatic launch edges in a graph: plain edges then
            if not ops.use_programmatic_dependent_launch(False):
                raise
            torch.cuda.synchronize(step_fn.device)
            try:
                self._capture(step_fn)
            except RuntimeError as second:
                # not the launch edges: a part that says `capturable` did what a capture forbids (a copy from
                # pageable host memory, a synchronisation, an allocation outside the graph's pool)
                raise RuntimeError(f"the step could not be captured in a CUDA graph: {first}") from second

    def _capture(self, step_fn: "StepFunction") -> None:
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(self.graph, pool=step_fn.graph_pool()):
            self.dev.copy_(self.host._pinned_tensor, non_blocking=True)
            self.logits = step_fn.forward(self.ctx)
            self.tokens = step_fn.sample(self.logits, self.ctx)
            self.tokens_host.copy_(self.tokens, non_blocking=True)
            self.error_host.copy_(self.error_word, non_blocking=True)
        self.kernels = ops.launch_count() - before

    def replay(self) -> None:
        self.graph.replay()
        self.done.record()
        self.host.copy_done = self.done
        ops.count_launches(self.kernels)

    def tokens_on_host(self, n: int) -> np.ndarray:
        """The last replay's first n tokens, once it has finished. Raises `ops.KernelTimeout` if a
        kernel of the step recorded that one of its bounded waits ran out."""
        self.done.synchronize()
        self.check()
        return self.tokens_host_np[:n]

    def check(self) -> None:
        if self.error_host_np[0]:
            code, self.error_host_np[0] = int(self.error_host_np[0]), 0
            ops.raise_on_device_error(self.device, code)


class StepFunction:
    def __init__(self, model, page_size: int, num_pages: int, max_requests: int, capture: bool = False,
                 capture_after: int = 1):
        """`capture`: steps run as CUDA graphs per shape bucket. A decode-only bucket is captured at
        first use; a bucket with prompt portions once its shape has come `capture_after` times
        before (0: at first use)."""
        self.model = model
        self.device = model.rt.device
        # the device's number, for the launch path that skips torch's device guard when it is the current one
        self._device_index = self.device.index if self.device.index is not None else (torch.cuda.current_device() if torch.cuda.is_available() else 0)
        self.groups, self.member_group = derive_groups(model.cache_members, page_size, num_pages)
        self.arena = KVArena(model.cache_members, self.groups, self.member_group, model.rt.dtype, self.device)
        self.state_tensors = [
            torch.zeros((max_requests,) + tuple(spec.shape), dtype=spec.dtype, device=self.device)
            for spec in model.state_members
        ]
        self.max_requests = max_requests
        self.table_widths = tuple(-(-model.max_seq_len // g.page_size) for g in self.groups)
        self._limits = BatchLimits(model.vocab_size, model.max_seq_len, self.groups, self.table_widths)
        # A mixer with state of its own folds an entry's rows on the host side of the launch, so
        # only models whose mixers all say `capturable` may run inside a CUDA graph.
        self.capture = capture and all(getattr(b.mixer, "capturable", False) for b in model.blocks)
        self._graphs: dict[tuple[int, int], StepGraph] = {}
        self.capture_after = capture_after
        self._seen: dict[tuple[int, int], int] = {}   # how often a shape with prompt portions has come
        self._pool = None
        self._batches: dict[tuple[int, int, int], StepBatch] = {}
        self.h2d_bytes = 0

    def graph_pool(self):
        """One memory pool for every graph of this step function: they never run at the same time,
        so their activations may share memory. A graph's outputs hold until the next step."""
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        return self._pool

    def cache_groups(self) -> list[GroupSpec]:
        return list(self.groups)

    # ---- batches ---------------------------------------------------------------------------
    def new_batch(self, n_tokens: int, n_entries: int, n_logit_rows: int, decode_only: bool = False) -> StepBatch:
        """A pinned host batch with room for the given counts. Batches are kept and handed
        out again; one is not reused before its last upload has finished."""
        t_cap = _bucket(n_tokens) if n_tokens <= 64 else -(-n_tokens // 128) * 128
        r_cap = _bucket(max(n_entries, 1))
        graph = None
        if self.capture and decode_only:
            graph = self._graph(r_cap, r_cap)
        elif self.capture and n_logit_rows <= n_entries and t_cap > r_cap:  # (t_cap == r_cap is the decode-only graph)
            if (t_cap, r_cap) in self._graphs or self._seen.get((t_cap, r_cap), 0) >= self.capture_after:
                graph = self._graph(t_cap, r_cap)
            else:
                self._seen[(t_cap, r_cap)] = self._seen.get((t_cap, r_cap), 0) + 1
        if graph is not None:
            batch = graph.host
        else:
            key = (t_cap, r_cap, _bucket(max(n_logit_rows, 1)) if n_logit_rows <= 64 else t_cap)
            batch = self._batches.get(key)
            if batch is None:
                batch = StepBatch(BatchLayout(key[0], key[1], max(key[2], n_logit_rows), self.table_widths), pinned=True)
                self._batches[key] = batch
        done = getattr(batch, "copy_done", None)
        if done is not None:
            done.synchronize()
        return batch

    def _graph(self, t_cap: int, r_cap: int) -> StepGraph:
        graph = self._graphs.get((t_cap, r_cap))
        if graph is None:
            with torch.cuda.device(self.device):
                graph = StepGraph(self, t_cap, r_cap)
            self._graphs[(t_cap, r_cap)] = graph
        return graph

    def _graph_of(self, batch: StepBatch) -> StepGraph | None:
        graph = self._graphs.get((batch.t_cap, batch.r_cap)) if self.capture else None
        return graph if graph is not None and batch is graph.host else None

    def upload(self, batch: StepBatch) -> StepContext:
        if not batch.trusted:
            batch.pad()
        dev = torch.empty(batch.buf.shape[0], dtype=torch.int32, device=self.device)
        dev.copy_(batch._pinned_tensor, non_blocking=True)
        batch.copy_done = torch.cuda.Event()
        batch.copy_done.record()
        self.h2d_bytes += batch.buf.nbytes
        return StepContext(batch, dev)

    def validate(self, batch: StepBatch) -> None:
        """Host-side bounds checks of a batch that the caller filled. A batch that the scheduler
        filled natively is inside the pool by construction and is not checked again."""
        if not batch.trusted:
            batch.check(self._limits)

    # ---- running ---------------------------------------------------------------------------
    def forward(self, ctx: StepContext) -> torch.Tensor:
        return self.model.forward(ctx, self.arena.members, self.state_tensors)

    def tokens_to_host(self, batch: StepBatch, tokens: torch.Tensor) -> np.ndarray:
        """The tokens that `step_and_sample(batch)` returned, on the host. A step that ran as a
        graph has them in pinned memory already; the view holds until that graph's next replay."""
        graph = self._graph_of(batch)
        if graph is not None and tokens.data_ptr() == graph.tokens.data_ptr():
            return graph.tokens_on_host(tokens.shape[0])
        out = tokens.cpu().numpy()
        ops.raise_on_device_error(self.device)
        return out

    def sample(self, logits: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.sample(logits, ctx.temperature, ctx.top_k, ctx.key0, ctx.key1, ctx.sample_pos)

    @torch.no_grad()
    def __call__(self, batch: StepBatch) -> torch.Tensor:
        """Logits [n_logit_rows, vocab] float32 on the device."""
        if batch.n_tokens == 0:
            return torch.empty(0, self.model.vocab_size, dtype=torch.float32, device=self.device)
        self.validate(batch)
        with torch.cuda.device(self.device):
            graph = self._graph_of(batch)
            if graph is not None:
                if not batch.trusted:
                    batch.pad()
                graph.replay()
                self.h2d_bytes += batch.buf.nbytes
                return graph.logits[: batch.n_logit_rows]
            return self.forward(self.upload(batch))

    def launch_graph(self, batch: StepBatch) -> StepGraph | None:
        """Launches the step as its CUDA graph, if the batch is one that the scheduler filled and
        has a graph: upload, forward pass, sampling and the copy of the tokens to pinned memory are
        all inside. Returns the graph (`tokens_on_host` waits for it), or None: run
        `step_and_sample` then."""
        if not batch.trusted:
            return None
        graph = self._graph_of(batch)
        if graph is None:
            return None
        if torch.cuda.current_device() != self._device_index:
            with torch.cuda.device(self.device):
                graph.replay()
        else:
            graph.replay()
        self.h2d_bytes += batch.buf.nbytes
        return graph

    @torch.no_grad()
    def step_and_sample(self, batch: StepBatch) -> torch.Tensor:
        """One token per logit row (int32, on the device); `batch.set_sampling` has been called."""
        self.validate(batch)
        with torch.cuda.device(self.device):
            graph = self._graph_of(batch)
            if graph is not None:
                if not batch.trusted:
                    batch.pad()
                graph.replay()
                self.h2d_bytes += batch.buf.nbytes
                return graph.tokens[: batch.n_logit_rows]
            ctx = self.upload(batch)
            return self.sample(self.forward(ctx), ctx)


def logit_rows_of_last(batch: StepBatch) -> np.ndarray:
    return batch.last_rows().astype(np.int32)
