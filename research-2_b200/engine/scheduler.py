"""The scheduler seen from Python: a handle on the native one (csrc/host/scheduler.h).

Exceptions carry the reference's names (kelpie-engine/kelpie_engine/sdk/engine.py:58-93):
Full, TooLong, ExceedsKvPool, Stalled, CommitError.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import numpy as np

from ..cache import _host
from ..cache.manager import CacheManager, GroupSpec, group_array

STATE_NAMES = {0: "free", 1: "waiting", 2: "running", 3: "finished_eos", 4: "finished_length", 5: "cancelled"}
ENTRY_PREFILL, ENTRY_DECODE = 0, 1
ORDERS = {"running_first": 0, "waiting_first": 1}
MAX_STOP_TOKENS = 8


class Full(RuntimeError):
    """Every request slot is taken."""


class TooLong(ValueError):
    """prompt + max_new_tokens exceeds max_seq_len."""


class ExceedsKvPool(ValueError):
    """The request could never fit the cache pool, even alone."""


class Stalled(RuntimeError):
    """A plan scheduled nothing, preempted nobody, and work is pending."""

    def __init__(self, req_id: int, n_work: int, need_pages: int, free_pages: int, group: int = 0):
        super().__init__(
            f"stalled: request {req_id} needs {need_pages} pages of cache group {group} for its next {n_work} tokens, "
            f"{free_pages} are free and nothing else can make progress"
        )
        self.req_id, self.n_work, self.need_pages, self.free_pages, self.group = req_id, n_work, need_pages, free_pages, group


class CommitError(RuntimeError):
    """The tokens handed to commit do not fit the plan; nothing was applied."""


@dataclass(frozen=True)
class SchedulerConfig:
    max_requests: int
    max_seq_len: int
    max_batch_tokens: int
    max_batch_reqs: int
    vocab_size: int
    eos_token: int | None = None
    order: str = "running_first"
    reserve_ratio: float = 0.0
    chunk_size: int = 0  # 0 = the token budget alone cuts prompts; else the most rows of a portion inside a history


class Plan:
    """One step's entries, decode entries first (kelpie-core/src/scheduler.zig:1315-1328): the
    counts, and per entry `req`, `start`, `rows`, `emits`, `kind`, `temperature`, `top_k`,
    `sample_pos`, `key0`, `key1`, per row `input_ids`. The arrays are copied out of the
    scheduler when one of them is first asked for (a step that fills its batch natively never
    asks) and are views of the scheduler's buffers: they hold until its next plan()."""

    ARRAYS = ("req", "start", "rows", "emits", "kind", "input_ids", "temperature", "top_k", "sample_pos", "key0", "key1")

    def __init__(self, scheduler: "Scheduler", n_entries: int, n_tokens: int):
        self._scheduler = scheduler
        self.n_entries = n_entries
        self.n_tokens = n_tokens

    def __getattr__(self, name: str):  # reached only for what is not set yet: the arrays
        if name in Plan.ARRAYS:
            if self._scheduler._plan is not self:
                raise RuntimeError("this plan's arrays were not read before the scheduler's next plan()")
            for field, value in zip(Plan.ARRAYS, self._scheduler._plan_buffers.take(self._scheduler._plan_c)):
                object.__setattr__(self, field, value)
            return self.__dict__[name]
        raise AttributeError(name)

    @property
    def decode_only(self) -> bool:
        """Every entry has one row (an entry has at least one)."""
        return self.n_entries > 0 and self.n_tokens == self.n_entries

    def token_lists(self) -> list[np.ndarray]:
        out, at = [], 0
        for n in self.rows:
            out.append(self.input_ids[at: at + n])
            at += int(n)
        return out


@dataclass(frozen=True)
class Poll:
    new_tokens: list[int]
    finished: bool
    reason: str  # the request's state: running, waiting, finished_eos, finished_length


@dataclass(frozen=True)
class RequestEvent:
    """One request's life in numbers (kelpie-core/src/events.zig:39-55); times are nanoseconds of a
    monotonic clock and 0 while the moment has not come."""

    t_arrival_ns: int
    t_first_sched_ns: int
    t_first_token_ns: int
    t_last_token_ns: int
    t_finish_ns: int
    first_step: int
    last_step: int
    request_id: int
    n_prompt: int
    n_generated: int
    max_new: int
    n_preempted: int
    n_chunks: int
    state: str
    peak_pages: int

    @property
    def time_to_first_token_ms(self) -> float | None:
        return (self.t_first_token_ns - self.t_arrival_ns) / 1e6 if self.t_first_token_ns else None


@dataclass(frozen=True)
class StepEvent:
    step: int
    n_entries: int
    n_tokens: int
    n_prefill_rows: int
    n_decode: int
    n_admitted: int
    n_preempted: int
    n_finished: int
    n_running: int
    n_waiting: int
    kv_free: int
    t_plan_ns: int
    t_commit_ns: int


class _PlanBuffers:
    """Arrays that receive a plan from the native side: sized once for the largest plan, filled by
    memmove, handed out as views (a Plan is valid until the next plan() of its scheduler)."""

    FIELDS = (("req", np.int32, False), ("start", np.int32, False), ("rows", np.int32, False), ("emits", np.int32, False),
              ("kind", np.int32, False), ("input_ids", np.int32, True), ("temperature", np.float32, False),
              ("top_k", np.int32, False), ("sample_pos", np.int32, False), ("key0", np.uint32, False),
              ("key1", np.uint32, False))  # in Plan.ARRAYS' order

    def __init__(self, max_entries: int, max_tokens: int):
        self.arrays = [np.zeros(max(max_tokens if per_token else max_entries, 1), dtype=dt) for _, dt, per_token in self.FIELDS]
        self.addresses = [a.ctypes.data for a in self.arrays]

    def take(self, p) -> list:
        out = []
        for (name, _, per_token), arr, addr in zip(self.FIELDS, self.arrays, self.addresses):
            n = p.n_tokens if per_token else p.n_entries
            if n:
                C.memmove(addr, getattr(p, name), n * 4)
            out.append(arr[:n])
        return out


class Scheduler:
    def __init__(self, config: SchedulerConfig, groups: list[GroupSpec]):
        self._lib = _host.lib()
        self.config = config
        self.groups = list(groups)
        if config.order not in ORDERS:
            raise ValueError(f"order must be one of {sorted(ORDERS)}, got {config.order!r}")
        c = _host.SchedulerConfigC(
            config.max_requests, config.max_seq_len, config.max_batch_tokens, config.max_batch_reqs,
            ORDERS[config.order], config.reserve_ratio,
            -1 if config.eos_token is None else config.eos_token, config.vocab_size, config.chunk_size,
        )
        handle = self._lib.r2_sched_create(C.byref(c), group_array(self.groups), len(self.groups))
        if not handle:
            raise ValueError(f"scheduler: {_host.last_error()}")
        self._h = C.c_void_p(handle)
        self.cache = CacheManager(self.groups, config.max_requests, config.max_seq_len, _borrowed=self)
        self._plan_buffers = _PlanBuffers(config.max_batch_reqs, config.max_batch_tokens)
        self._plan_c = _host.PlanC()
        self._plan: Plan | None = None
        self._poll_buf = np.zeros(config.max_seq_len, dtype=np.int32)
        self._poll_ptr = self._poll_buf.ctypes.data_as(_host.I32P)
        self._poll_flags = (C.c_int32(0), C.c_int32(0))

    def _cache_handle(self) -> int:
        return self._lib.r2_sched_cache(self._h)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.r2_sched_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    # ---- requests --------------------------------------------------------------------------
    def submit(  # noqa: PLR0913
        self, prompt, max_new_tokens: int, temperature: float = 0.0, top_k: int = 0, seed: int = 0,
        stop_token_ids=(),
    ) -> int:
        """Queue a request; it is admitted at a later plan. Checks in the reference's order
        (kelpie-core/src/c_api.zig:774-807; kelpie_engine/sdk/engine.py:298-305)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32).reshape(-1)
        stops = np.ascontiguousarray(list(stop_token_ids), dtype=np.int32)
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if not math.isfinite(temperature) or temperature < 0:
            raise ValueError(f"temperature must be finite and >= 0, got {temperature}")
        if not 0 <= top_k <= self.config.vocab_size:
            raise ValueError(f"top_k must be in [0, {self.config.vocab_size}], got {top_k}")
        if len(stops) > MAX_STOP_TOKENS:
            raise ValueError(f"at most {MAX_STOP_TOKENS} stop tokens, got {len(stops)}")
        if max_new_tokens < 0:
            raise ValueError(f"max_new_tokens must be >= 0, got {max_new_tokens}")
        rid = self._lib.r2_sched_submit(
            self._h, prompt.ctypes.data_as(_host.I32P), len(prompt), max_new_tokens, temperature, top_k,
            seed & 0xFFFFFFFFFFFFFFFF, stops.ctypes.data_as(_host.I32P), len(stops),
        )
        if rid >= 0:
            return rid
        if rid == -1:
            raise Full(f"all {self.config.max_requests} request slots are taken")
        if rid == -2:
            raise TooLong(
                f"prompt ({len(prompt)}) + max_new_tokens ({max(1, max_new_tokens)}) exceeds max_seq_len "
                f"({self.config.max_seq_len})"
            )
        if rid == -5:
            raise ExceedsKvPool(
                f"a request of {len(prompt)} + {max(1, max_new_tokens)} tokens needs more pages than the pool has"
            )
        if rid == -3:
            raise ValueError("bad request: a prompt token lies outside the vocabulary")
        raise ValueError(f"submit refused with status {rid}")

    def cancel(self, rid: int) -> None:
        if self._lib.r2_sched_cancel(self._h, rid) != 0:
            raise KeyError(f"no request {rid}")

    def poll(self, rid: int) -> Poll:
        finished, state = self._poll_flags
        n = self._lib.r2_sched_poll(self._h, rid, self._poll_ptr, self.config.max_seq_len, C.byref(finished), C.byref(state))
        if n < 0:
            raise KeyError(f"no request {rid}")
        return Poll(self._poll_buf[:n].tolist(), bool(finished.value), STATE_NAMES[state.value])

    def request_info(self, rid: int) -> dict:
        vals = [C.c_int32(0) for _ in range(5)]
        if self._lib.r2_sched_request_info(self._h, rid, *[C.byref(v) for v in vals]) != 0:
            raise KeyError(f"no request {rid}")
        state, n_prompt, n_tokens, n_computed, n_preempted = (v.value for v in vals)
        return {"state": STATE_NAMES[state], "n_prompt": n_prompt, "n_tokens": n_tokens,
                "n_computed": n_computed, "n_preempted": n_preempted}

    def request_event(self, rid: int) -> RequestEvent:
        """The request's record so far; complete once it has finished. It goes away with the
        request's slot, that is with the poll that reports `finished`: read it before that poll."""
        e = _host.RequestEventC()
        if self._lib.r2_sched_request_event(self._h, rid, C.byref(e)) != 0:
            raise KeyError(f"no request {rid}")
        values = {name: getattr(e, name) for name, _ in _host.RequestEventC._fields_}
        values["state"] = STATE_NAMES[values["state"]]
        return RequestEvent(**values)

    def finished_request_events(self) -> list[RequestEvent]:
        """Records of the requests whose slots were released since the last call (finished and polled
        to the end, or cancelled), oldest first."""
        buf = (_host.RequestEventC * 64)()
        out = []
        while True:
            n = self._lib.r2_sched_drain_request_events(self._h, buf, 64)
            for e in buf[:n]:
                values = {name: getattr(e, name) for name, _ in _host.RequestEventC._fields_}
                values["state"] = STATE_NAMES[values["state"]]
                out.append(RequestEvent(**values))
            if n < 64:
                return out

    @property
    def grain(self) -> int:
        """Portions that do not finish a history end on multiples of this (every group's page size divides it)."""
        return self._lib.r2_sched_grain(self._h)

    # ---- steps -----------------------------------------------------------------------------
    def plan(self) -> Plan:
        """The next step's entries (possibly none). Raises Stalled when nothing can run."""
        p = self._plan_c
        status = self._lib.r2_sched_plan(self._h, C.byref(p))
        if status != 0:
            raise RuntimeError("plan() while the previous plan has not been committed")
        plan = self._plan = Plan(self, p.n_entries, p.n_tokens)
        if p.n_entries == 0:
            stall = _host.StallC()
            if self._lib.r2_sched_stall(self._h, C.byref(stall)):
                self._lib.r2_sched_commit(self._h, None, 0)  # the empty plan is closed so that the caller can go on
                raise Stalled(stall.req_id, stall.n_work, stall.need_pages, stall.free_pages, stall.group)
        return plan

    def fill(self, batch) -> None:
        """The outstanding plan as a whole step batch, written natively into `batch`: tokens,
        positions, slots, block tables, one logit row per entry (its last) with its sampling
        parameters, padding. What it writes lies inside the pool by construction, so the step
        function does not check such a batch again."""
        status = self._lib.r2_sched_fill_step_batch(self._h, batch.native())
        if status < 0:
            raise RuntimeError(f"the plan does not fit the batch, or a row's page is not reserved (status {status})")
        p = self._plan_c
        batch.n_entries, batch.n_tokens, batch.n_logit_rows = p.n_entries, p.n_tokens, p.n_entries
        batch.trusted = True

    def commit(self, tokens) -> None:
        if not (isinstance(tokens, np.ndarray) and tokens.dtype == np.int32 and tokens.ndim == 1 and tokens.flags.c_contiguous):
            tokens = np.ascontiguousarray(tokens, dtype=np.int32).reshape(-1)
        status = self._lib.r2_sched_commit(self._h, tokens.ctypes.data_as(_host.I32P), len(tokens))
        if status == -9:
            raise CommitError("commit without a plan")
        if status != 0:
            raise CommitError("the tokens do not fit the plan (wrong count or a token outside the vocabulary)")

    def event(self) -> StepEvent:
        e = _host.StepEventC()
        self._lib.r2_sched_event(self._h, C.byref(e))
        return StepEvent(*(getattr(e, name) for name, _ in _host.StepEventC._fields_))

    def counts(self) -> tuple[int, int]:
        a, b = C.c_int32(0), C.c_int32(0)
        self._lib.r2_sched_counts(self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def has_work(self) -> bool:
        running, waiting = self.counts()
        return running + waiting > 0

    def set(self, **knobs) -> None:  # noqa: A003
        """Live knobs, applied at the next plan (kelpie-core/src/scheduler.zig:36-52)."""
        ids = {"max_batch_tokens": 0, "max_batch_reqs": 1, "order": 2, "reserve_ratio": 3, "chunk_size": 4}
        for name, value in knobs.items():
            if name not in ids:
                raise KeyError(f"unknown knob {name!r}; known: {sorted(ids)}")
            v = ORDERS[value] if name == "order" else value
            if self._lib.r2_sched_set(self._h, ids[name], float(v)) != 0:
                raise ValueError(f"{name}={value!r} is out of range")
