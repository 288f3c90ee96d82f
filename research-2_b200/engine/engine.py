"""The engine: a scheduler above a step function, with the reference's handle methods.

`submit / poll / wait / cancel / plan / commit` carry the names and meanings of the reference's
Engine (kelpie-engine/kelpie_engine/sdk/engine.py:240-753). The reference runs its step loop
on a thread of its own; here `step()` is a plain call and `wait()` steps until the request is
finished, so nothing happens behind the caller's back. `step(wait=False)` returns as soon as the
step's graph has been launched: what the caller does next (polling the tokens of earlier steps,
submitting) runs while the GPU works, and the step is completed by the next call that needs it.
"""

from __future__ import annotations

import time

import numpy as np

from ..config.engine_options import EngineOptions
from .scheduler import Plan, Poll, RequestEvent, Scheduler, SchedulerConfig, StepEvent  # noqa: F401


class Engine:
    def __init__(self, step_fn, scheduler: Scheduler, seed: int = 0):
        self.step_fn, self.scheduler = step_fn, scheduler
        self.seed = seed
        self._ordinal = 0
        self._pending: dict[int, list[int]] = {}
        self._plan: Plan | None = None
        self.events: list[StepEvent] = []
        self.keep_events = False
        self._launched = None   # (graph, number of entries) of a step that runs and is not committed yet

    @classmethod
    def for_model(cls, model, options: EngineOptions | None = None) -> "Engine":
        from .step import StepFunction

        opts = (options or EngineOptions()).validated(model.max_seq_len)
        step_fn = StepFunction(model, opts.block_size, opts.num_slabs, opts.max_requests, capture=bool(opts.capture))
        scheduler = Scheduler(
            SchedulerConfig(
                max_requests=opts.max_requests, max_seq_len=opts.max_seq_len, max_batch_tokens=opts.max_batch_tokens,
                max_batch_reqs=opts.max_batch_reqs, vocab_size=model.vocab_size, eos_token=model.eos_token,
                order=opts.order, reserve_ratio=opts.reserve_ratio, chunk_size=opts.chunk_size),
            step_fn.cache_groups())
        engine = cls(step_fn, scheduler, seed=opts.seed)
        engine.options = opts
        engine.model = model
        return engine

    # ---- requests --------------------------------------------------------------------------
    def submit(  # noqa: PLR0913
        self, prompt, max_new_tokens: int, temperature: float = 0.0, stop_token_ids=(), top_k: int = 0,
        seed: int | None = None,
    ) -> int:
        """Queue a request; it is admitted at the next step. `seed` keys this request's random
        draws (default: the engine's seed and the request's ordinal)."""
        if seed is None:
            seed = (self.seed & 0xFFFFFFFF) | ((self._ordinal & 0xFFFFFFFF) << 32)
        rid = self.scheduler.submit(prompt, max_new_tokens, temperature, top_k, seed, stop_token_ids)
        self._ordinal += 1
        self._pending[rid] = []
        return rid

    def cancel(self, rid: int) -> None:
        self.finish()
        self.scheduler.cancel(rid)
        self._pending.pop(rid, None)

    def poll(self, rid: int) -> Poll:
        return self.scheduler.poll(rid)

    def wait(self, rid: int, timeout_s: float | None = None) -> Poll:
        """Step until the request has finished; returns all tokens not polled before."""
        deadline = None if timeout_s is None else time.monotonic() + timeout_s
        tokens: list[int] = []
        while True:
            p = self.scheduler.poll(rid)
            tokens += p.new_tokens
            if p.finished:
                self._pending.pop(rid, None)
                return Poll(tokens, True, p.reason)
            if deadline is not None and time.monotonic() > deadline:
                return Poll(tokens, False, p.reason)
            self.step()

    # ---- steps -----------------------------------------------------------------------------
    def plan(self) -> Plan | None:
        """The next step's entries, or None when there is nothing to run (the by-hand rung:
        kelpie_engine/sdk/engine.py:585-601). Follow with `commit`."""
        self.finish(want_event=self.keep_events)   # (the record is only built where someone will read it)
        plan = self.scheduler.plan()
        if plan.n_entries == 0:
            self.scheduler.commit([])
            return None
        self._plan = plan
        return plan

    def commit(self, tokens) -> None:
        self.scheduler.commit(tokens)
        self._plan = None

    def build_batch(self, plan: Plan):
        batch = self.step_fn.new_batch(plan.n_tokens, plan.n_entries, plan.n_entries, decode_only=plan.decode_only)
        if plan is self.scheduler._plan:
            self.scheduler.fill(batch)  # one native call: entries, cache indices, logit rows, sampling, padding
            return batch
        batch.set_entries(plan.req, plan.start, plan.token_lists())
        self.scheduler.cache.fill(batch)
        batch.set_logit_rows(batch.last_rows())
        batch.set_sampling(plan.temperature, plan.top_k, plan.key0, plan.key1, plan.sample_pos)
        return batch

    def step(self, wait: bool = True) -> StepEvent | None:
        """One plan, one forward pass, one sampling call, one commit. With `wait=False` a step
        that runs as a CUDA graph is only launched: `finish()`, or the next `step`, `plan`, `wait`,
        `cancel` or `close`, waits for its tokens and commits them (`poll` before that returns
        what earlier steps produced); the return value is then None."""
        plan = self.plan()
        if plan is None:
            return None
        batch = self.build_batch(plan)
        graph = self.step_fn.launch_graph(batch)
        if graph is not None:
            self._launched = (graph, plan.n_entries)
            return self.finish() if wait else None
        tokens = self.step_fn.step_and_sample(batch)
        self.commit(self.step_fn.tokens_to_host(batch, tokens) if hasattr(tokens, "data_ptr") else np.asarray(tokens, dtype=np.int32))
        event = self.scheduler.event()
        if self.keep_events:
            self.events.append(event)
        return event

    def finish(self, want_event: bool = True) -> StepEvent | None:
        """Completes a step that `step(wait=False)` launched: waits for its tokens, commits them. Returns the
        step's record (None if nothing was launched, or with `want_event=False`)."""
        if self._launched is None:
            return None
        graph, n = self._launched
        self._launched = None
        self.commit(graph.tokens_on_host(n))
        if not want_event:
            return None
        event = self.scheduler.event()
        if self.keep_events:
            self.events.append(event)
        return event

    def request_events(self):
        """Per-request records (arrival, first token, finish, portions, preemptions, peak pages) of the
        requests that ended since the last call (kelpie-core/src/events.zig:39-55)."""
        return self.scheduler.finished_request_events()

    def has_work(self) -> bool:
        return self._launched is not None or self.scheduler.has_work()

    def set(self, **knobs) -> None:  # noqa: A003
        self.scheduler.set(**knobs)

    def close(self) -> None:
        self.finish()
        self.scheduler.close()

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
