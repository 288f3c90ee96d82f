"""The scheduler's decisions (no GPU): text traces, and a random caller against an exact oracle.

The oracle is the reference's idea of a model with no weights (kelpie/scripts/check_core_loop.py:
1-58): the fake "cache" stores the TOKEN written at each slot; every row must read back exactly
its request's history through its block table; pages of ended requests are poisoned. A wrong
plan, slot or table shows up as a wrong token, with no GPU involved.
"""

from __future__ import annotations

import random
import re
from pathlib import Path

import numpy as np
import pytest

from research_2_b200.cache import GroupSpec
from research_2_b200.engine.batch import batch_for
from research_2_b200.engine.scheduler import (
    CommitError, ExceedsKvPool, Full, Scheduler, SchedulerConfig, Stalled, TooLong,
)

TRACES = sorted((Path(__file__).parent / "sched_traces").glob("*.txt"))
ERRORS = {"TooLong": TooLong, "Full": Full, "ExceedsKvPool": ExceedsKvPool, "ValueError": ValueError}


def _kv(text: str) -> dict[str, str]:
    return dict(item.split("=", 1) for item in text.split())


class TraceRunner:
    def __init__(self):
        self.sched: Scheduler | None = None
        self.ids: dict[str, int] = {}
        self.plan = None
        self.stall = None
        self.polled: dict[str, list[int]] = {}
        self.final: dict[str, str] = {}

    def name_of(self, rid: int) -> str:
        return next(k for k, v in self.ids.items() if v == rid)

    def run(self, path: Path) -> None:
        for n, raw in enumerate(path.read_text().splitlines(), 1):
            line = raw.split("#", 1)[0].strip()
            if not line:
                continue
            try:
                self.line(line)
            except AssertionError as err:
                raise AssertionError(f"{path.name}:{n}: `{line}`: {err}") from None

    def line(self, line: str) -> None:
        word, _, rest = line.partition(" ")
        getattr(self, f"do_{word}")(rest.strip())

    def do_config(self, rest: str) -> None:
        kv = _kv(rest)
        # groups=all | window8 | all+window8 (one cache group each); num_blocks=6 or 6,2 (per group)
        windows = [int(g[len("window"):]) if g.startswith("window") else 0 for g in kv.get("groups", "all").split("+")]
        blocks = [int(b) for b in kv["num_blocks"].split(",")]
        blocks = blocks * len(windows) if len(blocks) == 1 else blocks
        eos = int(kv.get("eos", -1))
        cfg = SchedulerConfig(
            max_requests=int(kv.get("max_requests", 8)), max_seq_len=int(kv.get("max_seq_len", 64)),
            max_batch_tokens=int(kv["max_batch_tokens"]), max_batch_reqs=int(kv["max_batch_reqs"]),
            vocab_size=10000, eos_token=None if eos < 0 else eos, order=kv.get("order", "running_first"),
            reserve_ratio=float(kv.get("reserve_ratio", 0)), chunk_size=int(kv.get("chunk_size", 0)))
        self.sched = Scheduler(cfg, [GroupSpec(int(kv["block_size"]), w, n) for w, n in zip(windows, blocks)])
        self.ids, self.polled, self.final = {}, {}, {}

    def _submit(self, rest: str) -> int:
        name, _, opts = rest.partition(" ")
        kv = _kv(opts)
        base = (ord(name) - 64) * 100
        prompt = [base + i for i in range(int(kv["prompt"]))]
        stops = [int(s) for s in kv["stop"].split(",")] if "stop" in kv else []
        rid = self.sched.submit(prompt, int(kv["max_new"]), float(kv.get("temperature", 0.0)),
                                int(kv.get("top_k", 0)), 0, stops)
        self.ids[name] = rid
        self.polled[name] = []
        return rid

    def do_submit(self, rest: str) -> None:
        self._submit(rest)

    def do_cancel(self, rest: str) -> None:
        self.sched.cancel(self.ids.pop(rest))

    def do_set(self, rest: str) -> None:
        for k, v in _kv(rest).items():
            self.sched.set(**{k: v if k == "order" else (float(v) if k == "reserve_ratio" else int(v))})

    def do_step(self, rest: str) -> None:
        given = {}
        if rest.startswith("tokens="):
            given = {k: int(v) for k, v in (item.split(":") for item in rest[len("tokens="):].split(","))}
        self.stall = None
        try:
            self.plan = self.sched.plan()
        except Stalled as err:
            self.stall, self.plan, self.last_batch, self.last_kinds = err, None, [], []
            return
        names = [self.name_of(int(r)) for r in self.plan.req]
        kinds = {0: "prefill", 1: "decode"}
        self.last_batch = [f"{n}:{int(rows)}" for n, rows in zip(names, self.plan.rows)]
        self.last_kinds = [f"{n}:{kinds[int(k)]}" for n, k in zip(names, self.plan.kind)]
        self.sched.commit([given.get(n, 1) for n in names])
        self._drain()

    def _drain(self) -> None:
        for name, rid in list(self.ids.items()):
            p = self.sched.poll(rid)
            self.polled[name] += p.new_tokens
            if p.finished:
                self.final[name] = p.reason
                del self.ids[name]
            elif p.reason.startswith("finished"):
                self.final[name] = p.reason

    def do_expect(self, rest: str) -> None:
        what, _, arg = rest.partition(" ")
        arg = arg.strip()
        if what == "batch":
            got = self.last_batch
            assert got == arg.split(), f"batch is {' '.join(got) or '(empty)'}"
        elif what == "kinds":
            got = self.last_kinds
            assert got == arg.split(), f"kinds are {' '.join(got)}"
        elif what in ("free", "free1"):
            g = 1 if what == "free1" else 0
            assert self.sched.cache.n_free(g) == int(arg), f"{what} is {self.sched.cache.n_free(g)}"
        elif what == "request":
            name, _, opts = arg.partition(" ")
            event = self.sched.request_event(self.ids[name])
            for k, v in _kv(opts).items():
                assert str(getattr(event, k)) == v, f"request {name}: {k} is {getattr(event, k)}"
        elif what in ("running", "waiting"):
            got = sorted(n for n, rid in self.ids.items() if self.sched.request_info(rid)["state"] == what)
            assert got == sorted(arg.split()), f"{what} is {got}"
        elif what == "polled":
            name, _, toks = arg.partition(" ")
            want = [int(t) for t in re.findall(r"-?\d+", toks)]
            assert self.polled[name] == want, f"polled {self.polled[name]}"
            self.polled[name] = []
        elif what == "finished":
            name, _, reason = arg.partition(" ")
            assert self.final.get(name) == reason.split("=", 1)[1], f"state is {self.final.get(name)}"
        elif what == "stall":
            if arg == "none":
                assert self.stall is None, f"stalled: {self.stall}"
            else:
                name, _, opts = arg.partition(" ")
                kv = _kv(opts)
                s = self.stall
                assert s is not None, "no stall was reported"
                got = (self.name_of(s.req_id), s.n_work, s.need_pages, s.free_pages, s.group)
                assert got == (name, int(kv["n_work"]), int(kv["need"]), int(kv["free"]), int(kv.get("group", 0))), f"stall is {got}"
        elif what == "event":
            event = self.sched.event()
            for k, v in _kv(arg).items():
                assert getattr(event, k) == int(v), f"event.{k} is {getattr(event, k)}"
        elif what == "refused":
            body, _, err = arg.rpartition(" error=")
            with pytest.raises(ERRORS[err]):
                self._submit(body[len("submit "):])
        else:
            raise AssertionError(f"unknown expectation {what!r}")
        assert self.sched.cache.check() == ""


@pytest.mark.parametrize("path", TRACES, ids=[p.stem for p in TRACES])
def test_trace(path):
    TraceRunner().run(path)


def test_commit_is_checked_and_applies_nothing_on_error():
    s = Scheduler(SchedulerConfig(4, 32, 16, 4, 100), [GroupSpec(4, 0, 8)])
    rid = s.submit([1, 2, 3], 4)
    with pytest.raises(CommitError):
        s.commit([1])  # no plan
    plan = s.plan()
    assert plan.n_entries == 1
    with pytest.raises(CommitError):
        s.commit([1, 2])  # wrong count
    with pytest.raises(CommitError):
        s.commit([100])  # outside the vocabulary
    assert s.request_info(rid)["n_computed"] == 0 and s.request_info(rid)["n_tokens"] == 3
    s.commit([5])
    assert s.poll(rid).new_tokens == [5]
    with pytest.raises(RuntimeError):
        s.plan(); s.plan()  # a second plan before the commit


def test_exceeds_pool_is_refused_at_submit():
    s = Scheduler(SchedulerConfig(4, 64, 16, 4, 100), [GroupSpec(4, 0, 3)])
    with pytest.raises(ExceedsKvPool):
        s.submit(list(range(10)), 8)  # 17 positions need 5 pages, the pool has 3
    s.submit(list(range(10)), 3)  # 12 positions fit exactly


def test_temperature_zero_rule_and_seed_keys():
    s = Scheduler(SchedulerConfig(4, 32, 16, 4, 100), [GroupSpec(4, 0, 8)])
    s.submit([1, 2], 2, temperature=0.0, top_k=7, seed=5)
    s.submit([1, 2], 2, temperature=0.7, top_k=7, seed=(9 << 32) | 3)
    plan = s.plan()
    assert list(plan.temperature) == [1.0, pytest.approx(0.7)] and list(plan.top_k) == [1, 7]
    assert list(plan.key0) == [5, 3] and list(plan.key1) == [0, 9]
    assert list(plan.sample_pos) == [2, 2]


class TokenCacheModel:
    """A model without weights: its cache keeps the token written at each slot, and its
    "logits" are a checksum of what a row can read through its block table."""

    POISON = -7

    def __init__(self, groups, page_size):
        self.page_size = page_size
        self.store = np.full((groups[0].num_pages + 1) * page_size, self.POISON, dtype=np.int64)

    def step(self, batch, histories) -> list[int]:
        t = batch.n_tokens
        self.store[batch.slot_mapping[0, :t]] = batch.input_ids[:t]
        out = []
        for e in range(batch.n_entries):
            a, b = int(batch.q_start[e]), int(batch.q_start[e + 1])
            n = int(batch.seq_lens[e])
            table = batch.block_tables[0][e]
            slots = table[np.arange(n) // self.page_size] * self.page_size + np.arange(n) % self.page_size
            seen = self.store[slots]
            want = np.asarray(histories[int(batch.entry_req[e])][:n])
            assert np.array_equal(seen, want), f"entry {e}: the cache holds {seen.tolist()}, the history is {want.tolist()}"
            assert list(batch.positions[a:b]) == list(range(n - (b - a), n))
            out.append(int(seen.sum() * 31 + n) % 97)
        return out

    def poison(self, pages) -> None:
        for p in pages:
            self.store[p * self.page_size: (p + 1) * self.page_size] = self.POISON


@pytest.mark.parametrize("seed", range(5))
def test_random_caller_against_the_token_oracle(seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    groups = [GroupSpec(page, 0, rng.randint(10, 24))]
    cfg = SchedulerConfig(max_requests=5, max_seq_len=48, max_batch_tokens=rng.choice([8, 16, 24]),
                          max_batch_reqs=rng.choice([2, 4, 5]), vocab_size=97, eos_token=None)
    sched = Scheduler(cfg, groups)
    model = TokenCacheModel(groups, page)
    histories: dict[int, list[int]] = {}
    solo: dict[tuple, list[int]] = {}
    results: dict[int, list[int]] = {}
    prompts: dict[int, tuple] = {}
    submitted = finished = preempted = 0
    for it in range(400):
        if rng.random() < 0.3:
            prompt = [rng.randrange(97) for _ in range(rng.randint(1, 20))]
            max_new = rng.randint(1, 12)
            try:
                rid = sched.submit(prompt, max_new)
                histories[rid], results[rid], prompts[rid] = list(prompt), [], (tuple(prompt), max_new)
                submitted += 1
            except (Full, TooLong, ExceedsKvPool):
                pass
        if rng.random() < 0.03 and histories:
            rid = rng.choice(list(histories))
            sched.cancel(rid)
            del histories[rid], results[rid], prompts[rid]
        held_before = {r: set(int(p) for p in sched.cache.table(r) if p) for r in histories if sched.cache.is_open(r)}
        try:
            plan = sched.plan()
        except Stalled:
            raise AssertionError("a random caller within the limits must never stall") from None
        if plan.n_entries == 0:
            sched.commit([])
        else:
            # pages that left a table since the last step are poisoned before anyone reads
            for r, pages in held_before.items():
                now = set(int(p) for p in sched.cache.table(r) if p) if sched.cache.is_open(r) else set()
                model.poison(pages - now)
            batch = batch_for(sched.cache.table_widths, plan.n_tokens, plan.n_entries, plan.n_entries)
            batch.set_entries(plan.req, plan.start, plan.token_lists())
            sched.cache.fill(batch)
            batch.pad()
            # the native fill of a whole step batch writes what these calls write, padding included
            batch.set_logit_rows(batch.last_rows())
            batch.set_sampling(plan.temperature, plan.top_k, plan.key0, plan.key1, plan.sample_pos)
            roomy = batch_for(sched.cache.table_widths, plan.n_tokens + 5, plan.n_entries + 3, plan.n_entries + 3)
            roomy.buf[:] = 77  # stale values everywhere
            sched.fill(roomy)
            assert roomy.trusted and (roomy.n_tokens, roomy.n_entries, roomy.n_logit_rows) == (plan.n_tokens, plan.n_entries, plan.n_entries)
            by_hand = batch_for(sched.cache.table_widths, plan.n_tokens + 5, plan.n_entries + 3, plan.n_entries + 3)
            by_hand.set_entries(plan.req, plan.start, plan.token_lists())
            sched.cache.fill(by_hand)
            by_hand.set_logit_rows(by_hand.last_rows())
            by_hand.set_sampling(plan.temperature, plan.top_k, plan.key0, plan.key1, plan.sample_pos)
            by_hand.pad()
            for name, (at, size) in roomy._sections.items():
                if not name.startswith("_"):
                    assert np.array_equal(roomy.buf[at: at + size], by_hand.buf[at: at + size]), f"native fill: {name} differs"
            assert np.array_equal(roomy.entry_rows[: plan.n_entries], plan.rows)
            assert plan.n_tokens <= cfg.max_batch_tokens and plan.n_entries <= cfg.max_batch_reqs
            assert len(set(plan.req.tolist())) == plan.n_entries, "a request is in the batch twice"
            kinds = plan.kind.tolist()
            assert kinds == sorted(kinds, reverse=True), "decode entries come first"
            tokens = model.step(batch, histories)
            sched.commit(tokens)
            for r, emits, tok in zip(plan.req.tolist(), plan.emits.tolist(), tokens):
                if emits:
                    histories[r].append(tok)
        preempted += sched.event().n_preempted
        assert sched.cache.check() == ""
        for rid in list(histories):
            p = sched.poll(rid)
            results[rid] += p.new_tokens
            if p.finished:
                prompt, max_new = prompts[rid]
                assert results[rid] == histories[rid][len(prompt):]
                assert len(results[rid]) == max_new and p.reason == "finished_length"
                # the same request alone gives the same tokens: nothing depends on the batch
                key = (prompt, max_new)
                if key not in solo:
                    hist = list(prompt)
                    for _ in range(max_new):
                        hist.append(int(sum(hist) * 31 + len(hist)) % 97)
                    solo[key] = hist[len(prompt):]
                assert results[rid] == solo[key]
                finished += 1
                del histories[rid], results[rid], prompts[rid]
    assert finished > 10
    while sched.has_work():  # drain: everything ends and every page comes back
        plan = sched.plan()
        batch = batch_for(sched.cache.table_widths, max(plan.n_tokens, 1), max(plan.n_entries, 1), 1)
        if plan.n_entries:
            batch.set_entries(plan.req, plan.start, plan.token_lists())
            sched.cache.fill(batch)
        tokens = model.step(batch, histories) if plan.n_entries else []
        sched.commit(tokens)
        for r, emits, tok in zip(plan.req.tolist(), plan.emits.tolist(), tokens):
            if emits:
                histories[r].append(tok)
        for rid in list(histories):
            if sched.poll(rid).finished:
                del histories[rid]
    assert sched.cache.n_free(0) == groups[0].num_pages


def test_budget_below_a_page_is_refused_at_creation():
    with pytest.raises(ValueError, match="at least 8"):
        Scheduler(SchedulerConfig(4, 64, 4, 4, 100), [GroupSpec(8, 0, 8)])
    with pytest.raises(ValueError, match="at least 8"):
        Scheduler(SchedulerConfig(4, 64, 16, 4, 100, chunk_size=4), [GroupSpec(8, 0, 8)])
    with pytest.raises(ValueError, match="at least 24"):  # two groups: a portion ends on a page boundary of both
        Scheduler(SchedulerConfig(4, 64, 16, 4, 100), [GroupSpec(8, 0, 8), GroupSpec(12, 4, 8)])
    assert Scheduler(SchedulerConfig(4, 64, 24, 4, 100), [GroupSpec(8, 0, 8), GroupSpec(12, 4, 8)]).grain == 24


def test_request_events_outlive_their_slots():
    """Arrival, first token and finish of every request, read after its slot was given back."""
    s = Scheduler(SchedulerConfig(2, 32, 16, 2, 100), [GroupSpec(4, 0, 8)])
    a = s.submit([1, 2, 3, 4, 5], 2)
    b = s.submit([7], 3)
    s.cancel(b)
    while s.has_work():
        plan = s.plan()
        s.commit([9] * plan.n_entries)
        during = s.request_event(a) if s.request_info(a)["state"] != "free" else None
        s.poll(a)
    assert during is not None and during.n_generated == 2 and during.state == "finished_length"
    events = s.finished_request_events()
    assert [e.request_id for e in events] == [b, a] and s.finished_request_events() == []
    cancelled, done = events
    assert cancelled.state == "cancelled" and cancelled.t_first_token_ns == 0 and cancelled.time_to_first_token_ms is None
    assert done.n_prompt == 5 and done.n_generated == 2 and done.n_chunks == 2 and done.peak_pages == 2
    assert done.t_arrival_ns <= done.t_first_sched_ns <= done.t_first_token_ns <= done.t_last_token_ns <= done.t_finish_ns
    assert done.first_step == 1 and done.last_step == 2 and done.time_to_first_token_ms >= 0
