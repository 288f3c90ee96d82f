"""The engine above a step function that has no GPU: `step(wait=False)` launches, the next call
that needs the step completes it, and what requests produce does not depend on which of the
two ways the caller steps. The fake step function "samples" a token that is a fixed function of
the entry's last input token and its position, so every request's continuation is known."""

from __future__ import annotations

import numpy as np
import pytest

from research_2_b200.cache import GroupSpec
from research_2_b200.engine.api import generate_with
from research_2_b200.engine.batch import batch_for
from research_2_b200.engine.engine import Engine
from research_2_b200.engine.scheduler import Scheduler, SchedulerConfig

VOCAB = 211


def next_token(last: int, position: int) -> int:
    return (last * 31 + position * 7 + 3) % VOCAB


class FakeGraph:
    """What `launch_graph` hands back: the tokens of a launched step, read when it is completed."""

    io_inside = True

    def __init__(self):
        self.tokens = np.zeros(0, dtype=np.int32)
        self.reads = 0

    def tokens_on_host(self, n: int) -> np.ndarray:
        self.reads += 1
        return self.tokens[:n]


class FakeStepFunction:
    def __init__(self, groups, max_seq_len: int):
        self.groups = groups
        self.table_widths = tuple(-(-max_seq_len // g.page_size) for g in groups)
        self.graph = FakeGraph()
        self.launched = 0
        self.h2d_bytes = 0

    def cache_groups(self):
        return list(self.groups)

    def new_batch(self, n_tokens, n_entries, n_logit_rows, decode_only=False):
        return batch_for(self.table_widths, n_tokens, n_entries, n_logit_rows)

    def launch_graph(self, batch):
        assert batch.trusted, "the engine fills batches natively"
        out = []
        for e in range(batch.n_entries):
            last_row = int(batch.q_start[e + 1]) - 1
            out.append(next_token(int(batch.input_ids[last_row]), int(batch.positions[last_row])))
        self.graph.tokens = np.asarray(out, dtype=np.int32)
        self.launched += 1
        return self.graph


def make_engine(max_requests=3, pages=64, page_size=4, max_seq_len=96, budget=16) -> Engine:
    groups = [GroupSpec(page_size, 0, pages)]
    step_fn = FakeStepFunction(groups, max_seq_len)
    scheduler = Scheduler(
        SchedulerConfig(max_requests=max_requests, max_seq_len=max_seq_len, max_batch_tokens=budget, max_batch_reqs=max_requests,
                        vocab_size=VOCAB, eos_token=None, order="running_first", reserve_ratio=0.0),
        step_fn.cache_groups())
    return Engine(step_fn, scheduler)


def continuation(prompt: list[int], n: int, stop=()) -> list[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        token = next_token(ids[-1], len(ids) - 1)
        ids.append(token)
        out.append(token)
        if token in stop:
            break
    return out


PROMPTS = [[5, 9, 200, 17, 3, 3, 8], [1], [7] * 30, [100, 101], [9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 11, 12, 13]]


@pytest.mark.parametrize("wait", [True, False])
def test_continuations_do_not_depend_on_how_the_caller_steps(wait):
    with make_engine() as engine:
        got = generate_with(engine, PROMPTS, 12, wait=wait)
        assert engine.finish() is None and not engine.has_work()
        assert engine.scheduler.cache.check() == ""
    assert got == [continuation(p, 12) for p in PROMPTS]


def test_a_launched_step_is_completed_by_the_next_call_that_needs_it():
    with make_engine() as engine:
        rid = engine.submit(PROMPTS[0], max_new_tokens=4)
        assert engine.step(wait=False) is None and engine.has_work()
        assert engine.poll(rid).new_tokens == [], "a poll does not complete a launched step"
        event = engine.finish()
        assert event is not None and engine.finish() is None
        want = continuation(PROMPTS[0], 4)
        assert engine.poll(rid).new_tokens == want[:1]
        # the next step completes what was launched before it plans
        engine.step(wait=False)
        engine.step(wait=False)
        assert engine.poll(rid).new_tokens == want[1:2]
        # so does wait(), which returns everything not polled before
        done = engine.wait(rid)
        assert done.finished and done.new_tokens == want[2:]
        assert engine.step_fn.graph.reads == engine.step_fn.launched


def test_cancel_and_stop_tokens_with_a_step_in_flight():
    with make_engine() as engine:
        want = continuation(PROMPTS[4], 20)
        a = engine.submit(PROMPTS[4], max_new_tokens=20, stop_token_ids=[want[5]])
        b = engine.submit(PROMPTS[2], max_new_tokens=50)
        for _ in range(4):
            engine.step(wait=False)
        engine.cancel(b)  # completes the launched step first: the plan that names b is committed, then b goes
        with pytest.raises(KeyError):
            engine.poll(b)
        done = engine.wait(a)
        assert done.finished and done.reason == "finished_eos"
        assert done.new_tokens == want[: want.index(want[5]) + 1]
        assert not engine.has_work()
        free = engine.scheduler.cache.n_free(0)
        assert free == 64, f"pages were kept: {free} of 64 free"
