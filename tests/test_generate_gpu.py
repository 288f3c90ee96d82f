"""Generation through the entry point against the plain implementation: greedy and sampled,
alone and batched, with prompts cut into portions, and with so few pages that requests are
preempted and recomputed. The workloads are those named for the two tiny configurations."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests.helpers import TINY_A, TINY_B, make_model_dir, random_tokens
from tests.plain import gpt2_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def wide_a(tmp_path_factory):
    """Tiny A with a wider initialisation: clear gaps between the largest logits, so that greedy
    tokens do not hang on the last bits."""
    return make_model_dir(tmp_path_factory.mktemp("wide_a"), TINY_A, std=0.2)


@pytest.fixture(scope="module")
def wide_b(tmp_path_factory):
    return make_model_dir(tmp_path_factory.mktemp("wide_b"), TINY_B, std=0.2)


def plain_generate(folder, prompts, n, temperature=0.0, top_k=0, seed=0, stop=()):
    w, cfg = plain.read_model(folder, torch.float32)
    eos = cfg.get("eos_token_id")
    stops = tuple(stop) + ((eos,) if eos is not None else ())
    return [plain.generate(w, cfg, p, n, temperature, top_k, key=(seed & 0xFFFFFFFF, i), stop_token_ids=stops)
            for i, p in enumerate(prompts)]


def test_greedy_tiny_a_workload(wide_a):
    """Four requests with prompts of 1, 5, 17 and 32 tokens, 16 greedy tokens each, pages of 16."""
    import research_2_b200 as r2

    prompts = [random_tokens(1 + i, n, 512) for i, n in enumerate((1, 5, 17, 32))]
    want = plain_generate(wide_a, prompts, 16)
    got = r2.generate(wide_a, prompts, 16, dtype="float32", block_size=16)
    assert got == want
    solo = [r2.generate(wide_a, [p], 16, dtype="float32", block_size=16)[0] for p in prompts]
    assert solo == want, "a request's tokens depend on who it was batched with"


def test_pages_of_twelve_tokens_through_the_engine(wide_a):
    """A page size that is no power of two (positions are split into page and offset by division) through
    the scheduler, the native batch fill and every kernel, in both precisions' paths, with few pages."""
    import research_2_b200 as r2

    prompts = [random_tokens(90 + i, n, 512) for i, n in enumerate((1, 13, 40, 25))]
    want = plain_generate(wide_a, prompts, 20)
    got = r2.generate(wide_a, prompts, 20, dtype="float32", block_size=12, num_slabs=14, max_requests=3, max_batch_tokens=36)
    assert got == want
    assert r2.generate(wide_a, prompts, 20, dtype="float32", block_size=24, max_requests=4, capture=True) == want


def test_sampled_tiny_b_workload(wide_b):
    """Six requests, prompts of 3 to 130 tokens, 24 tokens at temperature 0.8 with seed 4, the
    largest prompt prefilled in portions of 48, pages of 8."""
    import research_2_b200 as r2

    prompts = [random_tokens(3 + i, n, 1031) for i, n in enumerate((3, 9, 40, 64, 100, 130))]
    want = plain_generate(wide_b, prompts, 24, temperature=0.8, seed=4)
    got = r2.generate(wide_b, prompts, 24, temperature=0.8, seed=4, dtype="float32", block_size=8, chunk_size=48)
    assert got == want
    got_k = r2.generate(wide_b, prompts[:3], 12, temperature=1.2, top_k=5, seed=9, dtype="float32", block_size=8)
    assert got_k == plain_generate(wide_b, prompts[:3], 12, temperature=1.2, top_k=5, seed=9)


def test_bfloat16_generation_runs_with_and_without_graphs(wide_b):
    """bfloat16 tokens may differ from float32 ones after a near-tie, but CUDA graphs must not
    change them, and the first token comes from logits within the bfloat16 budget."""
    import research_2_b200 as r2

    prompts = [random_tokens(20 + i, n, 1031) for i, n in enumerate((12, 70, 33))]
    eager = r2.generate(wide_b, prompts, 20, dtype="bfloat16", block_size=8, capture=False)
    graphs = r2.generate(wide_b, prompts, 20, dtype="bfloat16", block_size=8, capture=True)
    assert eager == graphs
    assert all(len(t) == 20 for t in eager)


def test_prompt_portions_run_as_graphs_when_a_shape_repeats(wide_b):
    """With capture on, a step with prompt portions is captured the second time its shape comes
    and replayed from then on: rows and entries beyond the batch's own are padding, and the
    tokens are those of the plain implementation (float32, so the comparison is exact)."""
    import research_2_b200 as r2
    from research_2_b200.engine.api import generate_with

    prompts = [random_tokens(60 + i, n, 1031) for i, n in enumerate((100, 100, 100, 100, 37, 100, 150, 100))]
    want = plain_generate(wide_b, prompts, 10, temperature=0.7, seed=11)
    with r2.run(wide_b, dtype="float32", block_size=8, max_requests=3, max_batch_tokens=64, capture=True) as engine:
        got = generate_with(engine, prompts, 10, temperature=0.7, seed=11)
        shapes = [key for key in engine.step_fn._graphs if key[0] > key[1]]
        assert shapes, "no step with prompt portions was captured"
    assert got == want


def test_steps_that_are_only_launched_give_the_same_tokens(wide_b):
    """`step(wait=False)` returns when the step's graph has been launched; polls in between see
    the tokens of earlier steps, and the step is completed by the next call that needs it. Prompts
    of several lengths, so that admissions, portions, decoding and finishing all pass through."""
    import research_2_b200 as r2
    from research_2_b200.engine.api import generate_with

    prompts = [random_tokens(80 + i, n, 1031) for i, n in enumerate((40, 9, 100, 3, 64))]
    want = plain_generate(wide_b, prompts, 14)
    with r2.run(wide_b, dtype="float32", block_size=8, max_requests=3, max_batch_tokens=64, capture=True) as engine:
        launched = []
        launch_graph = engine.step_fn.launch_graph
        engine.step_fn.launch_graph = lambda batch: launched.append(launch_graph(batch)) or launched[-1]
        got = generate_with(engine, prompts, 14, wait=False)
        assert generate_with(engine, prompts, 14, wait=True) == got
        assert engine.finish() is None and not engine.has_work()
        assert sum(g is not None for g in launched) > 10, "no step ran as a launched-only graph"
    assert got == want


def test_few_pages_preempt_and_recompute(wide_a):
    """So few pages that running requests are preempted: the tokens stay the same."""
    import research_2_b200 as r2
    from research_2_b200.engine.api import generate_with

    prompts = [random_tokens(40 + i, n, 512) for i, n in enumerate((30, 28, 25, 20))]
    want = plain_generate(wide_a, prompts, 30)
    with r2.run(wide_a, dtype="float32", block_size=4, num_slabs=34, max_requests=4, max_batch_tokens=64) as engine:
        engine.keep_events = True
        got = generate_with(engine, prompts, 30)
        assert sum(e.n_preempted for e in engine.events) > 0, "the pool was meant to be too small"
        assert engine.scheduler.cache.n_free(0) == 34 and engine.scheduler.cache.check() == ""
    assert got == want


def test_engine_handle_submit_wait_poll_and_stop_tokens(wide_a):
    import research_2_b200 as r2

    prompt = random_tokens(77, 9, 512)
    want = plain_generate(wide_a, [prompt], 12)[0]
    with r2.run(wide_a, dtype="float32") as engine:
        rid = engine.submit(prompt, max_new_tokens=12)
        done = engine.wait(rid, timeout_s=120.0)
        assert done.finished and done.new_tokens == want and done.reason in ("finished_length", "finished_eos")
        rid = engine.submit(prompt, max_new_tokens=12, stop_token_ids=[want[3]])
        done = engine.wait(rid)
        first = want.index(want[3])
        assert done.new_tokens == want[: first + 1] and done.reason == "finished_eos"
        rid = engine.submit(prompt, max_new_tokens=0)
        assert engine.wait(rid).new_tokens == want[:1]
        plan = None
        rid = engine.submit(prompt, max_new_tokens=3)
        plan = engine.plan()  # the by-hand rung
        assert plan is not None and plan.n_entries == 1 and int(plan.rows[0]) == len(prompt)
        batch = engine.build_batch(plan)
        tokens = engine.step_fn.step_and_sample(batch).cpu().numpy()
        engine.commit(tokens)
        assert engine.poll(rid).new_tokens == want[:1]
        engine.cancel(rid)
        assert engine.plan() is None


def test_command_line(wide_a):
    prompt = random_tokens(5, 6, 512)
    want = plain_generate(wide_a, [prompt], 5)[0]
    proc = subprocess.run(
        [sys.executable, "-m", "research_2_b200", "generate", "--model", str(wide_a), "--dtype", "float32",
         "--prompt-tokens", ",".join(map(str, prompt)), "--max-new-tokens", "5", "--max-requests", "2", "--block-size", "16"],
        capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["prompt"] == prompt and line["tokens"] == want


def test_a_kernels_timeout_reaches_the_caller(wide_a):
    """A kernel whose bounded wait runs out records a code and returns; the step's results are void and
    the caller must hear of it. A kernel that does nothing but let such a wait run out (on a barrier
    on which nothing arrives; nothing is in flight when it gives up) stands in for the failure: the
    next step of an engine, as a CUDA graph and eagerly, and of trace replay raises KernelTimeout;
    the step after it runs as if nothing had happened."""
    import research_2_b200 as r2
    from research_2_b200.engine.replay import Replay
    from research_2_b200.kernels import ops

    prompt = random_tokens(3, 9, 512)
    want = plain_generate(wide_a, [prompt], 6)[0]
    for capture in (True, False):
        with r2.run(wide_a, dtype="float32", capture=capture) as engine:
            rid = engine.submit(prompt, max_new_tokens=6)
            engine.step()
            ops.wait_selftest("cuda:0", polls=8)
            with pytest.raises(ops.KernelTimeout, match="code 99") as err:
                engine.step()
            assert err.value.code == 99
            assert ops.device_errors() == 0, "the error word is cleared once it has been reported"
        assert r2.generate(wide_a, [prompt], 6, dtype="float32", capture=capture) == [want]
    replay = Replay(str(wide_a), "float32", 64)
    replay.step({"step": 0, "entries": [{"id": "a", "tokens": prompt[:4], "want": [3]}]})
    ops.wait_selftest("cuda:0", polls=2000)
    with pytest.raises(ops.KernelTimeout):
        replay.step({"step": 1, "entries": [{"id": "a", "tokens": prompt[4:], "want": [0]}]})


def test_two_models_in_one_process_step_alternately(wide_a, wide_b):
    """Nothing about a model lives in the process: two engines over different models, stepped in
    turn, give each the tokens that it gives alone."""
    import research_2_b200 as r2

    pa = [random_tokens(31 + i, n, 512) for i, n in enumerate((14, 40))]
    pb = [random_tokens(41 + i, n, 1031) for i, n in enumerate((9, 70))]
    want_a, want_b = plain_generate(wide_a, pa, 12), plain_generate(wide_b, pb, 12)
    for dtype in ("float32", "bfloat16"):
        with r2.run(wide_a, dtype=dtype, max_requests=2) as ea, r2.run(wide_b, dtype=dtype, block_size=8, max_requests=2) as eb:
            ra, rb = [ea.submit(p, 12) for p in pa], [eb.submit(p, 12) for p in pb]
            while ea.has_work() or eb.has_work():
                if ea.has_work():
                    ea.step()
                if eb.has_work():
                    eb.step()
            got_a, got_b = [ea.poll(r).new_tokens for r in ra], [eb.poll(r).new_tokens for r in rb]
        if dtype == "float32":
            assert got_a == want_a and got_b == want_b
        else:  # bfloat16 tokens may leave the float32 ones after a near-tie; alone and in turn they are the same
            assert got_a == r2.generate(wide_a, pa, 12, dtype=dtype, max_requests=2)
            assert got_b == r2.generate(wide_b, pb, 12, dtype=dtype, block_size=8, max_requests=2)


def test_logits_of_steps_that_run_as_graphs_through_the_engine(tiny_c_dir):
    """The path that serving and the benchmark run: the scheduler fills a padded batch natively, the
    step runs as the CUDA graph of its bucket, bfloat16, head size 64. The logits that each step's
    graph holds at its entries' last rows are compared with the plain implementation at the same
    (request, position), teacher-forced on the engine's own tokens."""
    import numpy as np
    import research_2_b200 as r2
    from tests.helpers import assert_within_budget

    vocab = 777
    prompts = [random_tokens(70 + i, n, vocab) for i, n in enumerate((300, 130, 17, 200, 64, 129))]
    for dtype in ("bfloat16", "float32"):
        rows: dict[int, dict[int, np.ndarray]] = {}
        with r2.run(tiny_c_dir, dtype=dtype, block_size=16, max_requests=3, num_slabs=48, max_batch_tokens=160,
                    chunk_size=96, capture=True) as engine:
            engine.step_fn.capture_after = 0   # every shape runs as its graph from its first step on
            rids = [engine.submit(p, 24) for p in prompts[:3]]
            waiting = list(prompts[3:])
            of = {rid: i for i, rid in enumerate(rids)}
            n_graph_steps = 0
            done: dict[int, list[int]] = {i: [] for i in range(len(prompts))}
            while engine.has_work() or waiting:
                plan = engine.plan()
                if plan is None:
                    break
                batch = engine.build_batch(plan)
                entries = list(zip(plan.req.tolist(), plan.start.tolist(), plan.rows.tolist()))
                graph = engine.step_fn.launch_graph(batch)
                assert graph is not None, "a step did not run as a graph"
                n_graph_steps += 1
                tokens = graph.tokens_on_host(plan.n_entries).copy()
                logits = graph.logits[: plan.n_entries].float().cpu().numpy()
                for (req, start, n), row in zip(entries, logits):
                    rows.setdefault(of[req], {})[start + n - 1] = row
                engine.commit(tokens)
                for rid in list(of):
                    p = engine.poll(rid)
                    done[of[rid]] += p.new_tokens
                    if p.finished:
                        of.pop(rid)
                        if waiting:
                            nxt = len(prompts) - len(waiting)
                            of[engine.submit(waiting.pop(0), 24)] = nxt
            assert n_graph_steps > 30 and any(t > r for t, r in engine.step_fn._graphs), "no graph with prompt portions ran"
            assert engine.scheduler.cache.check() == ""
        for i, prompt in enumerate(prompts):
            assert len(done[i]) == 24
            seq = prompt + done[i]
            positions = sorted(rows[i])
            assert positions[-1] == len(seq) - 2 and len(positions) >= 24
            got = np.stack([rows[i][p] for p in positions])
            assert_within_budget(got, tiny_c_dir, seq[:-1], dtype, positions=positions, what=f"engine graphs {dtype} request {i}")
