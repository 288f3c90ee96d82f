"""Replay on the GPU against the plain implementation: the same requests whole, with the last
32 tokens decoded one by one, in portions of changing size, and mixed with other requests in
a pool of the trace's own peak demand plus one page, so that pages are used again (asserted); in
float32 and in bfloat16, for the two tiny configurations and for a third of head size 64 with prompts of
several 128-row tiles (the tensor-core attention); eagerly and as CUDA graphs."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests import traces
from tests.helpers import TINY, assert_within_budget, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

LENGTHS = {"a": (70, 45, 128, 33, 2, 97), "b": (130, 64, 9, 100, 40, 3, 256), "c": (300, 130, 64, 200, 17, 2, 129, 512)}


def requests_for(name: str) -> dict[str, list[int]]:
    vocab = TINY[name]["config"]["vocab_size"]
    return {f"r{i}": random_tokens(100 + i, n, vocab) for i, n in enumerate(LENGTHS[name])}


def round64(n: int) -> int:
    return -(-n // 64) * 64


def cut(requests, mode: str) -> traces.TraceBuilder:
    if mode == "whole":
        return traces.whole(requests)
    if mode == "decode32":
        return traces.prefill_then_decode(requests, 32)
    if mode == "portions":
        return traces.portions(requests)
    return traces.mixed(requests, max_live=4)


def run_trace(folder, tb, dtype, page_size, max_tokens=None, garbage=64.0, capture=False, expect_reuse=False):
    """Replays the trace; returns {step: logits}. With `max_tokens` None the pool is the trace's own
    peak demand plus one page, so that later requests can only run in pages that earlier ones gave
    back. `expect_reuse` asserts that this happened: at least a third of the pool's pages were held by
    two different requests one after the other, and pages that were handed out a second time still
    held what their previous owner wrote (so a kernel that read beyond its own tokens would see it)."""
    from research_2_b200.engine.replay import Replay

    live, round_to = traces.max_live(tb), 64
    if max_tokens is None:
        max_tokens, round_to = (traces.peak_pages(tb, page_size) + 1) * page_size, page_size
    replay = Replay(str(folder), dtype, max_tokens, block_size=page_size, max_live=max(live, 1), round_to=round_to, capture=capture)
    arena = replay.step_fn.arena
    arena.fill_(garbage)  # a slot that was never written reads loudly
    owners: dict[int, list[str]] = {}
    stale = 0
    out = {}
    for record in tb.steps:
        before = arena.tensors[0].clone() if expect_reuse else None
        logits = replay.step(record)
        if logits is not None:
            out[record["step"]] = logits
        for rid, per_group in replay.pages_of_last_step.items():
            for page in per_group[0]:
                seen = owners.setdefault(page, [])
                if not seen or seen[-1] != rid:
                    if seen and expect_reuse and bool((before[page] != garbage).any()):
                        stale += 1  # handed out with the previous owner's keys and values still in it
                    seen.append(rid)
    assert replay.cache.check() == ""
    for g in range(len(replay.cache.groups)):
        assert replay.cache.n_free(g) == replay.cache.groups[g].num_pages, "pages were lost"
    if expect_reuse:
        n_pages = replay.cache.groups[0].num_pages
        reused = sum(len(seen) >= 2 for seen in owners.values())
        assert 3 * reused >= n_pages, f"only {reused} of {n_pages} pages were used again"
        assert stale > 0, "no page was handed out with stale data in it"
        assert owners == {p: o for p, o in traces.page_traffic(tb, page_size, n_pages).items()}, "pages went other ways than the cache manager alone gives them"
    return out


def compare(folder, requests, tb, outputs, dtype, what, partial=False):
    """Every output row against the plain implementation at its (request, position). Unless
    `partial`, every position of every request must have been written exactly once."""
    assert sorted(outputs) == sorted(tb.rows), (sorted(outputs), sorted(tb.rows))
    per_request: dict[str, dict[int, np.ndarray]] = {}
    for step, rows in tb.rows.items():
        got = outputs[step]
        assert got.shape[0] == len(rows)
        for (rid, pos), logits in zip(rows, got):
            assert pos not in per_request.setdefault(rid, {}), f"{what}: position {pos} of {rid} written twice"
            per_request[rid][pos] = logits
    for rid, ids in requests.items():
        positions = sorted(per_request.get(rid, {}))
        if partial:
            assert positions, f"{what}: request {rid} has no wanted position"
        else:
            assert positions == list(range(len(ids))), f"{what}: request {rid} misses positions"
        got = np.stack([per_request[rid][p] for p in positions])
        assert_within_budget(got, folder, ids, dtype, positions=positions if partial else None, what=f"{what} request {rid}")
    return per_request


@pytest.fixture(scope="module")
def folders(tiny_a_dir, tiny_b_dir, tiny_c_dir):
    return {"a": tiny_a_dir, "b": tiny_b_dir, "c": tiny_c_dir}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("mode", ["whole", "decode32", "portions", "mixed"])
def test_replay_modes(folders, name, dtype, mode):
    folder, requests = folders[name], requests_for(name)
    page = TINY[name]["page_size"]
    tb = cut(requests, mode)
    outputs = run_trace(folder, tb, dtype, page, expect_reuse=mode == "mixed")
    compare(folder, requests, tb, outputs, dtype, f"{name}/{dtype}/{mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "decode32", "portions", "mixed"])
def test_replay_through_cuda_graphs(folders, dtype, mode):
    """The same cuttings with every step run as the CUDA graph of its shape bucket, as generation
    runs them: rows padded up to the bucket, empty entries, contexts bounded by the model's limit,
    other slice counts and kernel choices than the eager step of the exact shape. One logit row per
    entry (its last token), which is what a step's graph computes. Head size 64, bfloat16: the
    tensor-core attention and the cache write in the q/k/v product's epilogue."""
    folder, requests = folders["c"], requests_for("c")
    tb = traces.with_last_only(cut(requests, mode))
    outputs = run_trace(folder, tb, dtype, TINY["c"]["page_size"], capture=True, expect_reuse=mode == "mixed")
    compare(folder, requests, tb, outputs, dtype, f"c/{dtype}/{mode}/graphs", partial=True)


def test_float32_logits_do_not_depend_on_the_cutting_at_all(folders):
    """In float32 every output element is one thread's sum in a fixed order: whole, decoded one by
    one, in portions, mixed with others in recycled pages, the logits at a position are the same
    bits."""
    for name in ("b", "c"):
        folder, requests = folders[name], requests_for(name)
        page = TINY[name]["page_size"]
        results = {}
        for mode in ("whole", "decode32", "portions", "mixed"):
            tb = cut(requests, mode)
            results[mode] = compare(folder, requests, tb, run_trace(folder, tb, "float32", page), "float32", f"{name}/{mode}")
        for mode in ("decode32", "portions", "mixed"):
            for rid, rows in results["whole"].items():
                for pos, logits in rows.items():
                    assert np.array_equal(logits, results[mode][rid][pos]), f"{name}: {mode} differs from whole at {rid}[{pos}]"


def test_first_tokens(folders):
    """The first tokens of a sequence: one token, then one more, then two."""
    folder = folders["a"]
    ids = random_tokens(7, 4, TINY["a"]["config"]["vocab_size"])
    tb = traces.TraceBuilder()
    tb.step([("x", ids[:1], [0])])
    tb.step([("x", ids[1:2], [0])])
    tb.step([("x", ids[2:4], [0, 1])], end=["x"])
    for dtype in ("float32", "bfloat16"):
        compare(folder, {"x": ids}, tb, run_trace(folder, tb, dtype, 16, max_tokens=64), dtype, f"first tokens {dtype}")


def test_long_decoding(folders):
    """A short prompt and then every further token one by one up to the model's limit."""
    folder = folders["b"]
    ids = random_tokens(11, 256, TINY["b"]["config"]["vocab_size"])
    tb = traces.prefill_then_decode({"x": ids}, n_decode=250)
    for dtype in ("float32", "bfloat16"):
        compare(folder, {"x": ids}, tb, run_trace(folder, tb, dtype, 8, max_tokens=256), dtype, f"long decoding {dtype}")


def test_trace_run_program(folders, tmp_path):
    """The program itself: JSON lines in, `done <step>` lines and .f32 files out."""
    folder, name = folders["a"], "a"
    requests = {k: v for k, v in list(requests_for(name).items())[:3]}
    tb = traces.mixed(requests, max_live=3)
    out = tmp_path / "out"
    text = "".join(json.dumps(s) + "\n" for s in tb.steps)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(sum(round64(len(v)) for v in requests.values()))],
        input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(len(tb.steps))]
    vocab = TINY[name]["config"]["vocab_size"]
    outputs = {int(p.stem): np.fromfile(p, dtype="<f4").reshape(-1, vocab) for p in out.glob("*.f32")}
    compare(folder, requests, tb, outputs, "float32", "trace_run program")
