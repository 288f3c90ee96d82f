"""Replay on the GPU against the plain implementation: the same requests whole, with the last
32 tokens decoded one by one, in portions of changing size, and mixed with other requests in
so few pages that pages are used again; in float32 and in bfloat16, for the two tiny configurations
and for a third of head size 64 with prompts of several 128-row tiles (the tensor-core attention)."""

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


def run_trace(folder, tb, dtype, max_tokens, page_size, garbage=64.0):
    from research_2_b200.engine.replay import Replay

    replay = Replay(str(folder), dtype, max_tokens, block_size=page_size)
    replay.step_fn.arena.fill_(garbage)  # a slot that was never written reads loudly
    out = {}
    for record in tb.steps:
        logits = replay.step(record)
        if logits is not None:
            out[record["step"]] = logits
    assert replay.cache.check() == ""
    for g in range(len(replay.cache.groups)):
        assert replay.cache.n_free(g) == replay.cache.groups[g].num_pages, "pages were lost"
    return out


def compare(folder, requests, tb, outputs, dtype, what):
    assert sorted(outputs) == sorted(tb.rows), (sorted(outputs), sorted(tb.rows))
    per_request: dict[str, dict[int, np.ndarray]] = {}
    for step, rows in tb.rows.items():
        got = outputs[step]
        assert got.shape[0] == len(rows)
        for (rid, pos), logits in zip(rows, got):
            assert pos not in per_request.setdefault(rid, {}), f"{what}: position {pos} of {rid} written twice"
            per_request[rid][pos] = logits
    for rid, ids in requests.items():
        positions = sorted(per_request[rid])
        assert positions == list(range(len(ids))), f"{what}: request {rid} misses positions"
        got = np.stack([per_request[rid][p] for p in positions])
        assert_within_budget(got, folder, ids, dtype, what=f"{what} request {rid}")


@pytest.fixture(scope="module")
def folders(tiny_a_dir, tiny_b_dir, tiny_c_dir):
    return {"a": tiny_a_dir, "b": tiny_b_dir, "c": tiny_c_dir}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("mode", ["whole", "decode32", "portions", "mixed"])
def test_replay_modes(folders, name, dtype, mode):
    folder, requests = folders[name], requests_for(name)
    page = TINY[name]["page_size"]
    if mode == "whole":
        tb, live = traces.whole(requests), 1
    elif mode == "decode32":
        tb, live = traces.prefill_then_decode(requests, 32), 1
    elif mode == "portions":
        tb, live = traces.portions(requests), 1
    else:
        tb, live = traces.mixed(requests, max_live=4), 4
    biggest = sorted((round64(len(v)) for v in requests.values()), reverse=True)[:live]
    outputs = run_trace(folder, tb, dtype, sum(biggest), page)
    compare(folder, requests, tb, outputs, dtype, f"{name}/{dtype}/{mode}")


def test_first_tokens(folders):
    """The first tokens of a sequence: one token, then one more, then two."""
    folder = folders["a"]
    ids = random_tokens(7, 4, TINY["a"]["config"]["vocab_size"])
    tb = traces.TraceBuilder()
    tb.step([("x", ids[:1], [0])])
    tb.step([("x", ids[1:2], [0])])
    tb.step([("x", ids[2:4], [0, 1])], end=["x"])
    for dtype in ("float32", "bfloat16"):
        compare(folder, {"x": ids}, tb, run_trace(folder, tb, dtype, 64, 16), dtype, f"first tokens {dtype}")


def test_long_decoding(folders):
    """A short prompt and then every further token one by one up to the model's limit."""
    folder = folders["b"]
    ids = random_tokens(11, 256, TINY["b"]["config"]["vocab_size"])
    tb = traces.prefill_then_decode({"x": ids}, n_decode=250)
    for dtype in ("float32", "bfloat16"):
        compare(folder, {"x": ids}, tb, run_trace(folder, tb, dtype, 256, 8), dtype, f"long decoding {dtype}")


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
