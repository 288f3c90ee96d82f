"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same
model, step function, cache manager and kernels that generation uses. Steps arrive as JSON
lines `{"step": n, "entries": [{"id": "a", "tokens": [...], "want": [...]}], "end": [...]}`;
all entries of a step are one batch. For a step in which something is wanted the logits at
the wanted places go to `<out>/<step>.f32` as little-endian float32 [wanted, vocab], in the
order of the entries and of `want`. After every step `done <step>` is printed and flushed.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..models.loading import load_model
from .step import StepFunction


class Replay:
    """`max_tokens` is the most tokens that live requests hold at any time, each request's count
    rounded up to a multiple of `round_to`; the pool gets the pages for that many (a request whose
    rounded count is no multiple of the page size may need one page more, so with such a page
    size the pool gets one extra page per live request). `capture` runs the steps as CUDA graphs
    where the step function has one for the shape, as generation does."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, block_size: int = 16, device: str = "cuda:0",
                 max_live: int = 4, round_to: int = 64, capture: bool = False):
        if max_tokens < 1:
            raise ValueError(f"--max-tokens must be >= 1, got {max_tokens}")
        if block_size < 1 or max_live < 1 or round_to < 1:
            raise ValueError("block size, live requests and rounding must be >= 1")
        self.model = load_model(model_dir, dtype=dtype, device=device)
        num_pages = -(-max_tokens // block_size) + (max_live if round_to % block_size else 0)
        self.step_fn = StepFunction(self.model, block_size, num_pages, max_live, capture=capture, capture_after=0)
        self.cache = CacheManager(self.step_fn.cache_groups(), max_live, self.model.max_seq_len)
        self.slots: dict[str, int] = {}
        self.fed: dict[str, int] = {}
        self.max_live = max_live
        self.pages_of_last_step: dict[str, list[list[int]]] = {}  # request -> per cache group, the pages it held in the last step

    def _slot(self, rid: str) -> int:
        if rid in self.slots:
            return self.slots[rid]
        free = [s for s in range(self.max_live) if s not in self.slots.values()]
        if not free:
            raise RuntimeError(f"request {rid!r}: more than {self.max_live} requests are live")
        self.cache.open(free[0])
        self.slots[rid], self.fed[rid] = free[0], 0
        return free[0]

    def step(self, record: dict) -> np.ndarray | None:
        """Run one step; returns the wanted logits [n, vocab] (None when nothing is wanted)."""
        entries = record.get("entries", [])
        reqs, starts, token_lists, wants = [], [], [], []
        self.pages_of_last_step = {}
        for entry in entries:
            rid, tokens = str(entry["id"]), [int(t) for t in entry["tokens"]]
            if not tokens:
                raise ValueError(f"request {rid!r}: an entry needs at least one token")
            slot = self._slot(rid)
            start = self.fed[rid]
            self.cache.slide(slot, start)
            self.cache.reserve(slot, start, start + len(tokens))
            self.pages_of_last_step[rid] = [[int(p) for p in self.cache.table(slot, g) if p] for g in range(len(self.cache.groups))]
            want = [int(w) for w in entry.get("want", [])]
            if any(not 0 <= w < len(tokens) for w in want):
                raise ValueError(f"request {rid!r}: want {want} lies outside its {len(tokens)} tokens")
            reqs.append(slot)
            starts.append(start)
            token_lists.append(tokens)
            wants.append(want)
        result = None
        if reqs:
            n_want = sum(len(w) for w in wants)
            batch = self.step_fn.new_batch(sum(len(t) for t in token_lists), len(reqs), n_want,
                                           decode_only=all(len(t) == 1 for t in token_lists))
            batch.set_entries(reqs, starts, token_lists)
            self.cache.fill(batch)
            rows = [int(batch.q_start[e]) + w for e, want in enumerate(wants) for w in want]
            batch.set_logit_rows(rows)
            logits = self.step_fn(batch)
            for entry, tokens in zip(entries, token_lists):
                self.fed[str(entry["id"])] += len(tokens)
            if n_want:
                result = logits.to(torch.float32).cpu().numpy()
            else:
                torch.cuda.synchronize(self.step_fn.device)
            ops.raise_on_device_error(self.step_fn.device)  # a kernel that gave up a bounded wait: the step is void
        for rid in record.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                self.cache.close(self.slots.pop(rid))
                del self.fed[rid]
        return result


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="a folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="the most tokens that live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--max-live", type=int, default=4, help="the most requests that are live at a time")
    ap.add_argument("--round-to", type=int, default=64, help="each request's token count is rounded up to a multiple of this")
    ap.add_argument("--capture", action="store_true", help="run steps as CUDA graphs where generation would")
    args = ap.parse_args(argv)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    replay = Replay(args.model, args.dtype, args.max_tokens, args.block_size, args.device, max_live=args.max_live,
                    round_to=args.round_to, capture=args.capture)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = replay.step(record)
        if logits is not None:
            logits.astype("<f4").tofile(out / f"{record['step']}.f32")
        print(f"done {record['step']}", flush=True)
    return 0
