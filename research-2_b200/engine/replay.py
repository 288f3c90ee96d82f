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
from ..models.loading import load_model
from .step import StepFunction

MAX_LIVE = 4
ROUND_TO = 64


class Replay:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, block_size: int = 16, device: str = "cuda:0",
                 max_live: int = MAX_LIVE):
        if max_tokens < 1:
            raise ValueError(f"--max-tokens must be >= 1, got {max_tokens}")
        if ROUND_TO % block_size != 0:
            raise ValueError(f"the page size must divide {ROUND_TO}, got {block_size}")
        self.model = load_model(model_dir, dtype=dtype, device=device)
        num_pages = -(-max_tokens // block_size)
        self.step_fn = StepFunction(self.model, block_size, num_pages, max_live)
        self.cache = CacheManager(self.step_fn.cache_groups(), max_live, self.model.max_seq_len)
        self.slots: dict[str, int] = {}
        self.fed: dict[str, int] = {}
        self.max_live = max_live

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
        for entry in entries:
            rid, tokens = str(entry["id"]), [int(t) for t in entry["tokens"]]
            if not tokens:
                raise ValueError(f"request {rid!r}: an entry needs at least one token")
            slot = self._slot(rid)
            start = self.fed[rid]
            self.cache.slide(slot, start)
            self.cache.reserve(slot, start, start + len(tokens))
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
            batch = self.step_fn.new_batch(sum(len(t) for t in token_lists), len(reqs), n_want)
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
    args = ap.parse_args(argv)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    replay = Replay(args.model, args.dtype, args.max_tokens, args.block_size, args.device)
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
