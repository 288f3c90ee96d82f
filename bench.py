#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200: GPT-2 124M sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step. The default run decodes a batch of 8 requests whose prompts have
512 tokens (context grows from 512 towards 1024), prints ONE JSON line, and exits 0.

  value      decoded tokens per second, timed on the device with CUDA events around K graph
             replays; sampled tokens feed the next step on the device, nothing is skipped
  e2e        the same through the Python entry point (`Engine.submit / step / poll`): host
             tokens in and out, one pinned host-to-device copy and one device-to-host read a step
  prefill    one step of 2,048 prompt tokens (2 x 1,024); frac = flops / time / bf16 peak
  roofline   bytes a decode step must read (every weight once + the live requests' cache)
             / its time, against the measured copy bandwidth
  points     decode at batch 1 and 64, and at the headline's batch through the true 32-bit path
  mixed      64 requests with prompts of 16 to 768 tokens, 256 new tokens each, portions of 512 tokens a
             step beside the others' decoded tokens, through the Python entry point; with the median
             and 90th-percentile time to a request's first token
  kernels    the step's dominant kernels one by one: microseconds and fraction of the measured peak

`--model gpt2-355M` and `--model gpt2-1.5B` run the same at those sizes (the 1.5B decode workload has
1,000-token prompts and 24 new tokens, which bounds its steps).

Between timed steps nothing is flushed: each step reads weights and cache larger than L2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GPT2_124M = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 12, "n_embd": 768, "n_head": 12,
    "n_inner": 3072, "vocab_size": 50257, "n_positions": 1024, "activation_function": "gelu_new",
    "layer_norm_epsilon": 1e-5, "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True, "eos_token_id": None,
}
# The other sizes of the family that the baseline names (355M, 1.5B): the default run is 124M.
SIZES = {
    "gpt2-124M": GPT2_124M,
    "gpt2-355M": dict(GPT2_124M, n_layer=24, n_embd=1024, n_head=16, n_inner=4096),
    "gpt2-1.5B": dict(GPT2_124M, n_layer=48, n_embd=1600, n_head=25, n_inner=6400),
}
SEED, PAGE, PROMPT_LEN, CONTEXT = 5, 16, 512, 1024
# The prompts of each size's decode workload (the 1.5B workload fills the context with 1,000-token prompts
# and 24 new tokens); `main` sets PROMPT_LEN from it.
PROMPT_LENS = {"gpt2-124M": 512, "gpt2-355M": 512, "gpt2-1.5B": 1000}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"])}, "measured"
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_model(n_layer: int, dtype: str = "bfloat16", size: str = "gpt2-124M"):
    import torch
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.models import gpt2  # noqa: F401
    from research_2_b200.models.loading import compute_dtype
    from research_2_b200.parts import Runtime

    data = dict(SIZES[size], n_layer=n_layer)
    arch = architecture_of(data)
    cfg = arch.parse_config(data)
    tensors = arch.random_weights(cfg, SEED, std=0.02)
    tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}  # bf16 weights, as the config names
    return arch.build(cfg, tensors, Runtime(torch.device("cuda:0"), compute_dtype(dtype))), cfg


class DeviceLoopGraph:
    """Forward pass and sampling of a decode-only batch as one CUDA graph WITHOUT the host copies: the
    device-only loop below writes each step's index arrays into `dev` and feeds the sampled tokens back
    as the next step's input ids on the device. It is put together here from the step function's public
    pieces (`forward`, `sample`, a StepContext over a device buffer); the product's own StepGraph, which
    the end-to-end number runs through, copies the batch in and the tokens out inside the graph."""

    def __init__(self, step_fn, batch: int):
        import torch
        from research_2_b200.engine.batch import BatchLayout, StepBatch
        from research_2_b200.engine.step import StepContext
        from research_2_b200.kernels import ops

        self.host = StepBatch(BatchLayout(batch, batch, batch, step_fn.table_widths), pinned=True)
        self.host.max_context_bound = step_fn.model.max_seq_len
        self.host.pad()
        self.host.set_logit_rows([])
        self.host.set_sampling([], [], [], [], [])
        self.dev = torch.zeros(self.host.buf.shape[0], dtype=torch.int32, device=step_fn.device)
        self.dev.copy_(self.host._pinned_tensor)
        ctx = StepContext(self.host, self.dev, counts=(batch, batch, batch))
        side = torch.cuda.Stream(device=step_fn.device)
        side.wait_stream(torch.cuda.current_stream(step_fn.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                step_fn.sample(step_fn.forward(ctx), ctx)
        torch.cuda.current_stream(step_fn.device).wait_stream(side)
        torch.cuda.synchronize(step_fn.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(self.graph, pool=step_fn.graph_pool()):
            self.tokens = step_fn.sample(step_fn.forward(ctx), ctx)
        self.kernels = ops.launch_count() - before


class DecodeLoop:
    """B requests with PROMPT_LEN-token prompts, prefilled through the step function, then
    decoded with the decode graph; the sampled tokens feed the next step on the device."""

    def __init__(self, model, batch: int, n_steps: int):
        import numpy as np
        import torch
        from research_2_b200.cache.manager import CacheManager
        from research_2_b200.engine.step import StepFunction

        self.torch, self.np = torch, np
        self.batch, self.n_steps = batch, n_steps
        pages = batch * (CONTEXT // PAGE)
        self.step_fn = StepFunction(model, PAGE, pages, batch, capture=True)
        self.cache = CacheManager(self.step_fn.cache_groups(), batch, model.max_seq_len)
        gen = torch.Generator().manual_seed(SEED + 100 + batch)
        self.prompts = torch.randint(0, model.vocab_size, (batch, PROMPT_LEN), generator=gen, dtype=torch.int32).numpy()
        total = PROMPT_LEN + n_steps
        assert total <= CONTEXT, f"{PROMPT_LEN} prompt + {n_steps} steps exceed the context {CONTEXT}"
        for r in range(batch):
            self.cache.open(r)
            self.cache.reserve(r, 0, total)
        # prefill, at most 2,048 rows a step; the last prompt token is left for the first decode step
        per_step = max(1, 2048 // (PROMPT_LEN - 1))
        for r0 in range(0, batch, per_step):
            reqs = list(range(r0, min(batch, r0 + per_step)))
            b = self.step_fn.new_batch((PROMPT_LEN - 1) * len(reqs), len(reqs), 0)
            b.set_entries(reqs, [0] * len(reqs), [self.prompts[r, : PROMPT_LEN - 1] for r in reqs])
            self.cache.fill(b)
            b.set_logit_rows([])
            self.step_fn(b)
        torch.cuda.synchronize()
        # every decode step's batch, precomputed into one pinned array
        self.graph = DeviceLoopGraph(self.step_fn, batch)
        host = self.graph.host
        self.skip = host.section("positions")[0]  # input_ids stay on the device
        self.staged = torch.zeros(n_steps, host.buf.shape[0], dtype=torch.int32).pin_memory()
        reqs = list(range(batch))
        for i in range(n_steps):
            host.set_entries(reqs, [PROMPT_LEN - 1 + i] * batch, [[0]] * batch)
            self.cache.fill(host)
            host.set_logit_rows(host.last_rows())
            host.set_sampling([1.0] * batch, [1] * batch, [0] * batch, [0] * batch, [PROMPT_LEN + i] * batch)
            host.pad()
            self.staged[i].copy_(host._pinned_tensor)
        at, _ = host.section("input_ids")
        self.graph.dev[at: at + batch].copy_(torch.from_numpy(self.prompts[:, PROMPT_LEN - 1].copy()))
        self.input_ids = self.graph.dev[at: at + batch]
        self.at = 0

    def run(self, n: int) -> float:
        """n decode steps; returns device milliseconds."""
        torch = self.torch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(n):
            self.graph.dev[self.skip:].copy_(self.staged[self.at, self.skip:], non_blocking=True)
            self.graph.graph.replay()
            self.input_ids.copy_(self.graph.tokens[: self.batch])
            self.at += 1
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    def kv_bytes(self, first_step: int, n: int, model) -> float:
        """Average bytes of cache that one of the steps [first_step, first_step + n) reads."""
        per_token = sum(2 * m.n_kv_heads * m.head_dim for m in model.cache_members) * self.step_fn.arena.tensors[0].element_size()
        ctx = PROMPT_LEN + first_step + (n - 1) / 2.0
        return self.batch * ctx * per_token


def decode_point(model, batch: int, steps: int, warmup: int) -> tuple[float, float, "DecodeLoop", float]:
    loop = DecodeLoop(model, batch, steps + warmup)
    loop.run(warmup)
    ms = loop.run(steps)
    return batch * steps / (ms / 1e3), ms / steps, loop, loop.kv_bytes(warmup, steps, model)


def prefill_point(model, cfg, pk: dict) -> dict:
    import torch
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction

    n_req, length = 2, 1024
    step_fn = StepFunction(model, PAGE, n_req * length // PAGE, n_req, capture=True)  # a shape that repeats runs as a graph
    cache = CacheManager(step_fn.cache_groups(), n_req, model.max_seq_len)
    gen = torch.Generator().manual_seed(SEED + 1)
    prompts = torch.randint(0, model.vocab_size, (n_req, length), generator=gen, dtype=torch.int32).numpy()
    for r in range(n_req):
        cache.open(r)
        cache.reserve(r, 0, length)
    times = []
    for it in range(2 + 5):
        b = step_fn.new_batch(n_req * length, n_req, n_req)
        b.set_entries(list(range(n_req)), [0] * n_req, [prompts[r] for r in range(n_req)])
        cache.fill(b)
        b.set_logit_rows(b.last_rows())
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        step_fn(b)
        stop.record()
        torch.cuda.synchronize()
        if it >= 2:
            times.append(start.elapsed_time(stop))
    ms = statistics.median(times)
    d, f, layers, v, t = cfg.n_embd, cfg.n_inner, cfg.n_layer, cfg.vocab_size, n_req * length
    flops = 2 * t * layers * (3 * d * d + d * d + 2 * d * f) + layers * n_req * 4 * d * length * (length + 1) / 2 + 2 * n_req * d * v
    return {"value": t / (ms / 1e3), "tokens": t, "ms": ms, "frac": flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12)}


def e2e_point(model, batch: int, steps: int, warmup: int) -> dict:
    """Through the Python entry point: submit prompts (host token lists), step, poll tokens."""
    import torch
    from research_2_b200.config.engine_options import EngineOptions
    from research_2_b200.engine.engine import Engine

    opts = EngineOptions(dtype="bfloat16", max_requests=batch, block_size=PAGE, max_batch_tokens=2048, capture=True)
    engine = Engine.for_model(model, opts)
    gen = torch.Generator().manual_seed(SEED + 200)
    prompts = torch.randint(0, model.vocab_size, (batch, PROMPT_LEN), generator=gen).tolist()
    room = CONTEXT - PROMPT_LEN   # tokens a request can still generate
    steps = max(1, min(steps, room - warmup - 6))   # (requests must stay alive through the timed steps)
    rids = [engine.submit(p, max_new_tokens=min(steps + warmup + 8, room)) for p in prompts]
    while True:  # prefill until every request decodes
        engine.step()
        if all(engine.scheduler.request_info(r)["n_tokens"] > PROMPT_LEN for r in rids):
            break
    for _ in range(warmup):
        engine.step()
    for r in rids:
        engine.poll(r)
    h0 = engine.step_fn.h2d_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tokens = 0
    for _ in range(steps):
        engine.step(wait=False)   # launched; the polls below run while the GPU works and see the step before
        for r in rids:
            n_tokens += len(engine.poll(r).new_tokens)
    engine.finish()
    for r in rids:
        n_tokens += len(engine.poll(r).new_tokens)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (engine.step_fn.h2d_bytes - h0) / steps
    engine.close()
    return {"value": batch * steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": 4 * batch, "polled_tokens": n_tokens}


def mixed_point(model, n_requests: int = 64, new_tokens: int = 256) -> dict:
    """A continuous batch through the Python entry point: prompts of 16 to 768 tokens, portions
    of 512 tokens a step beside the decoded tokens of the others (the workload that the baseline
    names for the 355M size, here at the benchmark's own). The first pass captures the graphs of
    the shapes that come; the second is timed by the host's clock."""
    import random

    import torch
    from research_2_b200.config.engine_options import EngineOptions
    from research_2_b200.engine.api import generate_with
    from research_2_b200.engine.engine import Engine

    opts = EngineOptions(dtype="bfloat16", max_requests=n_requests, block_size=PAGE, max_batch_tokens=512 + n_requests, chunk_size=512,
                         capture=True)
    engine = Engine.for_model(model, opts)
    rng = random.Random(SEED + 300)
    gen = torch.Generator().manual_seed(SEED + 300)
    prompts = [torch.randint(0, model.vocab_size, (rng.randint(16, 768),), generator=gen).tolist() for _ in range(n_requests)]
    generate_with(engine, prompts, new_tokens, wait=False)
    engine.request_events()  # (the first pass's records)
    engine.keep_events = True
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = generate_with(engine, prompts, new_tokens, wait=False)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    steps = len(engine.events)
    records = engine.request_events()
    preempted = sum(e.n_preempted for e in engine.events)
    engine.close()
    n_out, n_in = sum(len(o) for o in out), sum(len(p) for p in prompts)
    ttft = sorted(r.time_to_first_token_ms for r in records if r.time_to_first_token_ms is not None)
    return {"generated_per_s": n_out / dt, "tokens_per_s": (n_in + n_out) / dt, "requests": n_requests,
            "prompt_tokens": n_in, "generated_tokens": n_out, "steps": steps, "ms": dt * 1e3, "preemptions": preempted,
            "ttft_ms_median": statistics.median(ttft) if ttft else None, "ttft_ms_p90": ttft[int(0.9 * (len(ttft) - 1))] if ttft else None}


def kernel_points(cfg, batch: int, pk: dict) -> dict:
    """The step's dominant kernels one by one at this configuration's sizes, each timed in a CUDA graph of
    20 launches: microseconds, and the fraction of the measured peak that its bytes (decode: the weights or
    the cache it must read) or its flops (prefill at 2,048 tokens) make of that time."""
    import torch
    from research_2_b200.profiling import kernel_cases

    kernel_cases.configure(cfg.n_embd, cfg.n_inner, cfg.n_head, cfg.head_dim, cfg.vocab_size, PAGE)
    out = {}
    for name, fn, n_bytes, flops in kernel_cases.cases(batch):
        wanted = (name.startswith("decode: ") and "sampling at" not in name and f"{batch} rows x {cfg.n_head} heads" in name or
                  name.startswith("decode: ") and " x " in name and "rows" not in name or
                  name.startswith(f"logits, {batch} rows") or name.startswith("decode: greedy") or
                  name.startswith("prefill") and "2,048" in name or "2 x 1,024" in name and "tcgen05" in name)
        if not wanted:
            continue
        us = kernel_cases.time_in_graph(fn)
        if n_bytes:
            out[name] = {"us": round(us, 2), "GB/s": round(n_bytes / us / 1e3, 1), "frac": round(n_bytes / us / 1e3 / pk["hbm_gbs"], 3)}
        else:
            out[name] = {"us": round(us, 2), "TFLOP/s": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}
    torch.cuda.empty_cache()
    return out


def resident_phases(model, batch: int) -> dict:
    """Where a layer's time goes inside the resident decode kernel (up to 64 rows): the kernel's own clock at
    the end of every phase and at the exit of every grid barrier (`ResidentLayers.stamps`), taken as the latest
    CTA's time minus the latest CTA's at the point before, mean over the middle layers, in microseconds."""
    import torch
    from research_2_b200.engine.step import StepContext
    from research_2_b200.kernels import ops

    before = ops.set_resident_decode_rows(64)
    try:
        loop = DecodeLoop(model, batch, 40)
        resident = getattr(model, "_resident", None)
        if resident is None:
            return {"unavailable": "the model's layers are not of the kind that the resident kernel runs"}
        n_layers = len(resident.schedule)
        n = 1 + 10 * n_layers
        ctx = StepContext(loop.graph.host, loop.graph.dev, counts=(batch, batch, batch))
        loop.run(3)
        for _ in range(3):
            stamps = torch.zeros(3 * n, dtype=torch.int64, device="cuda:0")
            stamps[n: 2 * n] = 1 << 62
            resident.stamps = stamps
            loop.step_fn.sample(loop.step_fn.forward(ctx), ctx)
            torch.cuda.synchronize()
        resident.stamps = None
        early, late = stamps[n: 2 * n].cpu().tolist(), stamps[2 * n:].cpu().tolist()
        names = ["A norm + q/k/v", "barrier", "B attention", "barrier", "C output + residual", "barrier", "D norm + feed-forward in", "barrier",
                 "E feed-forward out + residual", "barrier"]
        layers = range(min(3, n_layers - 1), max(min(3, n_layers - 1) + 1, n_layers - 1))
        out = {"rows": batch, "kernel_us": (late[-1] - early[0]) / 1e3, "phases_us": []}
        for i, name in enumerate(names):
            spans = [(late[1 + 10 * layer + i] - late[10 * layer + i]) / 1e3 for layer in layers]
            out["phases_us"].append([name, round(sum(spans) / len(spans), 2)])
        return out
    finally:
        ops.set_resident_decode_rows(before)


def logits_ctas(model, batch: int) -> dict:
    """How the CTAs of a decode step's last product (the logits) share the GPU: every CTA's own times
    (`ops.gemm_cta_stamps`), in microseconds from the first CTA's start."""
    import torch
    from research_2_b200.kernels import ops

    stamps = torch.zeros(2048, 6, dtype=torch.int64, device="cuda:0")
    ops.gemm_cta_stamps(stamps)
    try:
        loop = DecodeLoop(model, batch, 40)   # (the graph is captured with the buffer in the kernels' arguments)
        loop.run(6)
        torch.cuda.synchronize()
        n = min(ops.gemm_cta_stamps(None), stamps.shape[0])
    finally:
        ops.gemm_cta_stamps(None)
    from research_2_b200.profiling.kernel_cases import summarise_cta_stamps

    return {"rows": batch, **summarise_cta_stamps(stamps, n)}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="gpt2-124M", choices=sorted(SIZES), help="layer sizes (the default is the baseline's benchmark configuration)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has, if memory or time needs it")
    ap.add_argument("--no-points", action="store_true", help="skip prefill, e2e and the batch 1 / 64 points")
    ap.add_argument("--phases", action="store_true", help="print where a layer's time goes inside the resident decode kernel at --batch rows, and stop")
    ap.add_argument("--logits-ctas", action="store_true", help="print when each CTA of a decode step's logits product starts and ends (its waves), and stop")
    ap.add_argument("--prefill", action="store_true", help="print the prefill point (2 x 1,024 tokens in one step) alone, and stop")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.layers is None:
        args.layers = SIZES[args.model]["n_layer"]
    global PROMPT_LEN
    PROMPT_LEN = PROMPT_LENS[args.model]
    steps = min(args.steps, CONTEXT - PROMPT_LEN - args.warmup)
    if args.impl == "reference":
        from baseline import reference_arm

        cfg_data = SIZES[args.model]
        skeleton = {
            "metric": f"decode tokens/s (GPT-2 {args.model[5:]}, batch {args.batch}, {PROMPT_LEN}-token prompts)", "value": None, "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic tokens, random weights (seed 5)", "impl": "reference",
            "config": {"model": args.model, "n_layer": cfg_data["n_layer"], "n_layer_model": cfg_data["n_layer"], "n_embd": cfg_data["n_embd"],
                       "n_head": cfg_data["n_head"], "head_dim": cfg_data["n_embd"] // cfg_data["n_head"], "n_inner": cfg_data["n_inner"],
                       "vocab_size": cfg_data["vocab_size"], "n_positions": cfg_data["n_positions"], "global_batch": args.batch,
                       "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE, "parallelism": "none",
                       "l2": "inputs larger than L2, no flush"},
        }
        return reference_arm.main(args, cfg_data, SEED, PAGE, PROMPT_LEN, CONTEXT, skeleton)

    import torch
    from research_2_b200.kernels import ops

    pk, pk_source = peaks()
    model, cfg = build_model(args.layers, size=args.model)
    if args.phases:
        print(json.dumps(resident_phases(model, args.batch)))
        return 0
    if args.prefill:
        print(json.dumps(prefill_point(model, cfg, pk)))
        return 0
    if args.logits_ctas:
        print(json.dumps(logits_ctas(model, args.batch)))
        return 0
    sampler = ClockSampler()
    sampler.start()
    before = ops.launch_count()
    value, ms_per_step, loop, kv_bytes = decode_point(model, args.batch, steps, args.warmup)
    launches = loop.graph.kernels * steps
    clocks = sampler.stop()
    del before
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + kv_bytes) / (ms_per_step / 1e3) / 1e9
    del loop
    torch.cuda.empty_cache()

    line = {
        "metric": f"decode tokens/s (GPT-2 {args.model[5:]}, batch {args.batch}, {PROMPT_LEN}-token prompts)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic tokens, random weights (seed 5)",
        "impl": "ours",
        "config": {
            "model": args.model, "n_layer": args.layers, "n_layer_model": SIZES[args.model]["n_layer"], "n_embd": cfg.n_embd,
            "n_head": cfg.n_head, "head_dim": cfg.head_dim, "n_inner": cfg.n_inner, "vocab_size": cfg.vocab_size,
            "n_positions": cfg.n_positions, "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "page_size": PAGE, "parallelism": "none", "l2": "inputs larger than L2, no flush", "peaks": pk_source,
        },
        "clocks": clocks, "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
    }
    if not args.no_points:
        line["prefill"] = prefill_point(model, cfg, pk)
        torch.cuda.empty_cache()
        line["e2e"] = e2e_point(model, args.batch, min(steps, 128), args.warmup)
        torch.cuda.empty_cache()
        points = {}
        for b in (1, 64):
            v, _, lp, _ = decode_point(model, b, min(steps, 96), args.warmup)
            points[f"decode_b{b}"] = v
            del lp
            torch.cuda.empty_cache()
        line["points"] = points
        line["mixed"] = mixed_point(model)
        torch.cuda.empty_cache()
        line["kernels"] = kernel_points(cfg, args.batch, pk)
        # the true 32-bit path of the same model (CUDA-core products and attention, no tensor cores)
        del model
        torch.cuda.empty_cache()
        model32, _ = build_model(args.layers, dtype="float32", size=args.model)
        v32, ms32, lp, _ = decode_point(model32, args.batch, min(steps, 24), args.warmup)
        points[f"decode_b{args.batch}_float32"] = v32
        del lp
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
