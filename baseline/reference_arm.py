"""The reference arm of bench.py: the reference's own GPT-2 on the same workload.

`baseline/_ref/` holds the reference's two pure-Python packages, `kelpie_models` and
`kelpie_engine`, unmodified. What runs here is the reference's stock model path on CUDA: its
loader (`gpt2.load` on a model folder), its `gpt2.forward` with its own ops (`layer_norm`,
`gelu`, `paged_attention`: torch bodies and library matrix products) over its own paged cache
layout, and its sampler (`kernels/ops/sample.py`). The reference's scheduler is a Zig library
that cannot be built here, so the step's index arrays (`Tokens`, `Requests`) are made by hand
exactly as the reference's `to_device` makes them from a plan
(kelpie-models/kelpie_models/sdk/device.py:124-149). Nothing of this repository's engine,
models or kernels is on the path; the only thing shared is the model folder on disk (the same
random weights, seed 5).

Timing follows bench.py's contract (warm-up, then K steps between CUDA events; the sampled
tokens feed the next step on the device) so that the two arms are the same measurement.
"""

from __future__ import annotations

import json
import statistics
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def available() -> str | None:
    """None, or why the arm cannot run."""
    if not (REF / "kelpie_models" / "models" / "torch" / "gpt2.py").is_file():
        return ("baseline/_ref holds no kelpie_models package (pip cannot build it offline: its build backend, "
                "hatchling, is not in the image; the package folders are copied there by hand)")
    return None


class ReferenceGPT2:
    def __init__(self, folder: str, dtype_name: str, page: int, n_pages: int, device: str = "cuda:0"):
        import torch

        if str(REF) not in sys.path:
            sys.path.insert(0, str(REF))
        from kelpie_models.kernels.ops.sample import sample
        from kelpie_models.models.torch import gpt2
        from kelpie_models.sdk.device import Host, Requests, Tokens
        from kelpie_models.sdk.taps import taps_for

        self.torch, self.gpt2, self.sample_op = torch, gpt2, sample
        self.Tokens, self.Requests, self.Host, self.taps_for = Tokens, Requests, Host, taps_for
        self.device = torch.device(device)
        self.dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype_name]
        self.weights, self.cfg = gpt2.load(self.device, self.dtype, checkpoint=folder)
        self.page, self.n_pages = page, n_pages
        # the reference's layout: one member per layer, [pages, 2, block, H, D] as a view whose
        # K and V planes flatten without a copy (kernels/ops/paged_attention.py:28-42)
        self.kv = [tuple(
            torch.zeros(n_pages + 1, page, 2, self.cfg.n_kv_heads, self.cfg.head_dim, dtype=self.dtype, device=self.device)
            .permute(0, 2, 1, 3, 4) for _ in range(self.cfg.n_layers))]
        self.width = -(-self.cfg.max_seq_len // page)

    def views(self, input_ids, starts: list[int], rows: list[int], tables):
        """Tokens and Requests of entries (first position, rows) whose pages are `tables` [R, P]."""
        torch = self.torch
        qsl = [0]
        for n in rows:
            qsl.append(qsl[-1] + n)
        pos = torch.cat([torch.arange(s, s + n, dtype=torch.int32) for s, n in zip(starts, rows)])
        entry = torch.cat([torch.full((n,), e, dtype=torch.int32) for e, n in enumerate(rows)])
        slots = (tables[entry.long(), (pos // self.page).long()] * self.page + pos % self.page).to(torch.int32)
        seq = [s + n for s, n in zip(starts, rows)]
        dev = self.device
        last = torch.tensor([q - 1 for q in qsl[1:]], dtype=torch.int32)
        tokens = self.Tokens(input_ids=input_ids, positions=pos.to(dev, non_blocking=True),
                             row_request=entry.to(dev, non_blocking=True), last_rows=last.to(dev, non_blocking=True),
                             tail_rows=last.long()[:, None].to(dev, non_blocking=True))
        r = len(rows)
        requests = self.Requests(
            query_start_loc=torch.tensor(qsl, dtype=torch.int32).to(dev, non_blocking=True),
            seq_lens=torch.tensor(seq, dtype=torch.int32).to(dev, non_blocking=True),
            slot_mapping=(slots.to(dev, non_blocking=True),), block_tables=(tables.to(dev, non_blocking=True),),
            kind=torch.zeros(r, dtype=torch.int32, device=dev), n_extra=torch.zeros(r, dtype=torch.int32, device=dev),
            host=self.Host(r, qsl[-1], tuple(qsl), tuple(seq), tuple(range(r))))
        return tokens, requests

    def step(self, tokens, requests):
        """-> greedy tokens i32[R] on the device (the reference's all-greedy sampler path)."""
        torch = self.torch
        with torch.no_grad():
            logits = self.gpt2.forward(self.weights, self.cfg, tokens, requests, self.kv, self.taps_for(()))
            r = logits.shape[0]
            out = self.sample_op(logits, torch.ones(r, device=self.device), torch.ones(r, dtype=torch.int32, device=self.device),
                                 torch.zeros(2, dtype=torch.uint32, device=self.device),
                                 torch.full((r, 0), -1, dtype=torch.int32, device=self.device), True, 0)
        return out[:, 0]


def _tables(torch, batch: int, width: int):
    """Request r holds pages r * width + 1 ... (page 0 is the null page)."""
    return (torch.arange(batch * width, dtype=torch.int32).view(batch, width) + 1)


def decode_point(model: ReferenceGPT2, batch: int, prompt_len: int, steps: int, warmup: int, seed: int, e2e: bool = False):
    """`batch` requests with `prompt_len`-token prompts, prefilled one request a step, then
    decoded. -> (tokens/s, ms per step). With `e2e` every step's token ids come from host
    memory and its sampled tokens are read back to the host, timed by the host's clock."""
    torch = model.torch
    gen = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, model.cfg.vocab, (batch, prompt_len), generator=gen, dtype=torch.int32)
    tables = _tables(torch, batch, model.width)
    for r in range(batch):  # the last prompt token is left for the first decode step
        tok, req = model.views(prompts[r, : prompt_len - 1].to(model.device), [0], [prompt_len - 1], tables[r: r + 1])
        model.step(tok, req)
    ids = prompts[:, prompt_len - 1].to(model.device)
    host_ids = prompts[:, prompt_len - 1].clone()
    at = prompt_len - 1

    def run(n: int) -> float:
        nonlocal ids, host_ids, at
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        start.record()
        for _ in range(n):
            if e2e:
                ids = host_ids.pin_memory().to(model.device, non_blocking=True)
            tok, req = model.views(ids, [at] * batch, [1] * batch, tables)
            ids = model.step(tok, req)
            if e2e:
                host_ids = ids.cpu()
            at += 1
        stop.record()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 if e2e else start.elapsed_time(stop)

    run(warmup)
    ms = run(steps)
    return batch * steps / (ms / 1e3), ms / steps


def prefill_point(model: ReferenceGPT2, n_req: int, length: int, seed: int) -> dict:
    torch = model.torch
    gen = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, model.cfg.vocab, (n_req, length), generator=gen, dtype=torch.int32)
    tables = _tables(torch, n_req, model.width)
    times = []
    for it in range(1 + 3):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        tok, req = model.views(prompts.reshape(-1).to(model.device), [0] * n_req, [length] * n_req, tables)
        model.step(tok, req)
        stop.record()
        torch.cuda.synchronize()
        if it >= 1:
            times.append(start.elapsed_time(stop))
    ms = statistics.median(times)
    return {"value": n_req * length / (ms / 1e3), "tokens": n_req * length, "ms": ms}


def main(args, config: dict, seed: int, page: int, prompt_len: int, context: int, line: dict) -> int:
    """Prints the reference's JSON line for the workload that `line` (bench.py's own skeleton:
    metric, config, steps ...) describes."""
    why = available()
    if why is not None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        return 0
    sys.path.insert(0, str(ROOT))
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.models import gpt2 as _our_gpt2_config  # noqa: F401  (the random-weights writer only)
    from research_2_b200.weights import write_model_folder

    steps, warmup, batch = line["steps"], line["warmup"], args.batch
    with tempfile.TemporaryDirectory() as tmp:
        arch = architecture_of(config)
        folder = write_model_folder(Path(tmp) / "model", arch, arch.parse_config(config),
                                    seed, "bfloat16", std=0.02)
        data = json.loads((folder / "config.json").read_text())
        data["eos_token_id"] = data.get("eos_token_id") or 0   # the reference's config reader wants an integer
        (folder / "config.json").write_text(json.dumps(data))
        results = {}
        for dtype_name in ("bfloat16", "float32"):
            model = ReferenceGPT2(str(folder), dtype_name, page, 64 * (context // page))
            value, ms = decode_point(model, batch, prompt_len, steps, warmup, seed + 100 + batch)
            results[dtype_name] = {"value": value, "ms_per_step": ms}
            if dtype_name == "bfloat16":
                e2e_value, _ = decode_point(model, batch, prompt_len, min(steps, 128), warmup, seed + 200, e2e=True)
                extra = {}
                if not args.no_points:
                    extra["prefill"] = prefill_point(model, 2, 1024, seed + 1)
                    extra["points"] = {f"decode_b{b}": decode_point(model, b, prompt_len, min(steps, 32), warmup, seed + 100 + b)[0]
                                       for b in (1, 64)}
            del model
            torch.cuda.empty_cache()
    line.update({
        "impl": "reference", "value": results["bfloat16"]["value"], "ms_per_step": results["bfloat16"]["ms_per_step"],
        "dtype": "bf16", "same_config": True,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch * (4 + model_table_ints(context, page)),
                "d2h_bytes_per_step": 4 * batch},
        "stock_float32": results["float32"],
        "how": "unmodified kelpie_models gpt2.forward + kernels/ops/sample.py on cuda:0 (torch bodies, library products), eager; "
               "index arrays made by hand as sdk/device.py:124-149 does; bfloat16 via gpt2.load(dtype=...), float32 is its stock dtype",
        "gpu_launches": None,
    })
    line.update(extra)
    print(json.dumps(line))
    return 0


def model_table_ints(context: int, page: int) -> int:
    """int32 values per request that a step copies besides its token: position, entry, slot, last row, q_start, seq_len ... and its block table."""
    return 6 + context // page
