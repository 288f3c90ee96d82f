"""The Python entry point: `run(model_dir, ...)` gives an Engine, `generate(...)` runs a batch
of prompts to completion. `run` follows the reference's `with run(gpt2, device=...) as engine:
rid = engine.submit(prompt, max_new_tokens=12); done = engine.wait(rid)`
(kelpie/examples/run_gpt2.py:51-54; kelpie-models/kelpie_models/sdk/run.py:597-610)."""

from __future__ import annotations

from ..config.engine_options import EngineOptions
from ..models.loading import load_model
from .engine import Engine


def run(model, *, device: str = "cuda:0", dtype: str = "bfloat16", **options) -> Engine:
    """`model` is a model folder (config.json + model.safetensors) or an already loaded model.
    Keyword options are EngineOptions fields (max_requests, num_slabs, block_size,
    max_batch_tokens, max_batch_reqs, chunk_size, max_seq_len, reserve_ratio, order, capture, seed)."""
    opts = EngineOptions(dtype=dtype, **options)
    if isinstance(model, (str, bytes)) or hasattr(model, "__fspath__"):
        model = load_model(model, dtype=dtype, device=device)
    return Engine.for_model(model, opts)


def generate(  # noqa: PLR0913
    model, prompts, max_new_tokens: int, temperature: float = 0.0, top_k: int = 0, seed: int = 0,
    stop_token_ids=(), *, device: str = "cuda:0", dtype: str = "bfloat16", **options,
) -> list[list[int]]:
    """Token ids in, token ids out: every prompt's continuation, in the order of `prompts`.
    Request i draws with key (seed, i), so its tokens do not depend on the batch it runs in."""
    options.setdefault("max_requests", max(1, min(len(prompts), 256)))
    with run(model, device=device, dtype=dtype, seed=seed, **options) as engine:
        return generate_with(engine, prompts, max_new_tokens, temperature, top_k, seed, stop_token_ids)


def generate_with(engine: Engine, prompts, max_new_tokens, temperature=0.0, top_k=0, seed=0, stop_token_ids=(), wait=False):
    """Continuations of all prompts through one engine, as many at a time as it has request slots. With
    `wait=False` (the default) a step is only launched before the requests are polled, so the host's share
    of a step runs while the GPU works; the tokens are the same."""
    from .scheduler import Full

    out: list[list[int]] = [[] for _ in prompts]
    live: dict[int, int] = {}
    nxt = 0
    while nxt < len(prompts) or live:
        while nxt < len(prompts):
            try:
                rid = engine.submit(prompts[nxt], max_new_tokens, temperature, stop_token_ids, top_k,
                                    seed=(seed & 0xFFFFFFFF) | (nxt << 32))
            except Full:
                break
            live[rid] = nxt
            nxt += 1
        engine.step(wait=wait)  # (wait=False: the polls below run while the GPU works, and see the step before)
        for rid in list(live):
            p = engine.poll(rid)
            out[live[rid]] += p.new_tokens
            if p.finished:
                del live[rid]
    return out
