"""Command line: generate tokens, write a random model folder, replay a trace.

Option names follow the reference's `kelpie serve` where it has them (`--model`, `--device`,
`--max-requests`, `--num-slabs`, `--capture/--no-capture`: kelpie-http/kelpie_http/sdk/serve.py:
84-124) and its `Engine.submit` for the request (`max_new_tokens`, `temperature`, `top_k`,
`stop_token_ids`: kelpie-engine/kelpie_engine/sdk/engine.py:284-305). The reference has no
offline generation command; this one takes and prints token ids ("the core sees token ids
only", kelpie/docs/core-api.md:18).

    python -m research_2_b200 generate --model DIR --prompt-tokens 5,17,3 --max-new-tokens 16
    python -m research_2_b200 random --config config.json --seed 0 --out DIR
    python -m research_2_b200 replay --model DIR --dtype float32 --out DIR --max-tokens 256 < steps.jsonl
"""

from __future__ import annotations

import argparse
import json
import sys


def _engine_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True, help="a folder with config.json and model.safetensors")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    p.add_argument("--capture", action=argparse.BooleanOptionalAction, default=None,
                   help="CUDA graphs for decode-only steps (default: on for bfloat16)")
    p.add_argument("--max-requests", type=int, default=8)
    p.add_argument("--num-slabs", type=int, default=0, help="cache pages per group; 0 = room for max-requests full sequences")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--max-seq-len", type=int, default=0, help="0 = the model's own maximum")
    p.add_argument("--max-batch-tokens", type=int, default=1024)
    p.add_argument("--max-batch-reqs", type=int, default=0)
    p.add_argument("--chunk-size", type=int, default=0,
                   help="most tokens of a prompt portion that does not finish its prompt; 0 = the token budget decides")
    p.add_argument("--reserve-ratio", type=float, default=0.0)
    p.add_argument("--order", default="running_first", choices=("running_first", "waiting_first"))


def _ints(text: str) -> list[int]:
    return [int(t) for t in text.replace(" ", "").split(",") if t]


def cmd_generate(args) -> int:
    import torch

    from .engine.api import generate

    prompts = [_ints(p) for p in args.prompt_tokens]
    if args.prompt_len:
        from .config.registry import load_config

        _, cfg = load_config(args.model)
        gen = torch.Generator().manual_seed(args.seed)
        prompts += [torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=gen).tolist() for _ in range(args.num_prompts)]
    if not prompts:
        print("generate: give --prompt-tokens (repeatable) or --prompt-len", file=sys.stderr)
        return 2
    outs = generate(
        args.model, prompts, args.max_new_tokens, temperature=args.temperature, top_k=args.top_k, seed=args.seed,
        stop_token_ids=_ints(args.stop_token_ids), device=args.device, dtype=args.dtype, capture=args.capture,
        max_requests=args.max_requests, num_slabs=args.num_slabs, block_size=args.block_size, max_seq_len=args.max_seq_len,
        max_batch_tokens=args.max_batch_tokens, max_batch_reqs=args.max_batch_reqs, chunk_size=args.chunk_size, reserve_ratio=args.reserve_ratio,
        order=args.order)
    for prompt, out in zip(prompts, outs):
        print(json.dumps({"prompt": prompt, "tokens": out}))
    return 0


def cmd_random(args) -> int:
    from .config.registry import architecture_of
    from .models import gpt2  # noqa: F401
    from .weights.model_folder import write_model_folder

    with open(args.config) as f:
        data = json.load(f)
    arch = architecture_of(data)
    folder = write_model_folder(args.out, arch, arch.parse_config(data), args.seed, args.store_dtype, std=args.std)
    print(folder)
    return 0


def cmd_replay(args) -> int:
    from .engine.replay import main as replay_main

    argv = ["--model", args.model, "--dtype", args.dtype, "--out", args.out, "--max-tokens", str(args.max_tokens),
            "--block-size", str(args.block_size), "--device", args.device]
    return replay_main(argv)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="research_2_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="run prompts (token ids) to completion and print token ids")
    _engine_flags(g)
    g.add_argument("--prompt-tokens", action="append", default=[], metavar="1,2,3", help="one prompt; repeat for more")
    g.add_argument("--prompt-len", type=int, default=0, help="random prompts of this length instead")
    g.add_argument("--num-prompts", type=int, default=1)
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--stop-token-ids", default="", metavar="7,9")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("random", help="write a model folder with random weights from a config.json and a seed")
    r.add_argument("--config", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--store-dtype", default="bfloat16", choices=("bfloat16", "float32"))
    r.set_defaults(fn=cmd_random)
    t = sub.add_parser("replay", help="feed given tokens step by step and write logits (bin/trace_run)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--block-size", type=int, default=16)
    t.add_argument("--device", default="cuda:0")
    t.set_defaults(fn=cmd_replay)
    args = ap.parse_args(argv)
    return args.fn(args)
