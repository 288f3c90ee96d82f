"""Runs the hot kernels of a decoder of given layer sizes, each case twice, for ncu to capture one
kernel at a time (a few launches, one kernel name: a capture that ends by itself):

    python -m research_2_b200.profiling.kernel_cases --width 768 --inner 3072 --heads 12 --head-dim 64 \
        --vocab 50257 --case "qkv product, 2,048" &&
    ncu --set full --clock-control none -k regex:gemm_tc -c 2 -o qkv \
        python -m research_2_b200.profiling.kernel_cases --width 768 --inner 3072 --heads 12 --head-dim 64 \
        --vocab 50257 --case "qkv product, 2,048"

The sizes are arguments: nothing about a model lives here (bench.py passes its configuration's).
`--case TEXT` keeps the cases whose name contains TEXT; `--list` prints the names. With `--time`
each case is timed inside a CUDA graph of 20 launches (CUDA events around two replays; the same
buffers every launch, so whatever fits the L2 stays there) and microseconds per launch are printed.

Cases: prefill products at 2,048 and 8,192 tokens (q/k/v; the feed-forward's first product with its
activation), the logits product for 8 and 64 rows, a decode step's kernels at 8 rows (products with the
LayerNorm inside, attention with cache write, sampling), decode attention for 64 rows at context 640,
prefill attention (the tcgen05 kernel, then the mma.sync kernel) for 2 x and 8 x 1,024 tokens, one prompt of
128 to 1,024 tokens, a ragged length, and single decoded tokens beside a portion of a prompt.
"""
import argparse
import sys

import torch

from ..kernels import ops

dev = "cuda:0"
D = F = H = HD = V = 0   # set from the arguments
PS = 16


def paged(batch):
    n_pages = batch * (1024 // PS) + 1
    page_stride = 2 * H * PS * HD
    pool = torch.randn(n_pages, page_stride, device=dev).bfloat16()
    flat = pool.view(-1)
    tables = torch.arange(1, n_pages, dtype=torch.int32, device=dev).view(batch, 1024 // PS).contiguous()
    return flat, flat[H * PS * HD:], tables, page_stride, n_pages


def cases(rows: int = 8):
    """(name, function, bytes that the case must read, flops) tuples; every function launches the
    kernels of one case once. `rows` is the batch of the decode cases."""
    torch.manual_seed(0)
    Q = H * HD
    x = torch.randn(2048, D, device=dev).bfloat16()
    wqkv = (torch.randn(D, 3 * Q, device=dev) * 0.02).bfloat16()
    wfc = (torch.randn(D, F, device=dev) * 0.02).bfloat16()
    wproj = (torch.randn(Q, D, device=dev) * 0.02).bfloat16()
    wproj2 = (torch.randn(F, D, device=dev) * 0.02).bfloat16()
    wte = (torch.randn(V, D, device=dev) * 0.02).bfloat16()
    bf, bqkv, bd = torch.zeros(F, device=dev), torch.zeros(3 * Q, device=dev), torch.zeros(D, device=dev)
    x8k = torch.randn(8192, D, device=dev).bfloat16()
    h2k = torch.randn(2048, F, device=dev).bfloat16()
    r2k = torch.randn(2048, D, device=dev)
    out = []
    for t, xt in ((2048, x), (8192, x8k)):
        out += [
            (f"prefill: qkv product, {t:,} x {D:,} x {3 * Q:,}", lambda xt=xt: ops.linear(xt, wqkv, bqkv), 0, 2 * t * D * 3 * Q),
            (f"prefill: fc product with gelu, {t:,} x {D:,} x {F:,}", lambda xt=xt: ops.linear(xt, wfc, bf, act="gelu_new"), 0, 2 * t * D * F),
        ]
    # the same q/k/v product with the keys and values going straight into the rows' cache slots (2 x 1,024 tokens)
    kc2, vc2, _, stride2, pages2 = paged(2)
    slots2 = torch.arange(PS, PS + 2048, dtype=torch.int32, device=dev)
    scatter = ops.kv_scatter(slots2, kc2, vc2, stride2, PS, pages2, Q, Q, HD)
    q_out = torch.empty(2048, 3 * Q, device=dev, dtype=torch.bfloat16)
    out.append((f"prefill: qkv product with cache write, 2,048 x {D:,} x {3 * Q:,}", lambda: ops.linear(x, wqkv, bqkv, out=q_out, kv=scatter), 0, 2 * 2048 * D * 3 * Q))
    out += [
        (f"prefill: attention output product + residual, 2,048 x {Q:,} x {D:,}", lambda: ops.linear(x[:, :Q].contiguous() if Q != D else x, wproj, bd, residual=r2k), 0, 2 * 2048 * Q * D),
        (f"prefill: mlp output product + residual, 2,048 x {F:,} x {D:,}", lambda: ops.linear(h2k, wproj2, bd, residual=r2k), 0, 2 * 2048 * F * D),
    ]
    h128, r128 = h2k[:128].contiguous(), r2k[:128].contiguous()
    out.append((f"prefill: mlp output product + residual, 128 x {F:,} x {D:,} (6 tiles: what one SM takes in)",
                lambda: ops.linear(h128, wproj2, bd, residual=r128), 0, 2 * 128 * F * D))
    ln_out, ln_g, ln_b = torch.empty(2048, D, device=dev, dtype=torch.bfloat16), torch.ones(D, device=dev), torch.zeros(D, device=dev)
    out.append((f"prefill: LayerNorm, 2,048 x {D:,}", lambda: ops.layer_norm(r2k, ln_g, ln_b, 1e-5, torch.bfloat16, out=ln_out), 2048 * D * 6, 0))
    for r in sorted({8, 64, rows}):
        xr = x[:r].contiguous()
        out.append((f"logits, {r} rows x {D:,} x {V:,}", lambda xr=xr: ops.linear(xr, wte, None, w_is_nk=True, out_dtype=torch.float32),
                    wte.numel() * 2, 2 * r * D * V))
    # a decode step's kernels (the products of one layer with the LayerNorm inside, attention with cache write, sampling)
    hr = torch.randn(rows, D, device=dev)  # the residual stream is float32
    gamma, beta = torch.ones(D, device=dev), torch.zeros(D, device=dev)
    ar = torch.randn(rows, Q, device=dev).bfloat16()
    fr = torch.randn(rows, F, device=dev).bfloat16()
    normed = lambda: ops.NormedRows(hr, gamma, beta, 1e-5, torch.bfloat16)
    out += [
        (f"decode: LayerNorm + qkv product, {rows} x {D:,} x {3 * Q:,}", lambda: ops.linear(normed(), wqkv, bqkv), wqkv.numel() * 2, 2 * rows * D * 3 * Q),
        (f"decode: attention output product + residual, {rows} x {Q:,} x {D:,}", lambda: ops.linear(ar, wproj, bd, residual=hr), wproj.numel() * 2, 2 * rows * Q * D),
        (f"decode: LayerNorm + fc product with gelu, {rows} x {D:,} x {F:,}", lambda: ops.linear(normed(), wfc, bf, act="gelu_new"), wfc.numel() * 2, 2 * rows * D * F),
        (f"decode: mlp output product + residual, {rows} x {F:,} x {D:,}", lambda: ops.linear(fr, wproj2, bd, residual=hr), wproj2.numel() * 2, 2 * rows * F * D),
    ]
    logits = torch.randn(rows, V, device=dev)
    zeros_i = torch.zeros(rows, dtype=torch.int32, device=dev)
    ones_i, temp = torch.ones(rows, dtype=torch.int32, device=dev), torch.full((rows,), 0.8, device=dev)
    k40 = torch.full((rows,), 40, dtype=torch.int32, device=dev)
    out += [
        (f"decode: greedy sampling, {rows} rows x {V:,}", lambda: ops.sample(logits, temp, ones_i, zeros_i, zeros_i, zeros_i), rows * V * 4, 0),
        (f"decode: sampling at temperature 0.8, {rows} rows x {V:,}", lambda: ops.sample(logits, temp, zeros_i, zeros_i, zeros_i, zeros_i), rows * V * 4, 0),
        (f"decode: sampling at temperature 0.8 with top-k 40, {rows} rows x {V:,}", lambda: ops.sample(logits, temp, k40, zeros_i, zeros_i, zeros_i), rows * V * 4, 0),
    ]
    for batch, ctx_len in sorted({(rows, 768), (64, 640)}):
        kc, vc, tables, page_stride, n_pages = paged(batch)
        qkv = torch.randn(batch, 3 * Q, device=dev).bfloat16()
        row_ids = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), ctx_len - 1, dtype=torch.int32, device=dev)
        lens = torch.full((batch,), ctx_len, dtype=torch.int32, device=dev)
        slots = (tables[:, (ctx_len - 1) // PS] * PS + (ctx_len - 1) % PS).to(torch.int32)
        out.append((f"decode: attention with cache write, {batch} rows x {H} heads, context {ctx_len}",
                    lambda qkv=qkv, slots=slots, kc=kc, vc=vc, page_stride=page_stride, n_pages=n_pages, tables=tables, row_ids=row_ids,
                    pos=pos, lens=lens: ops.decode_attention_fused(qkv[:, :Q], qkv[:, Q: 2 * Q], qkv[:, 2 * Q:], slots, kc, vc, page_stride,
                                                                   PS, n_pages, tables, row_ids, pos, lens, H, H, HD, HD**-0.5, 0, 1024),
                    batch * ctx_len * 2 * Q * 2, 4 * batch * ctx_len * Q))
    # prefill attention: the tcgen05 kernel, then the mma.sync one. 2 and 8 prompts of 1,024 tokens; one prompt of 128 to
    # 1,024 tokens (every CTA alone on an SM: the time of a key tile and what a CTA costs besides); a length that is no
    # multiple of 128; single decoded tokens (context 600 and up) beside a portion of a prompt
    def attention_case(name, entries):   # entries: (rows, context length after them)
        batch = len(entries)
        rows = [r for r, _ in entries]
        kc, vc, tables, page_stride, n_pages = paged(batch)
        n = sum(rows)
        q = torch.randn(n, Q, device=dev).bfloat16()
        row_entry = torch.cat([torch.full((r,), e, dtype=torch.int32) for e, r in enumerate(rows)]).to(dev)
        positions = torch.cat([torch.arange(length - r, length, dtype=torch.int32) for r, length in entries]).to(dev)
        lens = torch.tensor([length for _, length in entries], dtype=torch.int32, device=dev)
        q_start = torch.tensor([sum(rows[:i]) for i in range(batch + 1)], dtype=torch.int32, device=dev)
        n_tiles = sum((r + 63) // 64 for r in rows)

        def attention(tc):
            before = ops.use_prefill_tc(tc)
            ops.paged_attention(q, kc, vc, page_stride, PS, n_pages, tables, row_entry, positions, lens, H, H, HD, HD**-0.5, 0,
                                q_start=q_start, n_tiles=n_tiles)
            ops.use_prefill_tc(before)

        flops = sum(4 * Q * (r * (length - r) + r * (r + 1) // 2) for r, length in entries)
        out.append((f"prefill attention on tcgen05, {name} x {H} heads", lambda: attention(True), 0, flops))
        out.append((f"prefill attention on mma.sync, {name} x {H} heads", lambda: attention(False), 0, flops))

    attention_case("2 x 1,024 tokens", [(1024, 1024)] * 2)
    attention_case("8 x 1,024 tokens", [(1024, 1024)] * 8)
    for n in (128, 512, 1024):
        attention_case(f"1 x {n:,} tokens", [(n, n)])
    attention_case("2 x 1,000 tokens", [(1000, 1000)] * 2)
    attention_case("64 decoded tokens beside a portion of 448", [(1, 600 + i) for i in range(64)] + [(448, 704)])
    return out


def time_in_graph(fn, launches=20) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / (2 * launches) * 1e3


def configure(width: int, inner: int, heads: int, head_dim: int, vocab: int, page_size: int = 16) -> None:
    """The layer sizes that `cases` builds its tensors for."""
    global D, F, H, HD, V, PS
    if width < 1 or heads * head_dim < 1:
        raise ValueError("sizes must be positive")
    D, F, H, HD, V, PS = width, inner, heads, head_dim, vocab, page_size


def summarise_cta_stamps(stamps: torch.Tensor, n: int) -> dict:
    """Every CTA's six times (`ops.gemm_cta_stamps`) as waves (CTAs that start within 2 us of one another),
    medians and the kernel's span, in microseconds from the first CTA's start."""
    import numpy as np

    t = stamps[:n].cpu().numpy().astype(np.int64)
    t = (t - t[:, 0].min()) / 1e3
    t[:, 3] = np.maximum(t[:, 3], t[:, 2])   # (forms without a norm inside leave this time unset)
    names = ["start", "before the wait", "after the wait", "tokens normalised", "products complete", "end"]
    starts = np.sort(t[:, 0])
    waves, at = [], 0
    while at < n:
        upto = int(np.searchsorted(starts, starts[at] + 2.0, side="right"))
        waves.append({"ctas": upto - at, "from_us": round(float(starts[at]), 2)})
        at = upto
    seg = np.diff(t, axis=1)
    return {"ctas": n, "waves": waves,
            "median_us": {name: round(float(np.median(t[:, i])), 2) for i, name in enumerate(names)},
            "segments_median_us": {name: round(float(v), 2) for name, v in zip(["set-up", "wait", "norm", "products", "epilogue"], np.median(seg, axis=0))},
            "cta_life_median_us": round(float(np.median(t[:, 5] - t[:, 0])), 2),
            "kernel_us": round(float(t[:, 5].max()), 2), "after_the_wait_us": round(float(t[:, 5].max() - np.median(t[:, 2])), 2)}


def main(argv):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--width", type=int, required=True)
    ap.add_argument("--inner", type=int, required=True)
    ap.add_argument("--heads", type=int, required=True)
    ap.add_argument("--head-dim", type=int, required=True)
    ap.add_argument("--vocab", type=int, required=True)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--rows", type=int, default=8, help="the batch of the decode cases")
    ap.add_argument("--case", default="", help="keep the cases whose name contains this text")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--ctas", action="store_true", help="for a case that is one tensor-core product (single-CTA form): when each of its CTAs starts and ends")
    args = ap.parse_args(argv)
    configure(args.width, args.inner, args.heads, args.head_dim, args.vocab, args.page_size)
    for name, fn, n_bytes, flops in cases(args.rows):
        if args.case not in name:
            continue
        if args.list:
            print(name)
        elif args.ctas:
            import json

            stamps = torch.zeros(4096, 6, dtype=torch.int64, device=dev)
            fn()
            ops.gemm_cta_stamps(stamps)
            try:
                fn()
                torch.cuda.synchronize()
                n = min(ops.gemm_cta_stamps(None), stamps.shape[0])
            finally:
                ops.gemm_cta_stamps(None)
            print(name, json.dumps(summarise_cta_stamps(stamps, n)))
        elif args.time:
            us = time_in_graph(fn)
            rate = f"{n_bytes / us / 1e3:7.0f} GB/s" if n_bytes else f"{flops / us / 1e6:7.0f} TFLOP/s"
            print(f"{us:8.1f} us  {rate}  {name}")
        else:
            fn()
            fn()
    torch.cuda.synchronize()
    print("ok", ops.device_errors())


if __name__ == "__main__":
    main(sys.argv[1:])
