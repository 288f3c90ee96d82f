"""Runs each hot kernel twice at benchmark shapes (GPT-2 124M), for ncu to capture:

    ncu --set full --clock-control none -k regex:'gemm_tc|mlp_fused|decode_kernel|prefill' -c 40 \
        -o kernels python -m research_2_b200.profiling.kernel_cases

With `--time` it instead times each case inside a CUDA graph of 20 launches (CUDA events around
two replays; the same buffers every launch, so whatever fits the L2 stays there) and prints
microseconds per launch.

Shapes: prefill products at 2,048 tokens (QKV and the MLP's first product with gelu) and at 8,192
tokens (the same two: persistent CTA pairs), the tied logits product for 8 and 64 rows (77 MB of
weights), a decode step's kernels at 8 rows, decode attention for 64 rows at context 640 (126 MB of cache), prefill attention for
2 x 1,024 and 8 x 1,024 tokens (the tcgen05 kernel `prefill_tc_kernel`, then the mma.sync kernel
`prefill_kernel`).
"""
import sys

import torch

from ..kernels import ops

dev = "cuda:0"
D, F, H, HD, V, PS = 768, 3072, 12, 64, 50257, 16


def paged(batch):
    n_pages = batch * (1024 // PS) + 1
    page_stride = 2 * H * PS * HD
    pool = torch.randn(n_pages, page_stride, device=dev).bfloat16()
    flat = pool.view(-1)
    tables = torch.arange(1, n_pages, dtype=torch.int32, device=dev).view(batch, 1024 // PS).contiguous()
    return flat, flat[H * PS * HD:], tables, page_stride, n_pages


def cases():
    """(name, function) pairs; every function launches the kernels of one case once."""
    torch.manual_seed(0)
    x = torch.randn(2048, D, device=dev).bfloat16()
    wqkv = (torch.randn(D, 3 * D, device=dev) * 0.02).bfloat16()
    wfc = (torch.randn(D, F, device=dev) * 0.02).bfloat16()
    wte = (torch.randn(V, D, device=dev) * 0.02).bfloat16()
    bias = torch.zeros(F, device=dev)
    bqkv = bias[: 3 * D].contiguous()
    x8k = torch.randn(8192, D, device=dev).bfloat16()
    x8, x64 = x[:8].contiguous(), x[:64].contiguous()
    out = [
        ("qkv product, 2,048 x 768 x 2,304", lambda: ops.linear(x, wqkv, bqkv)),
        ("fc product with gelu, 2,048 x 768 x 3,072", lambda: ops.linear(x, wfc, bias, act="gelu_new")),
        ("qkv product, 8,192 x 768 x 2,304", lambda: ops.linear(x8k, wqkv, bqkv)),
        ("fc product with gelu, 8,192 x 768 x 3,072", lambda: ops.linear(x8k, wfc, bias, act="gelu_new")),
        ("logits, 8 rows x 768 x 50,257", lambda: ops.linear(x8, wte, None, w_is_nk=True, out_dtype=torch.float32)),
        ("logits, 64 rows x 768 x 50,257", lambda: ops.linear(x64, wte, None, w_is_nk=True, out_dtype=torch.float32)),
    ]
    # a decode step's kernels at 8 rows (the products of one layer, the fused attention, sampling)
    h8 = torch.randn(8, D, device=dev)  # the residual stream is float32
    gamma, beta = torch.ones(D, device=dev), torch.zeros(D, device=dev)
    wproj = (torch.randn(D, D, device=dev) * 0.02).bfloat16()
    wproj2 = (torch.randn(F, D, device=dev) * 0.02).bfloat16()
    a8 = torch.randn(8, D, device=dev).bfloat16()
    f8 = torch.randn(8, F, device=dev).bfloat16()
    bd = bias[:D].contiguous()
    normed = lambda: ops.NormedRows(h8, gamma, beta, 1e-5, torch.bfloat16)
    out += [
        ("decode: LayerNorm + qkv product, 8 x 768 x 2,304", lambda: ops.linear(normed(), wqkv, bqkv)),
        ("decode: attention output product + residual, 8 x 768 x 768", lambda: ops.linear(a8, wproj, bd, residual=h8)),
        ("decode: LayerNorm + fc product with gelu, 8 x 768 x 3,072", lambda: ops.linear(normed(), wfc, bias, act="gelu_new")),
        ("decode: mlp output product + residual, 8 x 3,072 x 768", lambda: ops.linear(f8, wproj2, bd, residual=h8)),
    ]
    out.append(("decode: feed-forward in one kernel (off by default), 8 x 768 x 3,072 x 768",
                lambda: (ops.use_fused_mlp(True), ops.mlp(normed(), wfc, bias, "gelu_new", wproj2, bd, residual=h8), ops.use_fused_mlp(False))))
    logits8 = torch.randn(8, V, device=dev)
    zeros_i = torch.zeros(8, dtype=torch.int32, device=dev)
    ones_i, temp = torch.ones(8, dtype=torch.int32, device=dev), torch.full((8,), 0.8, device=dev)
    k40 = torch.full((8,), 40, dtype=torch.int32, device=dev)
    out += [
        ("decode: greedy sampling, 8 rows x 50,257", lambda: ops.sample(logits8, temp, ones_i, zeros_i, zeros_i, zeros_i)),
        ("decode: sampling at temperature 0.8, 8 rows x 50,257", lambda: ops.sample(logits8, temp, zeros_i, zeros_i, zeros_i, zeros_i)),
        ("decode: sampling at temperature 0.8 with top-k 40, 8 rows x 50,257", lambda: ops.sample(logits8, temp, k40, zeros_i, zeros_i, zeros_i)),
    ]
    batch, ctx_len = 8, 768
    kc8, vc8, tables8, page_stride8, n_pages8 = paged(batch)
    qkv8 = torch.randn(batch, 3 * D, device=dev).bfloat16()
    rows8 = torch.arange(batch, dtype=torch.int32, device=dev)
    pos8 = torch.full((batch,), ctx_len - 1, dtype=torch.int32, device=dev)
    lens8 = torch.full((batch,), ctx_len, dtype=torch.int32, device=dev)
    slots8 = (tables8[:, (ctx_len - 1) // PS] * PS + (ctx_len - 1) % PS).to(torch.int32)
    out.append(("decode: attention with cache write, 8 rows x 12 heads, context 768",
                lambda: ops.decode_attention_fused(qkv8[:, :D], qkv8[:, D: 2 * D], qkv8[:, 2 * D:], slots8, kc8, vc8, page_stride8, PS,
                                                   n_pages8, tables8, rows8, pos8, lens8, H, H, HD, 0.125, 0, 1024)))
    # decode attention, 64 rows at context 640
    batch, ctx_len = 64, 640
    kc, vc, tables, page_stride, n_pages = paged(batch)
    qkv = torch.randn(batch, 3 * D, device=dev).bfloat16()
    rows = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), ctx_len - 1, dtype=torch.int32, device=dev)
    lens = torch.full((batch,), ctx_len, dtype=torch.int32, device=dev)
    slots = (tables[:, (ctx_len - 1) // PS] * PS + (ctx_len - 1) % PS).to(torch.int32)
    out.append(("decode attention, 64 rows x 12 heads, context 640",
                lambda: ops.decode_attention_fused(qkv[:, :D], qkv[:, D: 2 * D], qkv[:, 2 * D:], slots, kc, vc, page_stride, PS,
                                                   n_pages, tables, rows, pos, lens, H, H, HD, 0.125, 0, 1024)))
    # prefill attention, 2 and 8 prompts of 1,024 tokens: the tcgen05 kernel, then the mma.sync one
    for batch in (2, 8):
        n = 1024
        kc, vc, tables, page_stride, n_pages = paged(batch)
        q = torch.randn(batch * n, D, device=dev).bfloat16()
        row_entry = torch.arange(batch, dtype=torch.int32, device=dev).repeat_interleave(n)
        positions = torch.arange(n, dtype=torch.int32, device=dev).repeat(batch)
        lens = torch.full((batch,), n, dtype=torch.int32, device=dev)
        q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev) * n

        def attention(tc, q=q, kc=kc, vc=vc, page_stride=page_stride, n_pages=n_pages, tables=tables, row_entry=row_entry,
                      positions=positions, lens=lens, q_start=q_start, batch=batch, n=n):
            before = ops.use_prefill_tc(tc)
            ops.paged_attention(q, kc, vc, page_stride, PS, n_pages, tables, row_entry, positions, lens, H, H, HD, 0.125, 0,
                                q_start=q_start, n_tiles=batch * n // 64)
            ops.use_prefill_tc(before)

        out.append((f"prefill attention on tcgen05, {batch} x 1,024 tokens x 12 heads", lambda f=attention: f(True)))
        out.append((f"prefill attention on mma.sync, {batch} x 1,024 tokens x 12 heads", lambda f=attention: f(False)))
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


def main(argv):
    timed = "--time" in argv
    for name, fn in cases():
        if timed:
            print(f"{time_in_graph(fn):8.1f} us  {name}")
        else:
            fn()
            fn()
    torch.cuda.synchronize()
    print("ok", ops.device_errors())


if __name__ == "__main__":
    main(sys.argv[1:])
