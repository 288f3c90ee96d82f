"""Runs each hot kernel once or twice at benchmark shapes (GPT-2 124M), for ncu to capture.

    ncu --set full --clock-control none -k regex:'gemm_tc|decode_kernel|prefill' -c 24 \
        -o kernels python -m research_2_b200.profiling.kernel_cases

Shapes: prefill products at 2,048 tokens (QKV and the MLP's first product with gelu: single-CTA
tiles) and at 8,192 tokens (the same two: persistent CTA pairs), the tied logits product for 8
and 64 rows (77 MB of weights), decode attention for 64 rows at context 640 (126 MB of cache),
prefill attention for 2 x 1,024 and 8 x 1,024 tokens (the tcgen05 kernel `prefill_tc_kernel`, then
the mma.sync kernel `prefill_kernel`).
"""
import torch

from ..kernels import ops

dev = "cuda:0"
torch.manual_seed(0)
D, F, H, HD, V, PS = 768, 3072, 12, 64, 50257, 16


def paged(batch, ctx_len):
    n_pages = batch * (1024 // PS) + 1
    page_stride = 2 * H * PS * HD
    pool = torch.randn(n_pages, page_stride, device=dev).bfloat16()
    flat = pool.view(-1)
    tables = torch.arange(1, n_pages, dtype=torch.int32, device=dev).view(batch, 1024 // PS).contiguous()
    return flat, flat[H * PS * HD:], tables, page_stride, n_pages


def main():
    x = torch.randn(2048, D, device=dev).bfloat16()
    wqkv = (torch.randn(D, 3 * D, device=dev) * 0.02).bfloat16()
    wfc = (torch.randn(D, F, device=dev) * 0.02).bfloat16()
    wte = (torch.randn(V, D, device=dev) * 0.02).bfloat16()
    bias = torch.zeros(F, device=dev)
    x8k = torch.randn(8192, D, device=dev).bfloat16()
    for _ in range(2):
        ops.linear(x, wqkv, bias[: 3 * D].contiguous())
        ops.linear(x, wfc, bias, act="gelu_new")
        ops.linear(x8k, wqkv, bias[: 3 * D].contiguous())
        ops.linear(x8k, wfc, bias, act="gelu_new")
        ops.linear(x[:8].contiguous(), wte, None, w_is_nk=True, out_dtype=torch.float32)
        ops.linear(x[:64].contiguous(), wte, None, w_is_nk=True, out_dtype=torch.float32)
    # decode attention, 64 rows at context 640
    batch, ctx_len = 64, 640
    kc, vc, tables, page_stride, n_pages = paged(batch, ctx_len)
    qkv = torch.randn(batch, 3 * D, device=dev).bfloat16()
    rows = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), ctx_len - 1, dtype=torch.int32, device=dev)
    lens = torch.full((batch,), ctx_len, dtype=torch.int32, device=dev)
    slots = (tables[:, (ctx_len - 1) // PS] * PS + (ctx_len - 1) % PS).to(torch.int32)
    for _ in range(2):
        ops.decode_attention_fused(qkv[:, :D], qkv[:, D: 2 * D], qkv[:, 2 * D:], slots, kc, vc, page_stride, PS, n_pages,
                                   tables, rows, pos, lens, H, H, HD, 0.125, 0, 1024)
    # prefill attention, 2 and 8 prompts of 1,024 tokens: the tcgen05 kernel, then the mma.sync one
    for batch in (2, 8):
        n = 1024
        kc, vc, tables, page_stride, n_pages = paged(batch, n)
        q = torch.randn(batch * n, D, device=dev).bfloat16()
        row_entry = torch.arange(batch, dtype=torch.int32, device=dev).repeat_interleave(n)
        positions = torch.arange(n, dtype=torch.int32, device=dev).repeat(batch)
        lens = torch.full((batch,), n, dtype=torch.int32, device=dev)
        q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev) * n
        for tc in (True, False):
            before = ops.use_prefill_tc(tc)
            for _ in range(2):
                ops.paged_attention(q, kc, vc, page_stride, PS, n_pages, tables, row_entry, positions, lens, H, H, HD, 0.125, 0,
                                    q_start=q_start, n_tiles=batch * n // 64)
            ops.use_prefill_tc(before)
    torch.cuda.synchronize()
    print("ok", ops.device_errors())


if __name__ == "__main__":
    main()
