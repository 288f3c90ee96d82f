"""Each kernel alone against a plain float32 statement of the same op, at sizes other than the
engine's: widths and vocabularies that are no power of two, several head sizes, grouped heads,
a window, mixed batches over a paged cache with garbage in every slot that was never written."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tests.plain import gpt2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from research_2_b200.kernels import ops as o

    return o


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("width", [64, 100, 768, 1600])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_layer_norm(width, out_dtype):
    torch.manual_seed(width)
    x = (torch.randn(37, width) * 3 + 1.5).to(DEV)
    g, b = torch.randn(width).to(DEV), torch.randn(width).to(DEV)
    for eps in (1e-5, 1e-2):
        want = F.layer_norm(x, (width,), g, b, eps)
        got = ops().layer_norm(x, g, b, eps, out_dtype)
        assert got.dtype == out_dtype
        torch.testing.assert_close(got.float(), want, **tol(out_dtype))
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32, device=DEV)
    got = ops().layer_norm(x, g, b, 1e-5, out_dtype, rows=rows)
    torch.testing.assert_close(got.float(), F.layer_norm(x[rows.long()], (width,), g, b, 1e-5), **tol(out_dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_with_and_without_positions(dtype):
    torch.manual_seed(1)
    table = torch.randn(1031, 96).to(dtype).to(DEV)
    pos_table = torch.randn(77, 96).to(dtype).to(DEV)
    ids = torch.randint(0, 1031, (50,), dtype=torch.int32, device=DEV)
    pos = torch.randint(0, 77, (50,), dtype=torch.int32, device=DEV)
    got = ops().embed(ids, table, pos, pos_table)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, table[ids.long()].float() + pos_table[pos.long()].float(), atol=0, rtol=0)
    torch.testing.assert_close(ops().embed(ids, table), table[ids.long()].float(), atol=0, rtol=0)


@pytest.mark.parametrize("m,k,n", [(1, 96, 288), (7, 100, 1031), (64, 768, 2304), (130, 320, 96), (300, 64, 50)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("w_is_nk", [False, True])
def test_linear(m, k, n, dtype, w_is_nk):
    torch.manual_seed(m + k + n)
    a = torch.randn(m, k).to(dtype).to(DEV)
    w = (torch.randn(n, k) if w_is_nk else torch.randn(k, n)).mul(k**-0.5).to(dtype).to(DEV)
    bias = torch.randn(n).to(DEV)
    res = torch.randn(m, n).to(DEV)
    base = a.float() @ (w.float().T if w_is_nk else w.float())
    t = tol(dtype)
    got = ops().linear(a, w, bias, w_is_nk=w_is_nk)
    assert got.dtype == dtype
    torch.testing.assert_close(got.float(), base + bias, **t)
    got = ops().linear(a, w, None, w_is_nk=w_is_nk, out_dtype=torch.float32)
    torch.testing.assert_close(got, base, **(t if dtype == torch.float32 else dict(atol=2e-4, rtol=2e-4)))
    got = ops().linear(a, w, bias, w_is_nk=w_is_nk, act="gelu_new")
    torch.testing.assert_close(got.float(), F.gelu(base + bias, approximate="tanh"), **t)
    got = ops().linear(a, w, bias, w_is_nk=w_is_nk, act="gelu")
    torch.testing.assert_close(got.float(), F.gelu(base + bias), **t)
    got = ops().linear(a, w, bias, w_is_nk=w_is_nk, residual=res)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, base + bias + res, **(t if dtype == torch.float32 else dict(atol=2e-4, rtol=2e-4)))


@pytest.mark.parametrize("m,k,n", [(192, 64, 128), (300, 200, 520), (2048, 768, 2304), (1000, 3072, 768), (257, 96, 1031), (512, 768, 3072), (5000, 136, 1160)])
@pytest.mark.parametrize("w_is_nk", [False, True])
def test_linear_many_rows_on_a_cta_pair(m, k, n, w_is_nk):
    """256-row tiles over two CTAs (tcgen05.mma.cta_group::2), persistent with two accumulators in
    tensor memory (the last shape gives every pair several tiles): same result as the single-CTA
    tiles and as a float32 statement, with every epilogue and ragged edges."""
    o = ops()
    torch.manual_seed(m + k + n)
    a = torch.randn(m, k).bfloat16().to(DEV)
    w = (torch.randn(n, k) if w_is_nk else torch.randn(k, n)).mul(k**-0.5).bfloat16().to(DEV)
    bias = torch.randn(n).to(DEV)
    res = torch.randn(m, n).to(DEV)
    base = a.float() @ (w.float().T if w_is_nk else w.float())

    def run():
        return (o.linear(a, w, bias, w_is_nk=w_is_nk, act="gelu_new"),
                o.linear(a, w, bias, w_is_nk=w_is_nk, residual=res),
                o.linear(a, w, None, w_is_nk=w_is_nk, out_dtype=torch.float32))

    before = o.use_pair_gemm("always")
    try:
        pair = run()
        o.use_pair_gemm(False)
        single = run()
    finally:
        o.use_pair_gemm(before)
    assert o.device_errors() == 0
    for x, y in zip(pair, single):
        torch.testing.assert_close(x.float(), y.float(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(pair[0].float(), F.gelu(base + bias, approximate="tanh"), **tol(torch.bfloat16))
    torch.testing.assert_close(pair[1], base + bias + res, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(pair[2], base, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("m,heads,kv_heads,hd,page", [(200, 4, 4, 64, 16), (65, 6, 2, 32, 8), (700, 5, 1, 48, 4), (2048, 12, 12, 64, 16)])
@pytest.mark.parametrize("pair", [False, "always"])
def test_linear_writes_keys_and_values_into_the_cache(m, heads, kv_heads, hd, page, pair):
    """The fused q/k/v product of more than 64 rows sends its key and value columns straight to
    the rows' cache slots: the cache then holds what the separate write kernel would have put
    there from the whole product, the query columns are the product's, other slots are untouched."""
    o = ops()
    torch.manual_seed(m + hd)
    k_in = 96
    qw, kvw = heads * hd, kv_heads * hd
    a = torch.randn(m, k_in).bfloat16().to(DEV)
    w = (torch.randn(k_in, qw + 2 * kvw) * k_in**-0.5).bfloat16().to(DEV)
    bias = torch.randn(qw + 2 * kvw).to(DEV)
    n_pages = -(-m // page) + 3
    stride = 2 * kv_heads * page * hd
    slots = (torch.randperm((n_pages - 1) * page)[:m] + page).to(torch.int32).to(DEV)  # never the null page
    pool_a = torch.full((n_pages, stride), 7.0).bfloat16().to(DEV)
    pool_b = pool_a.clone()
    before = o.use_pair_gemm(pair)
    try:
        whole = o.linear(a, w, bias)
        ka, va = pool_a.view(-1), pool_a.view(-1)[kv_heads * page * hd:]
        o.kv_write(whole[:, qw: qw + kvw], whole[:, qw + kvw:], ka, va, slots, kv_heads, hd, page, stride, n_pages)
        kb, vb = pool_b.view(-1), pool_b.view(-1)[kv_heads * page * hd:]
        got, written = o.linear(a, w, bias, kv=o.kv_scatter(slots, kb, vb, stride, page, n_pages, qw, kvw, hd))
    finally:
        o.use_pair_gemm(before)
    assert written and o.device_errors() == 0
    assert torch.equal(got[:, :qw], whole[:, :qw])
    assert torch.equal(pool_b, pool_a)
    few, written = o.linear(a[:40].contiguous(), w, bias, kv=o.kv_scatter(slots, kb, vb, stride, page, n_pages, qw, kvw, hd))
    assert not written and torch.equal(few, o.linear(a[:40].contiguous(), w, bias))


@pytest.mark.parametrize("m,k,n", [(1, 768, 2304), (8, 768, 3072), (64, 768, 2304), (5, 96, 288), (33, 1600, 4800), (17, 320, 96)])
@pytest.mark.parametrize("w_is_nk", [False, True])
def test_linear_with_the_norm_inside(m, k, n, w_is_nk):
    """LayerNorm of a few float32 rows computed inside the tensor-core product's kernel: same
    result as the LayerNorm kernel followed by the product, and as a plain float32 statement."""
    o = ops()
    torch.manual_seed(m + k)
    x = (torch.randn(m + 3, k) * 2 + 0.5).to(DEV)
    g, b = (1 + 0.1 * torch.randn(k)).to(DEV), (0.1 * torch.randn(k)).to(DEV)
    w = ((torch.randn(n, k) if w_is_nk else torch.randn(k, n)) * k**-0.5).bfloat16().to(DEV)
    bias = torch.randn(n).to(DEV)
    rows = torch.randperm(m + 3)[:m].to(torch.int32).to(DEV)
    for pick in (None, rows):
        lazy = o.NormedRows(x, g, b, 1e-5, torch.bfloat16, rows=pick)
        before = o.use_fused_norm(True)
        try:
            fused = o.linear(lazy, w, bias, w_is_nk=w_is_nk, act="gelu_new", out_dtype=torch.float32)
            o.use_fused_norm(False)
            apart = o.linear(lazy, w, bias, w_is_nk=w_is_nk, act="gelu_new", out_dtype=torch.float32)
        finally:
            o.use_fused_norm(before)
        src = x if pick is None else x[pick.long()]
        h = F.layer_norm(src, (k,), g, b, 1e-5).bfloat16().float()
        want = F.gelu(h @ (w.float().T if w_is_nk else w.float()) + bias, approximate="tanh")
        torch.testing.assert_close(fused, want, atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(fused, apart, atol=2e-2, rtol=2e-2)
    assert o.device_errors() == 0


def test_linear_rows_do_not_depend_on_the_batch():
    """In float32 a row's result is the same bits alone and among other rows."""
    torch.manual_seed(0)
    a = torch.randn(200, 333, device=DEV)
    w = torch.randn(333, 257, device=DEV)
    whole = ops().linear(a, w)
    for rows in (slice(0, 1), slice(5, 70), slice(199, 200)):
        assert torch.equal(ops().linear(a[rows].contiguous(), w), whole[rows])


def test_linear_refuses_what_it_cannot_do():
    o = ops()
    a = torch.randn(4, 8, device=DEV)
    with pytest.raises(o.KernelError, match="does not fit"):
        o.linear(a, torch.randn(9, 4, device=DEV))
    with pytest.raises(o.KernelError, match="must be torch.float32, got torch.bfloat16"):
        o.linear(a, torch.randn(8, 4, device=DEV).bfloat16())
    with pytest.raises(o.KernelError, match="unknown activation"):
        o.linear(a, torch.randn(8, 4, device=DEV), act="relu")
    with pytest.raises(o.KernelError, match="CUDA tensor"):
        o.linear(torch.randn(4, 8), torch.randn(8, 4))


class PagedCase:
    """Entries over a paged cache with shuffled pages; dense K and V per entry kept for the
    plain statement. Slots never written hold `garbage`."""

    def __init__(self, entries, n_heads, n_kv, hd, page, dtype, seed=0, garbage=64.0, mutate=None):
        g = torch.Generator().manual_seed(seed)
        self.entries, self.n_heads, self.n_kv, self.hd, self.page, self.dtype = entries, n_heads, n_kv, hd, page, dtype
        ctx = [start + rows for start, rows in entries]
        width = max(-(-c // page) for c in ctx)
        n_pages = sum(-(-c // page) for c in ctx) + 1
        order = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
        self.k_dense = [torch.randn(c, n_kv, hd, generator=g).to(dtype) for c in ctx]
        self.v_dense = [torch.randn(c, n_kv, hd, generator=g).to(dtype) for c in ctx]
        self.q = [torch.randn(rows, n_heads, hd, generator=g).to(dtype) for _, rows in entries]
        if mutate is not None:
            mutate(self)
        self.page_stride = 2 * n_kv * page * hd
        pool = torch.full((n_pages, self.page_stride), garbage).to(dtype)
        tables = torch.zeros(len(entries), width, dtype=torch.int32)
        slots, row_entry, positions = [], [], []
        for e, (start, rows) in enumerate(entries):
            for i in range(-(-ctx[e] // page)):
                tables[e, i] = order.pop()
            for pos in range(ctx[e]):
                p, off = int(tables[e, pos // page]), pos % page
                if pos < start:  # history: already in the cache
                    kv = pool[p].view(2, n_kv, page, hd)
                    kv[0, :, off], kv[1, :, off] = self.k_dense[e][pos], self.v_dense[e][pos]
                else:
                    slots.append(p * page + off)
                    row_entry.append(e)
                    positions.append(pos)
        self.pool = pool.to(DEV)
        flat = self.pool.view(-1)
        self.k_cache, self.v_cache = flat, flat[n_kv * page * hd:]
        self.n_pages = n_pages
        self.tables = tables.to(DEV)
        self.slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.row_entry = torch.tensor(row_entry, dtype=torch.int32, device=DEV)
        self.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
        self.seq_lens = torch.tensor(ctx, dtype=torch.int32, device=DEV)
        starts = [0]
        for _, rows in entries:
            starts.append(starts[-1] + rows)
        self.q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        self.n_tiles = sum(-(-rows // 64) for _, rows in entries)
        self.q_rows = torch.cat([q.reshape(q.shape[0], -1) for q in self.q]).to(DEV)
        self.k_new = torch.cat([self.k_dense[e][s:].reshape(r, -1) for e, (s, r) in enumerate(entries)]).to(DEV)
        self.v_new = torch.cat([self.v_dense[e][s:].reshape(r, -1) for e, (s, r) in enumerate(entries)]).to(DEV)

    def run(self, scale, window=0, **kernel_choice):
        o = ops()
        o.kv_write(self.k_new, self.v_new, self.k_cache, self.v_cache, self.slots, self.n_kv, self.hd, self.page,
                   self.page_stride, self.n_pages)
        return o.paged_attention(self.q_rows, self.k_cache, self.v_cache, self.page_stride, self.page, self.n_pages,
                                 self.tables, self.row_entry, self.positions, self.seq_lens, self.n_heads, self.n_kv,
                                 self.hd, scale, window, **kernel_choice)

    def run_fused(self, scale, window=0, max_context=4096):
        """The one-launch decode attention (every entry one row): cache write and slice merge inside."""
        o = ops()
        out = o.decode_attention_fused(self.q_rows, self.k_new, self.v_new, self.slots, self.k_cache, self.v_cache, self.page_stride,
                                       self.page, self.n_pages, self.tables, self.row_entry, self.positions, self.seq_lens,
                                       self.n_heads, self.n_kv, self.hd, scale, window, max_context)
        assert out is not None, "the fused decode attention did not take the case"
        return out

    def plain(self, scale, window=0):
        outs = []
        for e, (start, rows) in enumerate(self.entries):
            ctx = start + rows
            qfull = torch.zeros(ctx, self.n_heads, self.hd, dtype=torch.float64)
            qfull[start:] = self.q[e].double()
            out = plain.causal_attention(qfull, self.k_dense[e].double(), self.v_dense[e].double(), scale, window)
            outs.append(out[start:])
        return torch.cat(outs).float()


CASES = [
    # (entries (start, rows), heads, kv heads, head size, page size)
    ([(0, 40)], 4, 4, 16, 16),
    ([(0, 1), (37, 1), (5, 2), (0, 33), (60, 9)], 6, 2, 32, 8),
    ([(100, 1), (17, 30), (0, 3)], 3, 3, 64, 16),
    ([(250, 6), (0, 70)], 5, 1, 48, 4),
    ([(30, 20), (299, 1)], 2, 2, 128, 32),
    ([(10, 5)], 2, 1, 256, 16),
]


@pytest.mark.parametrize("case", CASES, ids=[f"hd{c[3]}_h{c[1]}kv{c[2]}_p{c[4]}" for c in CASES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 13])
def test_paged_attention(case, dtype, window):
    entries, h, hkv, hd, page = case
    pc = PagedCase(entries, h, hkv, hd, page, dtype, seed=hd + page)
    scale = hd**-0.5 / 1.5
    got = pc.run(scale, window).float().cpu()
    want = pc.plain(scale, window)
    assert torch.isfinite(got).all(), "garbage from a slot that was never written leaked in"
    torch.testing.assert_close(got, want, **(dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)))


PREFILL_CASES = CASES + [
    ([(0, 200), (100, 130), (511, 1), (0, 64), (64, 65)], 4, 4, 64, 16),
    ([(3, 129), (0, 2)], 6, 2, 32, 8),
    ([(40, 100)], 2, 1, 96, 16),
    ([(0, 70), (70, 70)], 2, 2, 112, 4),
]


@pytest.mark.parametrize("case", PREFILL_CASES, ids=[f"hd{c[3]}_h{c[1]}kv{c[2]}_p{c[4]}_{len(c[0])}e" for c in PREFILL_CASES])
@pytest.mark.parametrize("window", [0, 13, 70])
def test_prefill_attention(case, window):
    """The tensor-core prefill kernel on mixed batches (head sizes up to 128; larger ones fall
    back to the general kernel inside the same call)."""
    entries, h, hkv, hd, page = case
    pc = PagedCase(entries, h, hkv, hd, page, torch.bfloat16, seed=hd + page + window)
    scale = hd**-0.5 / 1.5
    got = pc.run(scale, window, q_start=pc.q_start, n_tiles=pc.n_tiles).float().cpu()
    want = pc.plain(scale, window)
    assert torch.isfinite(got).all(), "garbage from a slot that was never written leaked in"
    torch.testing.assert_close(got, want, atol=3e-2, rtol=3e-2)


DECODE_CASES = [
    # (contexts before the new token, heads, kv heads, head size, page size)
    ([0, 1, 31, 32, 33, 500], 4, 4, 64, 16),
    ([700, 5], 8, 1, 32, 8),
    ([129, 64, 1000, 3], 6, 3, 16, 4),
    ([260], 4, 2, 128, 32),
    ([90, 91], 2, 2, 48, 16),
    ([300, 17], 8, 2, 80, 8),
]


@pytest.mark.parametrize("case", DECODE_CASES, ids=[f"hd{c[3]}_h{c[1]}kv{c[2]}_p{c[4]}" for c in DECODE_CASES])
@pytest.mark.parametrize("window", [0, 40])
def test_decode_attention_tile_arithmetic_on_tensor_cores_and_scalar(case, window):
    """A tile's scores and outputs by mma.sync (head sizes up to 128) against the scalar float
    form of the same kernel: both within the bfloat16 budget of the plain statement, and close
    to each other (the tensor-core form rounds p to bfloat16 before p.v, as prefill does)."""
    contexts, h, hkv, hd, page = case
    o = ops()
    pc = PagedCase([(c, 1) for c in contexts], h, hkv, hd, page, torch.bfloat16, seed=hd + page + window, garbage=float("inf"))
    scale = hd**-0.5 / 1.5
    before = o.use_decode_mma(True, hd)
    try:
        by_mma = pc.run(scale, window, decode_only=True, max_context=4096).float().cpu()
        o.use_decode_mma(False, hd)
        by_scalar = pc.run(scale, window, decode_only=True, max_context=4096).float().cpu()
    finally:
        o.use_decode_mma(before, hd)
    want = pc.plain(scale, window)
    assert torch.isfinite(by_mma).all()
    torch.testing.assert_close(by_mma, want, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(by_scalar, want, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(by_mma, by_scalar, atol=2e-2, rtol=2e-2)


TMA_CASES = [
    ([(0, 200), (100, 130), (511, 1), (0, 64), (64, 65)], 4, 2, 64, 8),
    ([(3, 129), (0, 2), (300, 77)], 6, 6, 64, 32),
    ([(40, 100), (0, 333)], 2, 1, 64, 64),
    ([(0, 70), (190, 70)], 3, 3, 64, 128),
]


@pytest.mark.parametrize("case", TMA_CASES, ids=[f"p{c[4]}_h{c[1]}kv{c[2]}_{len(c[0])}e" for c in TMA_CASES])
@pytest.mark.parametrize("window", [0, 13, 70])
def test_prefill_attention_tiles_by_tensor_copies(case, window):
    """Head size 64 with pages of 8, 16, 32 or a multiple of 64 keys brings its tiles in by 4-D
    tensor copies into swizzled rows: the same numbers as the piecewise copies (to rounding of the
    same arithmetic: bit-equal), and as the plain statement; slots never written do not leak."""
    entries, h, hkv, hd, page = case
    o = ops()
    pc = PagedCase(entries, h, hkv, hd, page, torch.bfloat16, seed=page + window, garbage=float("inf"))
    scale = hd**-0.5 / 1.5
    before, before_tc = o.use_prefill_tma(True), o.use_prefill_tc(False)
    try:
        by_tma = pc.run(scale, window, q_start=pc.q_start, n_tiles=pc.n_tiles)
        o.use_prefill_tma(False)
        by_pieces = pc.run(scale, window, q_start=pc.q_start, n_tiles=pc.n_tiles)
    finally:
        o.use_prefill_tma(before)
        o.use_prefill_tc(before_tc)
    assert o.device_errors() == 0
    assert torch.isfinite(by_tma.float()).all(), "a slot that was never written leaked in"
    assert torch.equal(by_tma, by_pieces)
    torch.testing.assert_close(by_tma.float().cpu(), pc.plain(scale, window), atol=3e-2, rtol=3e-2)


TC_CASES = TMA_CASES + [
    ([(0, 1024), (0, 1024)], 12, 12, 64, 16),
    ([(900, 1), (17, 30), (0, 3), (500, 129)], 3, 3, 64, 16),
    ([(0, 128), (0, 127), (1, 129)], 2, 2, 64, 16),
]


@pytest.mark.parametrize("case", TC_CASES, ids=[f"p{c[4]}_h{c[1]}kv{c[2]}_{len(c[0])}e" for c in TC_CASES])
@pytest.mark.parametrize("window", [0, 13, 70])
def test_prefill_attention_on_tcgen05(case, window):
    """Head size 64 on the 5th-generation tensor cores (128-row tiles, scores and outputs in
    tensor memory, P handed to the second product through tensor memory, one softmax thread per row):
    the plain statement within the bfloat16 budget,
    close to the mma.sync kernel, nothing from slots that were never written."""
    entries, h, hkv, hd, page = case
    o = ops()
    pc = PagedCase(entries, h, hkv, hd, page, torch.bfloat16, seed=page + window + 5, garbage=float("inf"))
    scale = hd**-0.5 / 1.5
    before = o.use_prefill_tc("always")
    try:
        by_tc = pc.run(scale, window, q_start=pc.q_start, n_tiles=pc.n_tiles)
        o.use_prefill_tc(False)
        by_mma = pc.run(scale, window, q_start=pc.q_start, n_tiles=pc.n_tiles)
    finally:
        o.use_prefill_tc(before)
    assert o.device_errors() == 0
    assert torch.isfinite(by_tc.float()).all(), "a slot that was never written leaked in"
    torch.testing.assert_close(by_tc.float().cpu(), pc.plain(scale, window), atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(by_tc.float(), by_mma.float(), atol=2e-2, rtol=2e-2)


def test_prefill_attention_on_tcgen05_with_every_sm_shared_by_two_ctas():
    """Eight prompts of 1,024 tokens and twelve heads: several CTAs for every SM, two of them
    resident at a time, softmax warps of one CTA a tile apart (rows below the diagonal skip the
    mask). What depends on the order in which warps and products finish shows here and not in
    small cases, so the same launch runs several times and every row is compared."""
    o = ops()
    entries = [(0, 1024)] * 8
    pc = PagedCase(entries, 12, 12, 64, 16, torch.bfloat16, seed=77, garbage=float("inf"))
    scale = 0.125
    before = o.use_prefill_tc(False)
    try:
        by_mma = pc.run(scale, 0, q_start=pc.q_start, n_tiles=pc.n_tiles).float()
        o.use_prefill_tc("always")
        for _ in range(5):
            by_tc = pc.run(scale, 0, q_start=pc.q_start, n_tiles=pc.n_tiles).float()
            assert torch.isfinite(by_tc).all()
            worst = (by_tc - by_mma).abs().amax(dim=1)
            assert worst.max().item() < 2e-2, f"rows {(worst >= 2e-2).nonzero().flatten()[:8].tolist()} differ"
    finally:
        o.use_prefill_tc(before)
    assert o.device_errors() == 0


@pytest.mark.parametrize("case", DECODE_CASES, ids=[f"hd{c[3]}_h{c[1]}kv{c[2]}_p{c[4]}" for c in DECODE_CASES])
@pytest.mark.parametrize("window", [0, 40])
@pytest.mark.parametrize("sliced", [False, True])
def test_decode_attention(case, window, sliced):
    """The decode kernel (one new token per entry), with one slice of the keys and with several."""
    contexts, h, hkv, hd, page = case
    pc = PagedCase([(c, 1) for c in contexts], h, hkv, hd, page, torch.bfloat16, seed=hd + page + window)
    scale = hd**-0.5
    got = pc.run(scale, window, decode_only=True, max_context=4096 if sliced else 64).float().cpu()
    want = pc.plain(scale, window)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, atol=3e-2, rtol=3e-2)
    general = pc.run(scale, window).float().cpu()
    torch.testing.assert_close(got, general, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("case", DECODE_CASES, ids=[f"hd{c[3]}_h{c[1]}kv{c[2]}_p{c[4]}" for c in DECODE_CASES])
@pytest.mark.parametrize("window", [0, 40])
@pytest.mark.parametrize("max_context", [64, 300, 4096])
def test_decode_attention_in_one_launch(case, window, max_context):
    """The fused form: the kernel writes the new keys and values itself and merges 1, 2, 4 or 8
    slices inside a cluster. The cache must afterwards hold the new token."""
    contexts, h, hkv, hd, page = case
    pc = PagedCase([(c, 1) for c in contexts], h, hkv, hd, page, torch.bfloat16, seed=hd + page + window + 1)
    scale = hd**-0.5
    o = ops()
    got = o.decode_attention_fused(pc.q_rows, pc.k_new, pc.v_new, pc.slots, pc.k_cache, pc.v_cache, pc.page_stride,
                                   pc.page, pc.n_pages, pc.tables, pc.row_entry, pc.positions, pc.seq_lens, h, hkv, hd,
                                   scale, window, max_context)
    assert got is not None
    torch.testing.assert_close(got.float().cpu(), pc.plain(scale, window), atol=3e-2, rtol=3e-2)
    # the cache now holds the new keys and values: the general kernel reads them back
    again = o.paged_attention(pc.q_rows, pc.k_cache, pc.v_cache, pc.page_stride, pc.page, pc.n_pages, pc.tables,
                              pc.row_entry, pc.positions, pc.seq_lens, h, hkv, hd, scale, window)
    torch.testing.assert_close(again.float(), got.float(), atol=2e-2, rtol=2e-2)


def test_decode_slices_choice():
    o = ops()
    assert o.decode_slices(64, 12, 1024) == 1
    assert o.decode_slices(8, 12, 1024) == 6    # 576 CTAs: one wave of four to an SM
    assert o.decode_slices(16, 12, 1024) == 3
    assert o.decode_slices(1, 12, 1024) == 8
    assert o.decode_slices(1, 12, 100) == 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """One query and one far key are scaled so that this key's score stands out: the output must
    be (nearly) that key's value. A kernel that drops a page or a tile's edge shows here."""
    for far in (0, 15, 16, 255, 256, 300, 511):
        direction = torch.randn(64, generator=torch.Generator().manual_seed(far))
        direction /= direction.norm()

        def mutate(case, far=far, direction=direction):
            case.q[0][0, :] = (direction * 30).to(dtype)
            case.k_dense[0][far, :] = (direction * 30).to(dtype)

        case = PagedCase([(511, 1)], 2, 2, 64, 16, dtype, seed=far, mutate=mutate)
        want = case.v_dense[0][far].float()
        choices = [{}] if dtype == torch.float32 else [{}, dict(decode_only=True, max_context=64), dict(decode_only=True, max_context=4096),
                                                       dict(q_start=case.q_start, n_tiles=case.n_tiles)]
        for choice in choices:
            got = case.run(1.0, **choice).float().cpu().view(2, 64)
            assert torch.allclose(got, want, atol=5e-2), f"far key {far} {choice}: max diff {(got - want).abs().max():.3f}"


@pytest.mark.parametrize("entries,window", [([(0, 1024)], 0), ([(300, 700)], 0), ([(0, 1024)], 200), ([(77, 500), (0, 130)], 0)])
def test_prefill_attention_in_clusters_of_two_finds_every_row_its_key(entries, window):
    """With fewer CTAs than SMs the tcgen05 prefill kernel runs as clusters of two CTAs that take every other
    64-key tile of the same 128 rows and are joined at the end. Every query row is pointed at one key of its own
    (anywhere it may see: first tile, last tile, tiles of the first CTA and of the second, the tile before the
    window's edge), so that its output must be that key's value: a tile that is dropped, taken twice or joined
    with the wrong weight shows in the rows whose key lies there. Unwritten slots hold inf."""
    heads, hd, page = 2, 64, 16
    targets = []

    def mutate(case):
        g = torch.Generator().manual_seed(len(entries) + window)
        for e, (start, rows) in enumerate(entries):
            ctx = start + rows
            directions = torch.randn(ctx, hd, generator=g)
            directions /= directions.norm(dim=1, keepdim=True)
            case.k_dense[e][:, :, :] = (directions * 6).to(torch.bfloat16)[:, None, :]
            tgt = torch.empty(rows, dtype=torch.long)
            for r in range(rows):
                pos = start + r
                lo = max(0, pos - window + 1) if window else 0
                choice = r % 5   # the newest key, the oldest it may see, and three random ones
                tgt[r] = pos if choice == 0 else lo if choice == 1 else int(torch.randint(lo, pos + 1, (1,), generator=g))
            case.q[e][:, :, :] = (directions[tgt] * 6).to(torch.bfloat16)[:, None, :]
            targets.append(tgt)

    case = PagedCase(entries, heads, heads, hd, page, torch.bfloat16, seed=window + 3, garbage=float("inf"), mutate=mutate)
    o = ops()
    before = dict(o.kernel_uses())
    got = case.run(1.0, window, q_start=case.q_start, n_tiles=case.n_tiles).float().cpu()
    used = {k: v - before.get(k, 0) for k, v in o.kernel_uses().items() if v != before.get(k, 0)}
    assert any("prefill_tc" in k for k in used), f"the tcgen05 prefill kernel did not run: {used}"
    at = 0
    for e, (start, rows) in enumerate(entries):
        want = case.v_dense[e][targets[e]].float().reshape(rows, -1)     # scores: 36 at the key, about 36 * N(0, 1/8) elsewhere
        block = got[at: at + rows]
        bad = ((block - want).abs() > 0.06).any(dim=1).nonzero().flatten().tolist()
        assert not bad, f"entry {e}: rows {bad[:8]} (keys {targets[e][bad[:8]].tolist()}) did not get their key's value"
        at += rows
    torch.testing.assert_close(got, case.plain(1.0, window), atol=3e-2, rtol=3e-2)
    assert o.device_errors() == 0


def test_window_edge():
    """With a window the key just outside must not count and the one just inside must."""
    dtype = torch.float32
    for window, pos in ((8, 40), (16, 16), (17, 33)):
        inside, outside = pos - window + 1, pos - window
        for far, visible in ((inside, True), (outside, False)):
            if far < 0:
                continue
            d = torch.ones(16) / 4.0

            def mutate(case, far=far, d=d):
                case.q[0][0, 0] = d * 40
                case.k_dense[0][far, 0] = d * 40

            case = PagedCase([(pos, 1)], 1, 1, 16, 8, dtype, seed=window, mutate=mutate)
            got = case.run(1.0, window).cpu().view(16)
            hit = torch.allclose(got, case.v_dense[0][far, 0], atol=1e-3)
            assert hit == visible, f"window {window}, query {pos}, key {far}: visible={visible}, hit={hit}"


def _planted(entries, row, far, hd, page, seed):
    """A case whose query row `row` (of entry 0) and key `far` point the same way, thirty long."""
    direction = torch.randn(hd, generator=torch.Generator().manual_seed(seed))
    direction /= direction.norm()

    def mutate(case):
        case.q[0][row, :] = (direction * 30).to(torch.bfloat16)
        case.k_dense[0][far, :] = (direction * 30).to(torch.bfloat16)

    return PagedCase(entries, 1, 1, hd, page, torch.bfloat16, seed=seed, garbage=float("inf"), mutate=mutate)


@pytest.mark.parametrize("hd,page", [(64, 16), (32, 8), (128, 32)])
def test_window_edge_in_the_bfloat16_decode_kernels(hd, page):
    """The key just inside the window counts and the one just outside does not, in every form of
    the bfloat16 decode attention: one slice and several, tensor-core and scalar tiles, with the
    cache write and merge inside the kernel and without. Windows that end on a page's edge, a
    32-key tile's edge and in between; unwritten slots hold inf."""
    o = ops()
    for window, pos in ((8, 40), (16, 16), (17, 33), (33, 300), (64, 511), (129, 400)):
        for far, visible in ((pos - window + 1, True), (pos - window, False)):
            if far < 0:
                continue
            for mma in (True, False):
                before = o.use_decode_mma(mma, hd)
                try:
                    runs = {}
                    for name, max_context in (("one slice", 64), ("slices", 4096)):
                        case = _planted([(pos, 1)], 0, far, hd, page, seed=window + pos)
                        runs[name] = case.run(1.0, window, decode_only=True, max_context=max_context)
                        case = _planted([(pos, 1)], 0, far, hd, page, seed=window + pos)
                        runs[name + ", fused"] = case.run_fused(1.0, window, max_context=max_context)
                finally:
                    o.use_decode_mma(before, hd)
                want = case.v_dense[0][far, 0].float()
                for name, got in runs.items():
                    got = got.float().cpu().view(hd)
                    assert torch.isfinite(got).all(), f"{name}: an unwritten slot leaked in"
                    hit = torch.allclose(got, want, atol=5e-2)
                    assert hit == visible, f"{name} (mma={mma}): window {window}, query {pos}, key {far}: visible={visible}, hit={hit}"


@pytest.mark.parametrize("tc", [False, "always"])
def test_window_edge_in_the_bfloat16_prefill_kernels(tc):
    """The same for prompt portions in both prefill kernels (mma.sync with 64-row tiles, tcgen05 with
    128-row tiles): the query row is the portion's first row, the first row of a later tile, the last
    row of a tile and the portion's last row; windows that end on a page's edge and a key tile's."""
    o = ops()
    start, rows, hd, page = 40, 200, 64, 16
    before = o.use_prefill_tc(tc)
    uses = o.kernel_uses()
    try:
        for window in (24, 41, 64, 65, 130):
            for row in (0, 63, 64, 127, 128, 199):
                pos = start + row
                for far, visible in ((pos - window + 1, True), (pos - window, False)):
                    if far < 0:
                        continue
                    case = _planted([(start, rows)], row, far, hd, page, seed=window + row)
                    got = case.run(1.0, window, q_start=case.q_start, n_tiles=case.n_tiles).float().cpu()
                    assert torch.isfinite(got).all(), "an unwritten slot leaked in"
                    hit = torch.allclose(got[row], case.v_dense[0][far, 0].float(), atol=5e-2)
                    assert hit == visible, f"tc={tc}: window {window}, row {row} at {pos}, key {far}: visible={visible}, hit={hit}"
                    # the rows around it see what the plain statement says they see
                    torch.testing.assert_close(got, case.plain(1.0, window), atol=6e-2, rtol=6e-2)
    finally:
        o.use_prefill_tc(before)
    name = "attention_prefill_tc" if tc else "attention_prefill"
    assert o.kernel_uses().get(name, 0) > uses.get(name, 0), f"{name} never ran"
    assert o.device_errors() == 0


def test_pad_rows_are_zero():
    pc = PagedCase([(3, 2)], 2, 2, 16, 4, torch.float32)
    pc.row_entry[1] = -1
    out = pc.run(0.25)
    assert torch.count_nonzero(out[1]) == 0 and torch.count_nonzero(out[0]) > 0


def test_prefill_attention_on_tcgen05_takes_whole_prompts_and_mostly_empty_tiles():
    """Whole prompts go to the tcgen05 kernel (128-row tiles, one entry to a tile), and so does a
    batch of single decoded tokens beside one portion, whose tiles are mostly rows past their
    entry's last (those take the last row's mask and are never stored). Both give the plain
    statement's numbers."""
    o = ops()
    scale = 0.125
    for entries in ([(0, 300), (40, 200)], [(200 + i, 1) for i in range(24)] + [(0, 150)]):
        pc = PagedCase(entries, 3, 3, 64, 16, torch.bfloat16, seed=len(entries), garbage=float("inf"))
        before, uses = o.use_prefill_tc(True), o.kernel_uses()
        try:
            got = pc.run(scale, 0, q_start=pc.q_start, n_tiles=pc.n_tiles)
        finally:
            o.use_prefill_tc(before)
        after = o.kernel_uses()
        assert after.get("attention_prefill_tc", 0) == uses.get("attention_prefill_tc", 0) + 1, (uses, after)
        torch.testing.assert_close(got.float().cpu(), pc.plain(scale, 0), atol=3e-2, rtol=3e-2)
    assert o.device_errors() == 0


def test_sampling_greedy_first_index_on_ties():
    logits = torch.full((3, 50257), -1.0)
    logits[0, [7, 300, 50000]] = 5.0
    logits[1, 50256] = 9.0
    logits[2, 0] = 0.5
    n = 3
    tokens = ops().sample(logits.to(DEV), torch.ones(n, device=DEV), torch.ones(n, dtype=torch.int32, device=DEV),
                          torch.zeros(n, dtype=torch.int32, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                          torch.zeros(n, dtype=torch.int32, device=DEV))
    assert tokens.tolist() == [7, 50256, 0]


@pytest.mark.parametrize("vocab", [512, 1031])
def test_sampling_draws_equal_the_plain_sampler(vocab):
    torch.manual_seed(vocab)
    n = 24
    logits = torch.randn(n, vocab) * 2
    temps = torch.tensor([0.8, 1.0, 1.7, 0.3] * 6)
    top_ks = torch.tensor([0, 5, 40, 1, vocab, 2] * 4, dtype=torch.int32)
    key0 = torch.arange(n, dtype=torch.int64) * 7919 % (2**31)
    key1 = torch.arange(n, dtype=torch.int64) + 11
    pos = torch.arange(n, dtype=torch.int32) * 3 + 1
    got = ops().sample(logits.to(DEV), temps.to(DEV), top_ks.to(DEV), key0.to(torch.int32).to(DEV),
                       key1.to(torch.int32).to(DEV), pos.to(DEV)).tolist()
    want = [plain.sample_token(logits[i], float(temps[i]), int(top_ks[i]), (int(key0[i]), int(key1[i])), int(pos[i]))
            for i in range(n)]
    assert got == want


@pytest.mark.parametrize("vocab", [20011, 60013])
def test_sampling_rows_split_over_several_ctas(vocab):
    """A large vocabulary is cut into slices, one CTA each; the draw does not show the cut (ties
    go to the lower token across slices too), and a second launch finds the counters reset. The
    smaller row fits a CTA's shared memory for the top-k selection, the larger does not."""
    n = 8
    torch.manual_seed(5)
    logits = torch.randn(n, vocab) * 2
    logits[0, [4100, 19000]] = 30.0          # a tie across two slices, greedy
    temps = torch.tensor([1.0, 0.8, 1.0, 1.7, 0.3, 1.0, 0.9, 1.0])
    top_ks = torch.tensor([1, 0, 5, 40, vocab, 1, 2, 0], dtype=torch.int32)
    key0 = torch.arange(n, dtype=torch.int64) * 104729 % (2**31)
    key1 = torch.arange(n, dtype=torch.int64) + 3
    pos = torch.arange(n, dtype=torch.int32) * 5 + 2
    want = [plain.sample_token(logits[i], float(temps[i]), int(top_ks[i]), (int(key0[i]), int(key1[i])), int(pos[i]))
            for i in range(n)]
    assert want[0] == 4100
    for _ in range(2):
        got = ops().sample(logits.to(DEV), temps.to(DEV), top_ks.to(DEV), key0.to(torch.int32).to(DEV),
                           key1.to(torch.int32).to(DEV), pos.to(DEV)).tolist()
        assert got == want


def test_top_k_where_the_k_th_value_is_hard_to_find():
    """Rows made so that the k-th largest value is tied, lies among thousands of equal values (more than
    the kernel lists in shared memory: it falls back to its selection over the row), sits beside a
    neighbour one float away, is a zero of either sign, or is -inf; 64 rows of GPT-2's vocabulary so that
    rows are cut into slices and more CTAs than SMs run. Draws equal the plain sampler's, twice (the
    counters and bins are left clean)."""
    vocab, n = 50257, 64
    g = torch.Generator().manual_seed(12)
    logits = torch.randn(n, vocab, generator=g) * 2
    top_ks = torch.tensor([40, 5, 2, 300] * (n // 4), dtype=torch.int32)
    logits[1, [7, 30000, 50256, 123, 45000, 9]] = 9.5                      # six tied at the top, k = 5: all six are kept
    logits[2] = 1.25                                                      # every value equal, k = 2
    logits[3, :6000] = 3.0                                                # the k-th lies among 6,000 equal values
    logits[4, 100] = 8.0
    logits[4, 200:240] = torch.nextafter(torch.tensor(8.0), torch.tensor(0.0))   # one float below
    logits[5] = -torch.rand(vocab, generator=g) - 1.0                     # k = 5 among negatives, with zeros of both signs on top
    logits[5, [3, 4]] = 0.0
    logits[5, [10, 11, 12]] = -0.0
    logits[6, 50:] = float("-inf")                                        # fewer finite values than k = 2 ... no: 50 finite, k = 2
    logits[7, 300:] = float("-inf")                                       # exactly k = 300 finite values
    logits[11, 200:] = float("-inf")                                      # fewer finite values (200) than k = 300
    temps = torch.tensor([0.8, 1.0, 1.7, 0.3] * (n // 4))
    key0 = torch.arange(n, dtype=torch.int64) * 104729 % (2**31)
    key1 = torch.arange(n, dtype=torch.int64) + 5
    pos = torch.arange(n, dtype=torch.int32) * 7 + 3
    want = [plain.sample_token(logits[i], float(temps[i]), int(top_ks[i]), (int(key0[i]), int(key1[i])), int(pos[i]))
            for i in range(n)]
    for _ in range(2):
        got = ops().sample(logits.to(DEV), temps.to(DEV), top_ks.to(DEV), key0.to(torch.int32).to(DEV),
                           key1.to(torch.int32).to(DEV), pos.to(DEV)).tolist()
        assert got == want, [i for i in range(n) if got[i] != want[i]]


def test_top_k_frequencies():
    """Draws with top_k = 3 land on the three largest logits with softmax(top3 / T) frequencies
    (the reference's sampler check: kelpie/scripts/check_build_step.py:101-140)."""
    vocab, n, temp = 300, 20000, 0.7
    row = torch.randn(vocab)
    top = torch.topk(row, 3)
    logits = row.repeat(n, 1).to(DEV)
    tokens = ops().sample(logits, torch.full((n,), temp, device=DEV), torch.full((n,), 3, dtype=torch.int32, device=DEV),
                          torch.full((n,), 99, dtype=torch.int32, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                          torch.arange(n, dtype=torch.int32, device=DEV)).cpu()
    assert set(tokens.tolist()) <= set(top.indices.tolist())
    freq = torch.stack([(tokens == i).float().mean() for i in top.indices])
    want = torch.softmax(top.values / temp, 0)
    assert torch.allclose(freq, want, atol=0.02), (freq, want)
    assert not math.isnan(float(freq.sum()))
    _ = np  # keep numpy imported for debugging sessions
