"""The decode-attention entry point for callers that cannot allocate device memory.

Some hosts of this library may not call cudaMalloc: they live inside another process's memory
budget, or must stay allocation-free in the middle of work they do not control.
`r2_attention_decode_static` serves them: same inputs and outputs as `r2_attention_decode`, but
the scratch for the slices' partial results is an array inside the library instead of a buffer
from the caller. This test calls it through its exported C symbol, twice in a row (the second
call finds the first call's leftovers in the shared array), and compares each result with the
ordinary entry point's on the same inputs; it also checks that a request beyond the built-in
array's size is refused with a message and launches nothing.

The file name sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""

from __future__ import annotations

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_FLOATS = 512 * 1024
TOO_SMALL = -5


def _case(seed, contexts, n_heads, n_kv, hd, page):
    from tests.test_kernels_gpu import PagedCase

    case = PagedCase([(c, 1) for c in contexts], n_heads, n_kv, hd, page, torch.bfloat16, seed=seed)
    from research_2_b200.kernels import ops

    ops.kv_write(case.k_new, case.v_new, case.k_cache, case.v_cache, case.slots, case.n_kv, case.hd, case.page,
                 case.page_stride, case.n_pages)
    return case


def _library(hd):
    from research_2_b200.kernels import ops

    lib = ops._lib_for_head_dim("attention_decode", hd)
    lib.r2_attention_decode_static_error.restype = C.c_char_p
    return lib


def _args(case, out, scale, window, n_slices):
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    n = case.q_rows.shape[0]
    return [p(case.q_rows), case.q_rows.stride(0), p(out), out.stride(0), p(case.k_cache), p(case.v_cache),
            C.c_longlong(case.page_stride), case.page, case.n_pages, p(case.tables), case.tables.shape[1],
            p(case.row_entry), p(case.positions), p(case.seq_lens), n, case.n_heads, case.n_kv, C.c_float(scale),
            window, n_slices]


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    hd = 64
    lib = _library(hd)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second finds the first one's partials in the array
    problems = [(_case(1, [700, 33, 0, 129, 512], 4, 2, hd, 16), 6, 0), (_case(2, [90, 1000, 257], 4, 4, hd, 8), 3, 50)]
    for case, n_slices, window in problems:
        scale = hd**-0.5
        n = case.q_rows.shape[0]
        want = torch.empty(n, case.n_heads * hd, dtype=torch.bfloat16, device=DEV)
        got = torch.full_like(want, float("nan"))
        scratch = torch.empty(n * case.n_heads * n_slices * (hd + 2), dtype=torch.float32, device=DEV)
        status = lib.r2_attention_decode(*_args(case, want, scale, window, n_slices), C.c_void_p(scratch.data_ptr()),
                                         C.c_longlong(scratch.numel()), stream)
        assert status == 0
        before = torch.cuda.memory_allocated()
        status = lib.r2_attention_decode_static(*_args(case, got, scale, window, n_slices), stream)
        assert status == 0, lib.r2_attention_decode_static_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(got.float().cpu(), case.plain(scale, window), atol=3e-2, rtol=3e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    hd = 64
    lib = _library(hd)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    case = _case(3, [40] * 64, 8, 8, hd, 16)
    out = torch.full((64, 8 * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    n_slices = 32  # 64 rows x 8 heads x 32 slices x 66 floats > the built-in array
    assert 64 * 8 * n_slices * (hd + 2) > STATIC_FLOATS
    status = lib.r2_attention_decode_static(*_args(case, out, 0.125, 0, n_slices), stream)
    assert status == TOO_SMALL
    message = lib.r2_attention_decode_static_error().decode()
    assert "need" in message and str(STATIC_FLOATS) in message
    torch.cuda.synchronize()
    assert torch.all(out == 7.0), "a refused call must not launch anything"
    # one slice needs no scratch at all and always passes
    status = lib.r2_attention_decode_static(*_args(case, out, 0.125, 0, 1), stream)
    assert status == 0
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float().cpu(), case.plain(0.125, 0), atol=3e-2, rtol=3e-2)
