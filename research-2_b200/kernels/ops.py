"""Python faces of the CUDA kernels: argument checks on the host, then one C call.

Every function here launches hand-written sm_100a code from `csrc/kernels/` on the current
CUDA stream. There is no CPU fallback and no library model or attention code: if the extension
cannot be built or loaded, the call raises. Checks that a sanitizer would make on the device
are made here on the host: dtypes, contiguity, shapes, and that index tensors are int32.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

from ..csrc.build import kernel_library

F32, BF16 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
ACTIVATIONS = {None: ACT_NONE, "none": ACT_NONE, "gelu_new": ACT_GELU_TANH, "gelu": ACT_GELU_ERF}

_STATUS = {-1: "unsupported dtype", -2: "bad shape", -3: "bad alignment", -4: "unsupported size or option"}


class KernelError(RuntimeError):
    pass


class KernelTimeout(KernelError):
    """A bounded wait inside a kernel ran out: the kernel recorded a code and returned instead of
    spinning on. What it computed is not to be trusted. `code` is the recorded number."""

    CODES = {
        1: "a product's operand tile did not arrive (tensor copy)",
        2: "a product's operand stage was not released (tensor-core commit)",
        3: "a product's accumulator was not completed",
        4: "a product's normalised token tile was not built",
        5: "a key/value tile of prefill attention did not arrive (tensor copy)",
        6: "a stage of the tensor-core prefill attention did not complete",
        7: "a step of the resident decode kernel did not reach its grid barrier",
        99: "a wait that a test let run out",
    }

    def __init__(self, code: int):
        super().__init__(f"a kernel gave up a bounded wait (code {code}: {self.CODES.get(code, 'unknown')}); "
                         f"the step's results are not valid")
        self.code = code


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


_launches = 0


_uses: dict[str, int] = {}


def kernel_uses() -> dict[str, int]:
    """How often each attention kernel has been chosen (tests check the choice by it)."""
    return dict(_uses)


def _used(name: str) -> None:
    _uses[name] = _uses.get(name, 0) + 1


def launch_count() -> int:
    """How many kernels of this package have been launched (graph replays count their kernels)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status < 0:
        raise KernelError(f"{what}: refused ({_STATUS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


def _rows(t: torch.Tensor, name: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with contiguous rows, got shape {tuple(t.shape)} stride {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


_libs: dict[str, C.CDLL] = {}


_pdl = os.environ.get("R2_PDL", "1") != "0"


def use_programmatic_dependent_launch(on: bool) -> bool:
    """Kernels are launched so that each may start its prologue (set-up, weight prefetch) while
    its predecessor still runs; every kernel waits for the predecessor before it reads or writes
    anything the predecessor touches. Returns the previous setting."""
    global _pdl
    before, _pdl = _pdl, bool(on)
    for lib in _libs.values():
        lib.r2_set_pdl(int(_pdl))
    return before


def _lib(source: str) -> C.CDLL:
    lib = _libs.get(source)
    if lib is None:
        lib = kernel_library(source)
        lib.r2_set_pdl(int(_pdl))
        _libs[source] = lib
    return lib


def build_all(head_dims=()) -> None:
    """Compile every kernel library that does not depend on a model, and the attention kernels
    for the given head sizes (a model compiles its own head size at first use otherwise)."""
    for source in ("rowwise", "gemm_simt", "gemm_tc", "attention_simt", "attention_prefill_tc", "sampling", "wait_selftest"):
        _lib(source)
    kernel_library("sfu_probe")  # (profiling/sfu_probe.py: a measurement, no part of a step)
    for head_dim in head_dims:
        _lib_for_head_dim("attention_decode", head_dim)
        if head_dim <= 128:
            _lib_for_head_dim("attention_prefill", head_dim)
            _lib_for_head_dim("decode_resident", head_dim)


_tensor_core_gemm = os.environ.get("R2_GEMM", "tc") != "simt"
_fast_attention = os.environ.get("R2_ATTENTION", "fast") != "simt"
_fused_norm = os.environ.get("R2_FUSED_NORM", "1") != "0"
_fused_decode = os.environ.get("R2_FUSED_DECODE", "1") != "0"


def use_fused_decode_attention(on: bool) -> bool:
    """Switch the one-launch decode attention (cache write and slice merge inside) on or off."""
    global _fused_decode
    before, _fused_decode = _fused_decode, bool(on)
    return before


def use_fused_norm(on: bool) -> bool:
    """Switch the LayerNorm inside the matrix product's kernel (few rows, bfloat16) on or off."""
    global _fused_norm
    before, _fused_norm = _fused_norm, bool(on)
    return before


_sm_counts: dict = {}


def sm_count(device) -> int:
    """The device's number of multiprocessors (asked once per device)."""
    device = torch.device(device)
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = int(torch.cuda.get_device_properties(device).multi_processor_count)
    return n


_prefill_tc = {"0": False, "always": "always"}.get(os.environ.get("R2_PREFILL_TC", "1"), True)


def use_prefill_tc(on):
    """The tcgen05 prefill attention kernel (head size 64): False, the mma.sync kernel takes
    every shape; True (or "always", which older callers pass), the tcgen05 kernel takes every
    batch that it can take. Returns the previous setting."""
    global _prefill_tc
    before, _prefill_tc = _prefill_tc, ("always" if on == "always" else bool(on))
    return before


def use_prefill_tma(on: bool, head_dim: int = 64) -> bool:
    """Switch how the prefill attention kernel brings key and value tiles in: 4-D tensor copies
    (TMA, one per page; head size 64 and page sizes 8, 16, 32 or multiples of 64) or 16-byte
    cp.async pieces (every shape). Returns the previous setting."""
    return bool(_lib_for_head_dim("attention_prefill", head_dim).r2_attention_prefill_set_tma(int(bool(on))))


def use_decode_mma(on: bool, head_dim: int = 64) -> bool:
    """Switch the arithmetic of a decode-attention tile between the warp-level tensor cores
    (mma.sync; head sizes up to 128) and scalar float instructions. Returns the previous setting."""
    return bool(_lib_for_head_dim("attention_decode", head_dim).r2_attention_decode_set_mma(int(bool(on))))


def use_fast_attention(on: bool) -> bool:
    """Switch bfloat16 attention between the fast kernels and the general CUDA-core one."""
    global _fast_attention
    before, _fast_attention = _fast_attention, bool(on)
    return before


def decode_slices(n_rows: int, n_kv_heads: int, max_context: int, device="cuda:0") -> int:
    """Slices of the keys per (row, kv head) in decode attention: as many as keep every CTA
    resident at once (four to an SM is what every head size's kernel reaches; a second wave of
    CTAs costs more than the slices gain: 8 rows x 12 heads took 8.4 us with 6 slices, 10.3 us with
    8), never less than 128 keys a slice."""
    ctas = max(1, n_rows * n_kv_heads)
    want = max(1, 4 * sm_count(device) // ctas)
    most = max(1, max_context // 128)
    return max(1, min(want, most, 32))


def _lib_for_head_dim(source: str, head_dim: int) -> C.CDLL:
    key = f"{source}:{head_dim}"
    lib = _libs.get(key)
    if lib is None:
        lib = kernel_library(source, {"HEAD_DIM": head_dim})
        lib.r2_set_pdl(int(_pdl))
        if source == "attention_decode":
            lib.r2_attention_decode_scratch_floats.restype = C.c_longlong
        _libs[key] = lib
    return lib


def use_tensor_core_gemm(on: bool) -> bool:
    """Switch the bfloat16 matrix products between the tcgen05 kernel and the CUDA-core one
    (tests compare the two). Returns the previous setting."""
    global _tensor_core_gemm
    before, _tensor_core_gemm = _tensor_core_gemm, bool(on)
    return before


_kv_in_epilogue = os.environ.get("R2_KV_IN_EPILOGUE", "1") != "0"


def use_kv_in_epilogue(on: bool) -> bool:
    """Switch the writing of keys and values into the cache by the q/k/v product's epilogue (more
    than 64 bfloat16 rows) on or off; off, a kernel of its own writes them. Returns the previous setting."""
    global _kv_in_epilogue
    before, _kv_in_epilogue = _kv_in_epilogue, bool(on)
    return before


def use_pair_gemm(mode):
    """The two-CTA persistent form (tcgen05.mma.cta_group::2, 256-row tiles) of the tensor-core
    product: False never, True where it is the faster form (many tiles per SM), "always" wherever
    it can run (192 rows and 128 columns or more; tests compare it with the single-CTA form).
    Returns the previous setting in the same terms."""
    names = {0: False, 1: True, 2: "always"}
    code = {False: 0, True: 1, "always": 2}[mode]
    return names[_lib("gemm_tc").r2_gemm_tc_set_pair(code)]


def gemm_cta_stamps(buffer: torch.Tensor | None) -> int:
    """Profiling: the tensor-core products launched (or captured into a graph) from now on leave six times of
    the nanosecond clock per CTA in `buffer` (int64 [n, 6] on the device: start, before and after the wait on the
    kernel before, tokens normalised, products complete, end; single-CTA forms only); None switches it off.
    Returns the number of CTAs of the last such launch."""
    if buffer is None:
        return int(_lib("gemm_tc").r2_gemm_tc_set_cta_stamps(None, 0))
    _need(buffer, "buffer", torch.int64, 2)
    if buffer.shape[1] != 6 or not buffer.is_contiguous():
        raise KernelError("gemm_cta_stamps: the buffer must be a contiguous int64 [n, 6]")
    return int(_lib("gemm_tc").r2_gemm_tc_set_cta_stamps(C.c_void_p(buffer.data_ptr()), buffer.shape[0]))


if os.environ.get("R2_PAIR_GEMM", "1") == "0":
    use_pair_gemm(False)


class _Workspace:
    """Scratch of sliced decode attention (the slices' partial results, arrival counters that are
    zero between launches) and the word in which kernels record a bounded wait that ran out.
    One per device, sized once."""

    FLOATS = 4 * 1024 * 1024
    COUNTERS = 4096

    def __init__(self, device):
        self.floats = torch.empty(self.FLOATS, dtype=torch.float32, device=device)
        self.counters = torch.zeros(self.COUNTERS, dtype=torch.int32, device=device)
        self.error = torch.zeros(4, dtype=torch.int32, device=device)


_workspaces: dict = {}


def _workspace(device) -> _Workspace:
    ws = _workspaces.get(device)
    if ws is None:
        ws = _workspaces[device] = _Workspace(device)
    return ws


def device_errors(device="cuda:0") -> int:
    """0, or the code that a kernel left when one of its bounded waits ran out (synchronises)."""
    ws = _workspaces.get(torch.device(device))
    return 0 if ws is None else int(ws.error[0].item())


def error_word(device) -> torch.Tensor:
    """The device's error word (int32 [4]; element 0 holds the code): a step's graph copies it to the
    host beside its tokens, so that a time-out is seen without a transfer of its own."""
    return _workspace(torch.device(device)).error


def raise_on_device_error(device="cuda:0", code: int | None = None) -> None:
    """Raises KernelTimeout if a kernel on `device` has recorded that a bounded wait ran out, and
    clears the word so that later steps are checked on their own. `code` is the word's value when the
    caller has read it already (a graph's pinned copy); else it is read here (synchronises)."""
    if code is None:
        code = device_errors(device)
    if code:
        ws = _workspaces.get(torch.device(device))
        if ws is not None:
            ws.error.zero_()
        raise KernelTimeout(int(code))


def wait_selftest(device="cuda:0", polls: int = 64, code: int = 99) -> None:
    """Launches the kernel that waits `polls` polls on a barrier nothing arrives on and then records
    `code` in the device's error word (csrc/kernels/wait_selftest.cu). For tests of the error path."""
    ws = _workspace(torch.device(device))
    with torch.cuda.device(device):
        _check(_lib("wait_selftest").r2_wait_selftest(_p(ws.error), int(polls), int(code), _stream()), "wait_selftest")


# ---------------------------------------------------------------------------------------------


def embed(ids: torch.Tensor, table: torch.Tensor, positions: torch.Tensor | None = None,
          pos_table: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]] (+ pos_table[positions[t]]) as float32 [T, width]."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", dim=2)
    n, width = ids.shape[0], table.shape[1]
    if not table.is_contiguous():
        raise KernelError("table must be contiguous")
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype, 2)
        _need(positions, "positions", torch.int32, 1)
        if pos_table.shape[1] != width or not pos_table.is_contiguous() or positions.shape[0] != n:
            raise KernelError("pos_table / positions do not fit the token table")
    if out is None:
        out = torch.empty(n, width, dtype=torch.float32, device=ids.device)
    _need(out, "out", torch.float32, 2)
    fn = _lib("rowwise").r2_embed
    status = fn(_p(ids), _p(positions), _p(table), _p(pos_table), _p(out), n, width, table.shape[0],
                0 if pos_table is None else pos_table.shape[0], dtype_code(table.dtype), _stream())
    _check(status, "embed")
    return out


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, out_dtype: torch.dtype,
               rows: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """LayerNorm of float32 rows; `rows` (int32) picks input rows, else all rows in order."""
    _need(x, "x", torch.float32, 2)
    _need(gamma, "gamma", torch.float32, 1)
    _need(beta, "beta", torch.float32, 1)
    if not x.is_contiguous() or gamma.shape[0] != x.shape[1] or beta.shape[0] != x.shape[1]:
        raise KernelError(f"layer_norm: x {tuple(x.shape)} gamma {tuple(gamma.shape)} beta {tuple(beta.shape)}")
    n = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n = rows.shape[0]
    if out is None:
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
    status = _lib("rowwise").r2_layer_norm(_p(x), _p(rows), _p(gamma), _p(beta), _p(out), n, x.shape[1],
                                          C.c_float(eps), dtype_code(out.dtype), _stream())
    _check(status, "layer_norm")
    return out


class NormedRows:
    """LayerNorm of float32 rows that has not been computed yet: `linear` may compute it inside
    its own kernel (few rows, bfloat16), or `materialize()` runs the LayerNorm kernel."""

    def __init__(self, x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, dtype: torch.dtype,
                 rows: torch.Tensor | None = None):
        self.x, self.gamma, self.beta, self.eps, self.dtype, self.rows = x, gamma, beta, eps, dtype, rows
        self.shape = (x.shape[0] if rows is None else rows.shape[0], x.shape[1])
        self.device = x.device

    def materialize(self) -> torch.Tensor:
        return layer_norm(self.x, self.gamma, self.beta, self.eps, self.dtype, rows=self.rows)


def _linear_of_normed(a: NormedRows, w, bias, w_is_nk, act, residual, out_dtype, out):
    """The fused form, or None when the kernel does not take the shape."""
    m, k = a.shape
    n = w.shape[0] if w_is_nk else w.shape[1]
    if not (_tensor_core_gemm and _fused_norm and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and m <= 16 and k <= 1024):
        return None
    if (w.shape[1] if w_is_nk else w.shape[0]) != k:
        raise KernelError(f"linear: normed rows {a.shape} do not fit w {tuple(w.shape)} (w_is_nk={w_is_nk})")
    _need(a.x, "x", torch.float32, 2)
    if not a.x.is_contiguous():
        return None
    if out_dtype is None:
        out_dtype = torch.float32 if residual is not None else a.dtype
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    ldr = _rows(residual, "residual") if residual is not None else 0
    ws = _workspace(a.device)
    status = _lib("gemm_tc").r2_gemm_tc(
        None, 0, _p(w), _rows(w, "w"), int(w_is_nk), _p(bias), _p(residual), ldr, _p(out), _rows(out, "out"), m, n, k,
        ACTIVATIONS[act], dtype_code(out.dtype), _p(ws.error), _p(a.x), a.x.stride(0), _p(a.rows), _p(a.gamma),
        _p(a.beta), C.c_float(a.eps), None, C.c_longlong(0), None, _stream())
    if status == -4:
        return None
    _check(status, "linear (tensor cores, fused norm)")
    return out


def mlp(h, w_in: torch.Tensor, b_in: torch.Tensor, act: str, w_out: torch.Tensor, b_out: torch.Tensor | None,
        residual: torch.Tensor | None = None) -> torch.Tensor:
    """act(h @ w_in + b_in) @ w_out + b_out (+ residual), both matrices stored [in, out]. `h` may be
    NormedRows (the LayerNorm then runs inside the first product's kernel where it can)."""
    inner = linear(h, w_in, b_in, act=act)
    return linear(inner, w_out, b_out, residual=residual)


class KvScatter(C.Structure):
    """Where the key and value columns of a fused q/k/v product go: the rows' cache slots.
    `col` is the first key column, `width` the keys' (and the values') width."""

    _fields_ = [("slots", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("page_stride", C.c_longlong),
                ("page_size", C.c_int), ("n_pages", C.c_int), ("col", C.c_int), ("width", C.c_int), ("head_dim", C.c_int)]


def kv_scatter(slot_mapping: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_stride: int, page_size: int,
               n_pages: int, col: int, width: int, head_dim: int) -> KvScatter:
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    return KvScatter(_p(slot_mapping), _p(k_cache), _p(v_cache), page_stride, page_size, n_pages, col, width, head_dim)


def linear(a, w: torch.Tensor, bias: torch.Tensor | None = None, *, w_is_nk: bool = False,
           act: str | None = None, residual: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None, kv: KvScatter | None = None):
    """act(a @ w + bias) (+ residual). `w` is [K, N], or [N, K] with w_is_nk. `a` and `w`
    share a dtype; bias and residual are float32; a float32 residual makes a float32 result.
    `a` may be NormedRows: the LayerNorm then runs inside the product's kernel where it can.

    With `kv` (a fused q/k/v product) the result is (out, written): where the tensor-core kernel
    takes the case (more than 64 bfloat16 rows), the key and value columns go straight into the
    rows' cache slots, `written` is True and those columns of `out` are left undefined; else
    `written` is False and `out` is whole."""
    if kv is not None:
        rows = a.shape[0]
        if _tensor_core_gemm and _kv_in_epilogue and rows > 64 and act is None and residual is None and out_dtype in (None, torch.bfloat16):
            tokens = a.materialize() if isinstance(a, NormedRows) else a
            if tokens.dtype == torch.bfloat16:
                written = _linear_kv(tokens, w, bias, w_is_nk, out, kv)
                if written is not None:
                    return written, True
            a = tokens
        return linear(a, w, bias, w_is_nk=w_is_nk, act=act, residual=residual, out_dtype=out_dtype, out=out), False
    if isinstance(a, NormedRows):
        if act not in ACTIVATIONS:
            raise KernelError(f"linear: unknown activation {act!r}; known: {sorted(k for k in ACTIVATIONS if k)}")
        fused = _linear_of_normed(a, w, bias, w_is_nk, act, residual, out_dtype, out)
        if fused is not None:
            return fused
        a = a.materialize()
    _need(a, "a", dim=2)
    _need(w, "w", a.dtype, 2)
    m, k = a.shape
    n = w.shape[0] if w_is_nk else w.shape[1]
    if (w.shape[1] if w_is_nk else w.shape[0]) != k:
        raise KernelError(f"linear: a {tuple(a.shape)} does not fit w {tuple(w.shape)} (w_is_nk={w_is_nk})")
    lda, ldw = _rows(a, "a"), _rows(w, "w")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError(f"linear: bias {tuple(bias.shape)} does not fit n={n}")
    if out_dtype is None:
        out_dtype = torch.float32 if residual is not None else a.dtype
    ldr = 0
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
        if tuple(residual.shape) != (m, n):
            raise KernelError(f"linear: residual {tuple(residual.shape)} is not [{m}, {n}]")
        ldr = _rows(residual, "residual")
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    if tuple(out.shape) != (m, n):
        raise KernelError(f"linear: out {tuple(out.shape)} is not [{m}, {n}]")
    if act not in ACTIVATIONS:
        raise KernelError(f"linear: unknown activation {act!r}; known: {sorted(k for k in ACTIVATIONS if k)}")
    if a.dtype == torch.bfloat16 and _tensor_core_gemm:
        ws = _workspace(a.device)
        status = _lib("gemm_tc").r2_gemm_tc(
            _p(a), lda, _p(w), ldw, int(w_is_nk), _p(bias), _p(residual), ldr, _p(out), _rows(out, "out"), m, n, k,
            ACTIVATIONS[act], dtype_code(out.dtype), _p(ws.error), None, 0, None, None, None, C.c_float(0.0),
            None, C.c_longlong(0), None, _stream())
        if status != -4:  # -4: a shape the tensor-core kernel does not take; the CUDA-core kernel does
            _check(status, "linear (tensor cores)")
            return out
    status = _lib("gemm_simt").r2_gemm_simt(
        _p(a), lda, _p(w), ldw, int(w_is_nk), _p(bias), _p(residual), ldr, _p(out), _rows(out, "out"), m, n, k,
        ACTIVATIONS[act], dtype_code(a.dtype), dtype_code(out.dtype), _stream())
    _check(status, "linear")
    return out


def _linear_kv(a: torch.Tensor, w: torch.Tensor, bias, w_is_nk: bool, out, kv: KvScatter):
    """The fused q/k/v product with keys and values written to the cache by the epilogue; None
    where the tensor-core kernel does not take the case."""
    _need(a, "a", torch.bfloat16, 2)
    _need(w, "w", a.dtype, 2)
    m, k = a.shape
    n = w.shape[0] if w_is_nk else w.shape[1]
    if (w.shape[1] if w_is_nk else w.shape[0]) != k:
        raise KernelError(f"linear: a {tuple(a.shape)} does not fit w {tuple(w.shape)} (w_is_nk={w_is_nk})")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    ws = _workspace(a.device)
    status = _lib("gemm_tc").r2_gemm_tc(
        _p(a), _rows(a, "a"), _p(w), _rows(w, "w"), int(w_is_nk), _p(bias), None, 0, _p(out), _rows(out, "out"), m, n, k,
        ACTIVATIONS[None], dtype_code(out.dtype), _p(ws.error), None, 0, None, None, None, C.c_float(0.0),
        None, C.c_longlong(0), C.byref(kv), _stream())
    if status == -4:
        return None
    _check(status, "linear (tensor cores, keys and values into the cache)")
    return out


def kv_write(k_src: torch.Tensor, v_src: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             slot_mapping: torch.Tensor, n_kv_heads: int, head_dim: int, page_size: int, page_stride: int,
             n_pages: int) -> None:
    """Scatter this step's keys and values [T, n_kv_heads * head_dim] into their cache slots."""
    _need(k_src, "k_src", dim=2)
    _need(v_src, "v_src", k_src.dtype, 2)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    if k_cache.dtype != k_src.dtype or v_cache.dtype != k_src.dtype:
        raise KernelError("kv_write: the cache and the new keys/values must share a dtype")
    n = k_src.shape[0]
    if k_src.shape[1] != n_kv_heads * head_dim or v_src.shape != k_src.shape or slot_mapping.shape[0] < n:
        raise KernelError("kv_write: shapes do not fit")
    stride = _rows(k_src, "k_src")
    if _rows(v_src, "v_src") != stride:
        raise KernelError("kv_write: k and v must share a row stride")
    status = _lib("rowwise").r2_kv_write(_p(k_src), _p(v_src), stride, _p(k_cache), _p(v_cache), _p(slot_mapping), n,
                                        n_kv_heads, head_dim, page_size, C.c_longlong(page_stride), n_pages,
                                        dtype_code(k_src.dtype), _stream())
    _check(status, "kv_write")


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_stride: int, page_size: int,
                    n_pages: int, block_tables: torch.Tensor, row_entry: torch.Tensor, positions: torch.Tensor,
                    seq_lens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                    window: int = 0, out: torch.Tensor | None = None, *, decode_only: bool = False,
                    max_context: int = 0, q_start: torch.Tensor | None = None, n_tiles: int = 0) -> torch.Tensor:
    """Causal attention of q [T, n_heads * head_dim] over the paged cache -> [T, n_heads * head_dim].
    `decode_only` says that every row is an entry of its own (one new token each) and
    `max_context` bounds the rows' context lengths; `q_start` (int32 [R + 1]) with `n_tiles`, the
    sum over entries of ceil(rows / 64), lets the tensor-core prefill kernel take the batch. They
    only choose the kernel and its slicing."""
    _need(q, "q", dim=2)
    for name, t in (("row_entry", row_entry), ("positions", positions), ("seq_lens", seq_lens)):
        _need(t, name, torch.int32, 1)
    _need(block_tables, "block_tables", torch.int32, 2)
    if not block_tables.is_contiguous():
        raise KernelError("block_tables must be contiguous")
    n = q.shape[0]
    if q.shape[1] != n_heads * head_dim:
        raise KernelError(f"attention: q {tuple(q.shape)} is not [T, {n_heads} * {head_dim}]")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise KernelError("attention: q and the cache must share a dtype")
    if head_dim % 16 != 0:
        raise KernelError(f"attention: head sizes come in steps of 16, got {head_dim}")
    if out is None:
        out = torch.empty(n, n_heads * head_dim, dtype=q.dtype, device=q.device)
    group = n_heads // max(n_kv_heads, 1)
    if q.dtype == torch.bfloat16 and decode_only and _fast_attention and group in (1, 2, 4, 8):
        lib = _lib_for_head_dim("attention_decode", head_dim)
        n_slices = decode_slices(n, n_kv_heads, max_context, q.device)
        ws = _workspace(q.device)
        need = lib.r2_attention_decode_scratch_floats(n, n_heads, n_slices)
        if need > ws.floats.numel():
            n_slices, need = 1, 0
        status = lib.r2_attention_decode(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride),
            page_size, n_pages, _p(block_tables), block_tables.shape[1], _p(row_entry), _p(positions), _p(seq_lens),
            n, n_heads, n_kv_heads, C.c_float(scale), window, n_slices, _p(ws.floats), C.c_longlong(ws.floats.numel()),
            _stream())
        _check(status, "paged_attention (decode)")
        if n_slices > 1:
            count_launches(1)  # the merge kernel
        return out
    if q.dtype == torch.bfloat16 and _fast_attention and _prefill_tc and q_start is not None and n_tiles > 0 and head_dim == 64:
        # tcgen05 form (head size 64, pages of 8, 16, 32 or a multiple of 64 keys): 128-row tiles, one entry to a
        # tile. Also where most tiles are mostly empty (single decoded tokens beside a portion: 64 such rows
        # and 448 of a prompt take 40 us against the mma.sync kernel's 49).
        _need(q_start, "q_start", torch.int32, 1)
        n_entries = q_start.shape[0] - 1
        status = _lib("attention_prefill_tc").r2_attention_prefill_tc(
            _p(q), _rows(q, "q"), n, _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride),
            page_size, n_pages, _p(block_tables), block_tables.shape[1], _p(q_start), _p(seq_lens), n_entries,
            (n_tiles + n_entries + 1) // 2, n_heads, n_kv_heads, C.c_float(scale), window, _p(_workspace(q.device).error), _stream())
        if status != -4:
            _check(status, "paged_attention (prefill, tcgen05)")
            _used("attention_prefill_tc")
            return out
    if (q.dtype == torch.bfloat16 and _fast_attention and q_start is not None and n_tiles > 0 and head_dim <= 128
            and _rows(q, "q") % 8 == 0 and q.data_ptr() % 16 == 0):
        _need(q_start, "q_start", torch.int32, 1)
        lib = _lib_for_head_dim("attention_prefill", head_dim)
        status = lib.r2_attention_prefill(
            _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride),
            page_size, n_pages, _p(block_tables), block_tables.shape[1], _p(q_start), _p(seq_lens),
            q_start.shape[0] - 1, n_tiles, n_heads, n_kv_heads, C.c_float(scale), window, _p(_workspace(q.device).error),
            _stream())
        _check(status, "paged_attention (prefill)")
        _used("attention_prefill")
        return out
    status = _lib("attention_simt").r2_attention_simt(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride),
        page_size, _p(block_tables), block_tables.shape[1], _p(row_entry), _p(positions), _p(seq_lens), n, n_heads,
        n_kv_heads, head_dim, C.c_float(scale), window, n_pages, dtype_code(q.dtype), _stream())
    _check(status, "paged_attention")
    return out


def decode_attention_fused(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, slot_mapping: torch.Tensor,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, page_stride: int, page_size: int, n_pages: int,
                           block_tables: torch.Tensor, row_entry: torch.Tensor, positions: torch.Tensor,
                           seq_lens: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                           window: int, max_context: int) -> torch.Tensor | None:
    """Decode attention in ONE launch for a batch in which every row is an entry of its own: the
    kernel writes the new keys and values to their cache slots, and the slice that finishes last
    merges all slices of its row. Returns None when it does not take the case (the caller then writes
    the cache and calls `paged_attention`)."""
    group = n_heads // max(n_kv_heads, 1)
    if not (_fast_attention and _fused_decode and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and group in (1, 2, 4, 8) and head_dim % 16 == 0):
        return None
    _need(q, "q", dim=2)
    _need(k_new, "k_new", torch.bfloat16, 2)
    _need(v_new, "v_new", torch.bfloat16, 2)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    _need(block_tables, "block_tables", torch.int32, 2)
    n = q.shape[0]
    stride = _rows(k_new, "k_new")
    if _rows(v_new, "v_new") != stride or k_new.shape != (n, n_kv_heads * head_dim) or slot_mapping.shape[0] < n:
        raise KernelError("decode attention: the new keys and values do not fit the rows")
    slices = decode_slices(n, n_kv_heads, max_context, q.device)
    lib = _lib_for_head_dim("attention_decode", head_dim)
    ws = _workspace(q.device)
    if (lib.r2_attention_decode_scratch_floats(n, n_heads, slices) > ws.floats.numel()
            or n * n_kv_heads > ws.counters.numel()):
        slices = 1
    out = torch.empty(n, n_heads * head_dim, dtype=q.dtype, device=q.device)
    status = lib.r2_attention_decode_fused(
        _p(q), _rows(q, "q"), _p(out), _rows(out, "out"), _p(k_cache), _p(v_cache), C.c_longlong(page_stride), page_size,
        n_pages, _p(block_tables), block_tables.shape[1], _p(row_entry), _p(positions), _p(seq_lens), n, n_heads,
        n_kv_heads, C.c_float(scale), window, slices, _p(k_new), _p(v_new), stride, _p(slot_mapping), _p(ws.floats),
        C.c_longlong(ws.floats.numel()), _p(ws.counters), ws.counters.numel(), _stream())
    if status == -4:
        return None
    _check(status, "decode attention (fused)")
    return out


_resident_decode = os.environ.get("R2_RESIDENT_DECODE", "1") != "0"


def use_resident_decode(on: bool) -> bool:
    """Switch the one-kernel form of a decode step's layers (csrc/kernels/decode_resident.cu) on or
    off; off, every part of a layer launches its own kernels. Returns the previous setting."""
    global _resident_decode
    before, _resident_decode = _resident_decode, bool(on)
    return before


_resident_rows = int(os.environ.get("R2_RESIDENT_ROWS", "16"))


def set_resident_decode_rows(n: int) -> int:
    """The most rows of a decode-only batch that run as the resident kernel (it takes up to 64). The
    default is 16: up to there it measured faster than the chain of kernels at GPT-2 124M sizes (0.39 against
    0.46 ms a step of 8 rows, 0.46 against 0.54 at 12, 0.53 against 0.57 at 16), at 24 rows the same (0.62) and
    beyond it slower (0.73 against 0.69 at 32, 1.07 against 0.88 at 64: every CTA reads all rows of a
    product's input). Returns the previous value."""
    global _resident_rows
    before, _resident_rows = _resident_rows, int(n)
    return before


def resident_decode_rows() -> int:
    return _resident_rows if (_resident_decode and _tensor_core_gemm and _fast_attention) else 0


RESIDENT_MAX_GROUPS = 4


class ResidentLayerC(C.Structure):
    """One layer of the resident decode kernel (R2ResidentLayer in csrc/kernels/decode_resident.cu)."""

    _fields_ = [("w_qkv", C.c_void_p), ("w_out", C.c_void_p), ("w_fc", C.c_void_p), ("w_pr", C.c_void_p),
                ("b_qkv", C.c_void_p), ("b_out", C.c_void_p), ("b_fc", C.c_void_p), ("b_pr", C.c_void_p),
                ("ln1_g", C.c_void_p), ("ln1_b", C.c_void_p), ("ln2_g", C.c_void_p), ("ln2_b", C.c_void_p),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("page_stride", C.c_longlong),
                ("group", C.c_int), ("page_size", C.c_int), ("n_pages", C.c_int), ("window", C.c_int),
                ("scale", C.c_float), ("eps1", C.c_float), ("eps2", C.c_float), ("act", C.c_int)]


class ResidentShapeC(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("width", C.c_int), ("inner", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("n_rows", C.c_int)]


class ResidentBuffersC(C.Structure):
    _fields_ = [("x", C.c_void_p), ("qkv", C.c_void_p), ("mixed", C.c_void_p), ("hidden", C.c_void_p),
                ("barrier", C.c_void_p), ("error_flag", C.c_void_p), ("positions", C.c_void_p), ("seq_lens", C.c_void_p),
                ("block_tables", C.c_void_p * RESIDENT_MAX_GROUPS), ("slot_mapping", C.c_void_p * RESIDENT_MAX_GROUPS),
                ("table_width", C.c_int * RESIDENT_MAX_GROUPS), ("stamps", C.c_void_p)]


def pack_weight_tiles(w: torch.Tensor) -> torch.Tensor:
    """A [K, N] matrix (stored [in, out]) in the order in which the resident decode kernel's warps hold
    it: [N / 16 feature tiles][K / 16 k tiles][32 lanes][8 values], a lane's eight values being its
    registers of the 16 x 16 operand tile of mma.sync m16n8k16 (rows = features, columns = k)."""
    k, n = w.shape
    if k % 16 or n % 16:
        raise KernelError(f"pack_weight_tiles: both sizes must be multiples of 16, got {tuple(w.shape)}")
    lane = torch.arange(32, device=w.device)
    g, t = lane >> 2, lane & 3
    r, e = torch.arange(4, device=w.device), torch.arange(2, device=w.device)
    m_idx = (g[:, None, None] + 8 * (r[None, :, None] & 1) + 0 * e[None, None, :])      # feature within the tile
    k_idx = (2 * t[:, None, None] + e[None, None, :] + 8 * (r[None, :, None] >> 1))      # k within the tile
    tiles = w.reshape(k // 16, 16, n // 16, 16).permute(2, 0, 3, 1)                      # [feature tile, k tile, feature, k]
    return tiles[:, :, m_idx, k_idx].contiguous().view(-1)


def decode_resident_library(head_dim: int) -> C.CDLL:
    return _lib_for_head_dim("decode_resident", head_dim)


def decode_resident(head_dim: int, layers: torch.Tensor, shape: ResidentShapeC, buffers: ResidentBuffersC, page_shift: int,
                    device) -> bool:
    """All layers of a decode-only step in one launch; False where the kernel does not take the case."""
    status = decode_resident_library(head_dim).r2_decode_resident(
        _p(layers), C.byref(shape), C.byref(buffers), page_shift, sm_count(device), _stream())
    if status == -4:
        return False
    _check(status, "decode step (resident kernel)")
    _used("decode_resident")
    return True


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, key0: torch.Tensor,
           key1: torch.Tensor, sample_pos: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V] -> int32 [R]."""
    _need(logits, "logits", torch.float32, 2)
    n, vocab = logits.shape
    _need(temperature, "temperature", torch.float32, 1)
    _need(top_k, "top_k", torch.int32, 1)
    _need(sample_pos, "sample_pos", torch.int32, 1)
    for name, t in (("key0", key0), ("key1", key1)):
        if not t.is_cuda or t.dtype not in (torch.int32, torch.uint32) or t.dim() != 1:
            raise KernelError(f"{name} must be a 1-D CUDA tensor of 32-bit integers")
    if min(temperature.shape[0], top_k.shape[0], key0.shape[0], key1.shape[0], sample_pos.shape[0]) < n:
        raise KernelError("sample: a per-row parameter is shorter than the logits")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    status = _lib("sampling").r2_sample(_p(logits), _rows(logits, "logits"), n, vocab, _p(temperature), _p(top_k),
                                       _p(key0), _p(key1), _p(sample_pos), _p(out), _stream())
    _check(status, "sample")
    return out
