"""ctypes declarations of the host library's C ABI (csrc/host/engine_abi.h)."""

from __future__ import annotations

import ctypes as C

from ..csrc.build import host_library

ABI_VERSION = 4
I32P = C.POINTER(C.c_int32)


class GroupSpecC(C.Structure):
    _fields_ = [("page_size", C.c_int32), ("window", C.c_int32), ("num_pages", C.c_int32)]


class SchedulerConfigC(C.Structure):
    _fields_ = [
        ("max_requests", C.c_int32), ("max_seq_len", C.c_int32), ("max_batch_tokens", C.c_int32),
        ("max_batch_reqs", C.c_int32), ("order", C.c_int32), ("reserve_ratio", C.c_float),
        ("eos_token", C.c_int32), ("vocab_size", C.c_int32), ("chunk_size", C.c_int32),
    ]


class PlanC(C.Structure):
    _fields_ = [
        ("n_entries", C.c_int32), ("n_tokens", C.c_int32),
        ("req", I32P), ("start", I32P), ("rows", I32P), ("emits", I32P), ("kind", I32P),
        ("input_ids", I32P), ("temperature", C.POINTER(C.c_float)), ("top_k", I32P),
        ("sample_pos", I32P), ("key0", C.POINTER(C.c_uint32)), ("key1", C.POINTER(C.c_uint32)),
    ]


class StepBatchC(C.Structure):
    """A step batch's arrays in the caller's memory with their capacities (R2StepBatch)."""

    _fields_ = [
        ("t_cap", C.c_int32), ("r_cap", C.c_int32), ("w_cap", C.c_int32), ("reserved", C.c_int32),
        ("input_ids", C.c_void_p), ("positions", C.c_void_p), ("row_entry", C.c_void_p), ("q_start", C.c_void_p),
        ("seq_lens", C.c_void_p), ("state_slot", C.c_void_p), ("fresh", C.c_void_p), ("logit_rows", C.c_void_p),
        ("temperature", C.c_void_p), ("top_k", C.c_void_p), ("key0", C.c_void_p), ("key1", C.c_void_p),
        ("sample_pos", C.c_void_p), ("slot_mapping", C.c_void_p), ("block_tables", C.c_void_p),
        ("entry_req", C.c_void_p), ("entry_start", C.c_void_p), ("entry_rows", C.c_void_p),
    ]


class StallC(C.Structure):
    _fields_ = [("stalled", C.c_int32), ("req_id", C.c_int32), ("n_work", C.c_int32),
                ("need_pages", C.c_int32), ("free_pages", C.c_int32), ("group", C.c_int32)]


class RequestEventC(C.Structure):
    _fields_ = [
        ("t_arrival_ns", C.c_int64), ("t_first_sched_ns", C.c_int64), ("t_first_token_ns", C.c_int64),
        ("t_last_token_ns", C.c_int64), ("t_finish_ns", C.c_int64), ("first_step", C.c_int64), ("last_step", C.c_int64),
        ("request_id", C.c_int32), ("n_prompt", C.c_int32), ("n_generated", C.c_int32), ("max_new", C.c_int32),
        ("n_preempted", C.c_int32), ("n_chunks", C.c_int32), ("state", C.c_int32), ("peak_pages", C.c_int32),
    ]


class StepEventC(C.Structure):
    _fields_ = [
        ("step", C.c_int64),
        ("n_entries", C.c_int32), ("n_tokens", C.c_int32), ("n_prefill_rows", C.c_int32), ("n_decode", C.c_int32),
        ("n_admitted", C.c_int32), ("n_preempted", C.c_int32), ("n_finished", C.c_int32),
        ("n_running", C.c_int32), ("n_waiting", C.c_int32), ("kv_free", C.c_int32),
        ("t_plan_ns", C.c_int64), ("t_commit_ns", C.c_int64),
    ]


_lib = None


def lib() -> C.CDLL:
    """The host library with argument types declared; checked against the ABI version and the
    struct sizes (the reference's tripwire: kelpie-core/src/abi_ids.zig:1-40)."""
    global _lib
    if _lib is not None:
        return _lib
    h = host_library()
    vp, i32, f32, u64 = C.c_void_p, C.c_int32, C.c_float, C.c_uint64
    sig = {
        "r2_abi_version": (i32, []),
        "r2_sizeof": (i32, [i32]),
        "r2_last_error": (C.c_char_p, []),
        "r2_cache_create": (vp, [C.POINTER(GroupSpecC), i32, i32, i32]),
        "r2_cache_destroy": (None, [vp]),
        "r2_cache_n_groups": (i32, [vp]),
        "r2_cache_table_width": (i32, [vp, i32]),
        "r2_cache_n_free": (i32, [vp, i32]),
        "r2_cache_open": (i32, [vp, i32]),
        "r2_cache_close": (i32, [vp, i32]),
        "r2_cache_is_open": (i32, [vp, i32]),
        "r2_cache_reserve": (i32, [vp, i32, i32, i32]),
        "r2_cache_can_reserve": (i32, [vp, i32, i32, i32, i32]),
        "r2_cache_slide": (i32, [vp, i32, i32]),
        "r2_cache_pages_held": (i32, [vp, i32, i32]),
        "r2_cache_worst_pages": (i32, [vp, i32, i32, i32, i32]),
        "r2_cache_table": (i32, [vp, i32, i32, I32P, i32]),
        "r2_cache_fill_batch": (i32, [vp, i32, I32P, I32P, I32P, i32, i32] + [I32P] * 8),
        "r2_cache_check": (i32, [vp, C.c_char_p, i32]),
        "r2_sched_create": (vp, [C.POINTER(SchedulerConfigC), C.POINTER(GroupSpecC), i32]),
        "r2_sched_destroy": (None, [vp]),
        "r2_sched_cache": (vp, [vp]),
        "r2_sched_submit": (i32, [vp, I32P, i32, i32, f32, i32, u64, I32P, i32]),
        "r2_sched_cancel": (i32, [vp, i32]),
        "r2_sched_plan": (i32, [vp, C.POINTER(PlanC)]),
        "r2_sched_fill_step_batch": (i32, [vp, C.POINTER(StepBatchC)]),
        "r2_step_batch_check": (i32, [C.POINTER(StepBatchC), i32, i32, i32, i32, C.POINTER(GroupSpecC), I32P, i32, I32P]),
        "r2_sched_commit": (i32, [vp, I32P, i32]),
        "r2_sched_poll": (i32, [vp, i32, I32P, i32, I32P, I32P]),
        "r2_sched_stall": (i32, [vp, C.POINTER(StallC)]),
        "r2_sched_event": (i32, [vp, C.POINTER(StepEventC)]),
        "r2_sched_counts": (i32, [vp, I32P, I32P]),
        "r2_sched_request_info": (i32, [vp, i32] + [I32P] * 5),
        "r2_sched_request_event": (i32, [vp, i32, C.POINTER(RequestEventC)]),
        "r2_sched_drain_request_events": (i32, [vp, C.POINTER(RequestEventC), i32]),
        "r2_sched_grain": (i32, [vp]),
        "r2_sched_set": (i32, [vp, i32, C.c_double]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(h, name)
        fn.restype = res
        fn.argtypes = args
    if h.r2_abi_version() != ABI_VERSION:
        raise RuntimeError(f"host library ABI {h.r2_abi_version()} != expected {ABI_VERSION}")
    for which, struct in enumerate((GroupSpecC, SchedulerConfigC, PlanC, StallC, StepEventC, StepBatchC, RequestEventC)):
        if h.r2_sizeof(which) != C.sizeof(struct):
            raise RuntimeError(f"host library struct {struct.__name__}: size {h.r2_sizeof(which)} != {C.sizeof(struct)}")
    _lib = h
    return h


def last_error() -> str:
    return lib().r2_last_error().decode()
