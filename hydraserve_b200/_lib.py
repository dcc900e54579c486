"""ctypes binding of the C ABI declared in ``include/hs_sampler.h``.

The library is loaded from ``hydraserve_b200/lib``; if it has not been built the import
of this module fails with instructions, it never falls back to another implementation.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libhs_sampler.so"

HS_MAX_LOGPROBS = 20
HS_DTYPE_F32, HS_DTYPE_BF16 = 0, 1
HS_ROW_PLAIN_GREEDY = 1
HS_SAMPLE_APPEND_TOKEN = 1
HS_SAMPLE_GENERAL_KERNEL = 2
HS_CREATE_FORCE_GENERAL = 1
HS_CREATE_PHASE_CLOCKS = 2


def HS_CREATE_CLUSTER(n: int) -> int:
    return (int(n) & 0xF) << 8


HS_NOALLOC_MAX_BATCH = 1024

# Mirrors of struct hs_row_params / hs_row_out (natural C alignment, no padding needed).
ROW_PARAMS = np.dtype([
    ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"),
    ("repetition_penalty", "<f4"), ("presence_penalty", "<f4"), ("frequency_penalty", "<f4"),
    ("top_k", "<i4"), ("n_logprobs", "<i4"), ("seed", "<u8"), ("flags", "<u4"), ("slot", "<i4"),
], align=True)
ROW_OUT = np.dtype([
    ("token", "<i4"), ("logprob", "<f4"), ("n_top", "<i4"), ("status", "<i4"),
    ("n_kept", "<i4"), ("n_after_topk", "<i4"), ("n_after_minp", "<i4"), ("n_after_topp", "<i4"),
    ("cut_bits", "<u4"), ("n_cut_ties", "<i4"), ("row_max", "<f4"), ("log_z", "<f4"),
    ("top_ids", "<i4", (HS_MAX_LOGPROBS,)), ("top_logprobs", "<f4", (HS_MAX_LOGPROBS,)),
], align=True)
HS_SHARD_CAND = 64
SHARD_REC = np.dtype([
    ("row_max", "<f4"), ("pad", "<f4"), ("z_mass", "<u8"), ("n", "<i4"), ("status", "<i4"),
    ("ids", "<i4", (HS_SHARD_CAND,)), ("scores", "<f4", (HS_SHARD_CAND,)),
], align=True)
assert ROW_PARAMS.itemsize == 48 and ROW_OUT.itemsize == 208 and SHARD_REC.itemsize == 536

EXPORTS = {
    # name: (restype, argtypes)
    "hs_abi_version": (C.c_int, []),
    "hs_status_string": (C.c_char_p, [C.c_int]),
    "hs_last_error": (C.c_char_p, [C.c_void_p]),
    "hs_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "hs_create_ex": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint32, C.POINTER(C.c_void_p)]),
    "hs_destroy": (C.c_int, [C.c_void_p]),
    "hs_slots_reset": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "hs_slots_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                  C.c_int, C.c_void_p]),
    "hs_slot_unique_count": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_int)]),
    "hs_sample": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_void_p,
                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "hs_sample_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_void_p,
                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "hs_greedy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_void_p,
                            C.c_void_p]),
    "hs_greedy_noalloc": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "hs_greedy_noalloc_error": (C.c_char_p, []),
    "hs_sample_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "hs_sharded_partial": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_void_p]),
    "hs_sharded_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p]),
    "hs_query": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "hs_debug_phase_clocks": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "hs_debug_set": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library once; raise if it is not there."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m hydraserve_b200.build` "
                "(there is no non-CUDA implementation to fall back to)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


class SamplerError(RuntimeError):
    pass


def check(lib, handle, status: int, what: str) -> None:
    if status != 0:
        detail = lib.hs_last_error(handle).decode() if handle else ""
        raise SamplerError(f"{what}: {lib.hs_status_string(status).decode()} ({status}) {detail}")
