"""ctypes binding of the C ABI in include/battn.h.  Loads the in-tree libbattn.so; raises if it
has not been built (there is no fallback implementation)."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbattn.so")

IPC_HANDLE_BYTES = 64
OK, ERR_ARG, ERR_CAPACITY, ERR_CUDA, ERR_DEVICE = 0, 1, 2, 3, 4
DEV_BAD_POSITION, DEV_WAIT_TIMEOUT = 1, 2
STATUS_NAMES = {0: "BATTN_OK", 1: "BATTN_ERR_ARG", 2: "BATTN_ERR_CAPACITY", 3: "BATTN_ERR_CUDA",
                4: "BATTN_ERR_DEVICE"}


class BattnError(RuntimeError):
    def __init__(self, fn: str, code: int, cuda: int = 0):
        self.code, self.cuda = code, cuda
        super().__init__(f"{fn} -> {STATUS_NAMES.get(code, code)}" + (f" (cudaError {cuda})" if cuda else ""))


class CGeom(C.Structure):
    _fields_ = [("n_head", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int), ("window", C.c_int),
                ("slot_ctx", C.c_int), ("n_slots", C.c_int), ("q_dtype", C.c_int),
                ("out_dtype", C.c_int), ("softmax_scale", C.c_float)]


class CPages(C.Structure):
    """battn_pages: a paged cache of one full-causal layer (pool pointers, the device-resident page table)."""
    _fields_ = [("pool_k", C.c_void_p), ("pool_v", C.c_void_p), ("table", C.c_void_p),
                ("n_pages", C.c_int), ("n_tables", C.c_int), ("max_pages", C.c_int), ("page_len", C.c_int)]


_P, _I, _SZP = C.c_void_p, C.c_int, C.POINTER(C.c_size_t)
_PG = C.POINTER(CPages)

# name -> (restype, argtypes); exactly the symbols include/battn.h declares
SIGNATURES = {
    "battn_version": (_I, []),
    "battn_init": (_I, [C.POINTER(CGeom), _I, C.POINTER(_P)]),
    "battn_destroy": (_I, [_P]),
    "battn_kv_layer_bytes": (_I, [_P, _I, _SZP]),
    "battn_workspace_bytes": (_I, [_P, _I, _I, _SZP]),
    "battn_call_workspace_bytes": (_I, [C.POINTER(CGeom), _I, _I, _I, _SZP]),
    "battn_exact_workspace_bytes": (_I, [_P, _I, _I, _I, _SZP]),
    "battn_kv_append": (_I, [_P] * 8 + [_I, _I, _I, _P]),
    "battn_kv_copy_prefix": (_I, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "battn_qkv_prep": (_I, [_P] * 8 + [_I] + [_P] * 5 + [_I, _I, _I, _P]),
    "battn_rope_tables": (_I, [_P] * 4 + [_I, _I, _P]),
    "battn_decode": (_I, [_P] * 9 + [_I, _I, _P]),
    "battn_decode_append": (_I, [_P] * 11 + [_I, _I, _P]),
    "battn_qkv_decode": (_I, [_P] * 8 + [_I] + [_P] * 6 + [_I, _I, _P]),
    "battn_decode_noalloc": (_I, [_P] * 8 + [_I, _I, _P]),
    "battn_verify": (_I, [_P] * 9 + [_I, _I, _I, _P]),
    "battn_prefill": (_I, [_P] * 7 + [_I, _I, _P]),
    "battn_gate_norm": (_I, [_P] * 8 + [_I, _P]),
    "battn_prefill_gate_norm": (_I, [_P] * 12 + [_I, _I, _P]),
    "battn_attend_exact": (_I, [_P] * 9 + [_I, _I, _I, _I, _P]),
    "battn_partials": (_I, [_P] * 9 + [_I, _I, _I, _P]),
    "battn_merge": (_I, [_P, _P, _P, _I, _I, _P]),
    "battn_set_early_kv_stream": (_I, [_P, _I]),
    "battn_pages_pool_bytes": (_I, [_P, _I, _I, _SZP]),
    "battn_pages_copy": (_I, [_P, _PG, _I, _I, _P]),
    "battn_kv_append_paged": (_I, [_P, _PG] + [_P] * 5 + [_I, _I, _P]),
    "battn_qkv_prep_paged": (_I, [_P] * 8 + [_I, _PG] + [_P] * 3 + [_I, _I, _P]),
    "battn_decode_paged": (_I, [_P, _P, _P, _PG] + [_P] * 4 + [_I, _P]),
    "battn_decode_append_paged": (_I, [_P] * 5 + [_PG] + [_P] * 4 + [_I, _P]),
    "battn_qkv_decode_paged": (_I, [_P] * 8 + [_I] + [_PG] + [_P] * 4 + [_I, _P]),
    "battn_verify_paged": (_I, [_P, _P, _P, _PG] + [_P] * 4 + [_I, _I, _P]),
    "battn_prefill_paged": (_I, [_P, _P, _P, _PG, _I, _P, _P, _I, _P]),
    "battn_attend_exact_paged": (_I, [_P, _P, _P, _PG] + [_P] * 4 + [_I, _I, _I, _P]),
    "battn_xchg_create": (_I, [_P, _I, _I, _I, C.POINTER(_P), _P]),
    "battn_xchg_connect": (_I, [_P, _P]),
    "battn_xchg_area": (_I, [_P, C.POINTER(_P), _SZP]),
    "battn_xchg_connect_ptrs": (_I, [_P, C.POINTER(_P)]),
    "battn_xchg_set_wait_polls": (_I, [_P, C.c_uint]),
    "battn_xchg_destroy": (_I, [_P]),
    "battn_partials_push": (_I, [_P] * 10 + [_I, _I, _I, _P, _I, _P]),
    "battn_merge_wait": (_I, [_P, _P, _P, _I, _P, _P]),
    "battn_device_status": (_I, [_P, C.POINTER(_I), _I]),
    "battn_selftest_wait_timeout": (_I, [_P, C.c_uint, _P]),
    "battn_profile_start": (_I, [_P, _I]),
    "battn_profile_stop": (_I, [_P, C.POINTER(C.c_float), _I, C.POINTER(_I)]),
    "battn_last_cuda_error": (_I, [_P]),
    "battn_launch_count": (C.c_longlong, [_P]),
}

_lib = None


def load():
    """dlopen the in-tree library and attach prototypes.  Raises FileNotFoundError when the CUDA
    library was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python bruce-engine_b200/build.py` "
                "(the attention path has no non-CUDA implementation)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)      # AttributeError if the header and the library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
