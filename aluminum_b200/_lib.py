"""ctypes binding of ``libal_b200.so`` (the C interface in ``include/al/al_c.h``).

The library is built in-tree on first use when it is missing.  Every wrapper
raises :class:`AlError` with the library's own message when a call fails, so a
missing or broken native library can never be mistaken for a working fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "lib" / "libal_b200.so"
_lock = threading.Lock()
_lib = None


class AlError(RuntimeError):
    """A call into the native library failed."""


# numeric codes shared with the C++ enums ------------------------------------------------
DTYPES = {"int8": 0, "uint8": 1, "int16": 2, "uint16": 3, "int32": 4, "uint32": 5, "int64": 6, "uint64": 7,
          "float16": 8, "bfloat16": 9, "float32": 10, "float64": 11}
DTYPE_SIZES = {0: 1, 1: 1, 2: 2, 3: 2, 4: 4, 5: 4, 6: 8, 7: 8, 8: 2, 9: 2, 10: 4, 11: 8}
OPS = {"sum": 0, "prod": 1, "min": 2, "max": 3, "lor": 4, "land": 5, "lxor": 6, "bor": 7, "band": 8, "bxor": 9,
       "avg": 10}
KINDS = {"allreduce": 0, "reduce": 1, "reduce_scatter": 2, "allgather": 3, "alltoall": 4, "bcast": 5, "gather": 6,
         "scatter": 7, "barrier": 8}
ALGOS = {"auto": 0, "one_shot": 1, "two_shot": 2, "nvls": 3, "ll": 4}
PATHS = {"auto": 0, "staged": 1, "window": 2, "ll": 3, "nvls": 4}  # data path of every collective but allreduce
COMM_STREAM = C.c_void_p(-1 & (2 ** 64 - 1))


def lib_path() -> Path:
    return _LIB_PATH


def _declare(lib) -> None:
    vp, sz, i, d, u64p = C.c_void_p, C.c_size_t, C.c_int, C.c_double, C.POINTER(C.c_uint64)
    szp, ip, vpp = C.POINTER(C.c_size_t), C.POINTER(C.c_int), C.POINTER(C.c_void_p)
    sig = {
        "al_last_error": (C.c_char_p, []),
        "al_init": (i, []), "al_finalize": (i, []), "al_initialized": (i, []),
        "al_world_rank": (i, []), "al_world_size": (i, []), "al_world_local_rank": (i, []),
        "al_world_local_size": (i, []), "al_world_num_nodes": (i, []), "al_world_peer_alive": (i, [i]), "al_world_node_index": (i, []), "al_cuda_available": (i, []),
        "al_info": (i, [C.c_char_p, sz]),
        "al_set_tuning": (i, [C.c_char_p, d]), "al_get_tuning": (d, [C.c_char_p]),
        "al_trace_enable": (None, [i]), "al_trace_snapshot": (i, [C.c_char_p, sz]), "al_trace_clear": (None, []),
        "al_host_comm_create": (vp, []), "al_host_comm_split": (vp, [vp, i, i]), "al_host_comm_destroy": (None, [vp]),
        "al_host_comm_rank": (i, [vp]), "al_host_comm_size": (i, [vp]),
        "al_host_comm_local_rank": (i, [vp]), "al_host_comm_local_size": (i, [vp]), "al_host_comm_local": (vp, [vp]),
        "al_host_comm_stats": (i, [vp, u64p]), "al_host_comm_abort": (i, [vp, C.c_char_p]),
        "al_dev_comm_abort": (i, [vp, C.c_char_p]),
        "al_host_collective": (i, [vp, i, vp, vp, sz, i, i, i, i, i, szp, szp, szp, szp, vpp]),
        "al_host_p2p": (i, [vp, i, ip, ip, vpp, szp, vpp]),
        "al_host_test": (i, [vpp, ip]), "al_host_wait": (i, [vpp]),
        "al_dev_comm_create": (vp, [vp]), "al_dev_comm_create_emulated": (vp, [i, vp]),
        "al_dev_comm_create_group": (vp, [C.POINTER(C.c_int), i, vp]),
        "al_host_comm_create_group": (vp, [C.POINTER(C.c_int), i]),
        "al_dev_comm_split": (vp, [vp, i, i, vp]), "al_dev_comm_destroy": (None, [vp]),
        "al_dev_comm_rank": (i, [vp]), "al_dev_comm_size": (i, [vp]), "al_dev_comm_nlocal": (i, [vp]),
        "al_dev_comm_has_multicast": (i, [vp]), "al_dev_comm_backing": (C.c_char_p, [vp]),
        "al_dev_comm_set_timeout_ms": (i, [vp, d]), "al_dev_comm_stats": (i, [vp, u64p]),
        "al_dev_comm_status": (i, [vp, u64p]),
        "al_dev_collective": (i, [vp, i, i, vpp, vpp, sz, i, i, i, i, i, i, i, szp, szp, szp, szp, d, i, i, vp, vpp]),
        "al_dev_exchange_rows": (i, [vp, i, vpp, vpp, vpp, vpp, sz, sz, sz, szp, szp, szp, szp, szp, szp, vp, vpp]),
        "al_dev_latency_breakdown": (i, [vp, i, vp, vp, sz, i, i, i, i, i, vp, C.POINTER(C.c_double)]),
        "al_dev_register": (i, [vp, vp, sz]), "al_dev_register_emulated": (i, [vp, vpp, i, sz]),
        "al_dev_unregister": (i, [vp, vp]),
        "al_dev_time_collective": (i, [vp, i, vp, vp, sz, i, i, i, i, vp, C.POINTER(C.c_float)]),
        "al_dev_p2p": (i, [vp, i, ip, ip, ip, vpp, szp, vp, vpp]),
        "al_dev_test": (i, [vpp, ip]), "al_dev_wait": (i, [vpp]),
        "al_dev_check_guards": (i, [vp]), "al_dev_symm_alloc": (vp, [vp, sz]), "al_dev_symm_free": (i, [vp, vp]),
        "al_dev_symm_peer_ptr": (vp, [vp, vp, i]),
        "al_rma_attach": (vp, [vp, vp, i]), "al_rma_detach": (i, [vp, vp, i]),
        "al_rma_put": (i, [vp, vp, i, vp, sz]), "al_rma_get": (i, [vp, vp, i, vp, sz]), "al_rma_notify": (i, [vp, i]), "al_rma_wait": (i, [vp, i]),
        "al_rma_sync": (i, [vp, i]),
        "al_halo_exchange": (i, [vp, vpp, sz, sz, sz, sz, i, i, vp]),
        "al_halo_pack": (i, [vp, vp, sz, sz, sz, sz, sz, i, vp]),
        "al_scale_cast": (i, [vp, i, vp, i, sz, d, vp]),
        "al_sgd_momentum": (i, [vp, vp, vp, sz, C.c_float, C.c_float, C.c_float, C.c_float, i, i, vp]),
        "al_fill_u32": (i, [vp, sz, C.c_uint32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def load():
    """Return the loaded library, building it first if the shared object is absent."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists() or os.environ.get("AL_REBUILD"):
            from . import _build
            _build.build(tools=True)
        if not _LIB_PATH.exists():
            raise AlError(f"native library missing: {_LIB_PATH}")
        lib = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
        _declare(lib)
        _lib = lib
        return lib


def check(rc: int) -> None:
    if rc != 0:
        raise AlError(load().al_last_error().decode(errors="replace"))


def check_ptr(p):
    if not p:
        raise AlError(load().al_last_error().decode(errors="replace"))
    return p


def size_array(values):
    if values is None:
        return None
    arr = (C.c_size_t * len(values))(*[int(v) for v in values])
    return arr
