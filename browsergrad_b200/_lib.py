"""ctypes binding of ``libbgcuda.so`` (declarations in ``include/bgcuda.h``).

The library is built in-tree by ``browsergrad_b200/csrc/Makefile`` (``__graft_entry__.build()``).
There is no CPU fallback: if the shared object is missing, or no sm_100 device is present when a
bridge is created, the error is raised to the caller.
"""
from __future__ import annotations

import ctypes as C
import os

MAX_RANK = 8
MAX_STEP_INPUTS = 8
REF_NONE = -(2 ** 31)

DTYPES = ("float16", "float32", "float64", "int8", "int16", "int32", "int64",
          "uint8", "uint16", "uint32", "uint64", "bool", "bfloat16")
DTYPE_CODE = {n: i for i, n in enumerate(DTYPES)}
DTYPE_SIZE = {"float16": 2, "float32": 4, "float64": 8, "int8": 1, "int16": 2, "int32": 4,
              "int64": 8, "uint8": 1, "uint16": 2, "uint32": 4, "uint64": 8, "bool": 1,
              "bfloat16": 2}
OPCODES = ("BUFFER", "LOAD", "CONST", "CAST", "ADD", "MUL", "DIV", "NEG", "EXP", "LOG", "ABS", "SIGN",
           "SIN", "COS", "ISNAN", "CMP", "WHERE", "MATMUL", "REDUCE", "RESHAPE", "PERMUTE",
           "BROADCAST_TO", "LAYER_NORM", "CROSS_ENTROPY", "INDEX", "FUSED_ELEMENTWISE",
           "FUSED_SOFTMAX", "ATTENTION_FORWARD", "TRIL", "TRIU", "FLIP", "CONCAT", "CUMSUM",
           "SORT_INDICES", "TOPK_INDICES", "SCATTER", "SLICE")
OP_CODE = {n: i for i, n in enumerate(OPCODES)}
CMP_CODE = {"eq": 0, "ne": 1, "lt": 2, "le": 3, "gt": 4, "ge": 5}
REDUCE_CODE = {"sum": 0, "max": 1, "min": 2, "mean": 3, "argmax": 4, "argmin": 5, "any": 6, "all": 7, "prod": 8}

STATUS_NAMES = {1: "invalid argument", 2: "unsupported", 3: "CUDA error", 4: "out of device memory",
                5: "unknown handle", 6: "device-side wait timed out", 7: "index out of range"}


class PlanStep(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("rank", C.c_int32), ("n_inputs", C.c_int32),
                ("shape", C.c_int64 * MAX_RANK), ("input_ids", C.c_int32 * MAX_STEP_INPUTS),
                ("iarg", C.c_int64 * MAX_RANK), ("farg", C.c_double * 2),
                ("ext_offset", C.c_int32), ("ext_count", C.c_int32)]


class Plan(C.Structure):
    _fields_ = [("steps", C.POINTER(PlanStep)), ("n_steps", C.c_int32), ("root_id", C.c_int32),
                ("ext", C.POINTER(C.c_int32)), ("n_ext", C.c_int32)]


class PlanInput(C.Structure):
    _fields_ = [("value_id", C.c_int32), ("reserved", C.c_int32), ("handle", C.c_int64),
                ("data", C.c_void_p), ("nbytes", C.c_size_t)]


class ResourceStats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "current_bytes", "peak_bytes", "total_allocated_bytes", "total_released_bytes", "alive_handles",
        "logical_tensor_plan_peak_bytes", "kernel_launches", "plan_cache_hits", "plan_cache_misses")]


class ProfileEntry(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("ms", C.c_float), ("launches", C.c_int32)]


# name -> (restype, argtypes); every symbol include/bgcuda.h declares
SIGNATURES = {
    "bg_abi_version": (C.c_int, []),
    "bg_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "bg_destroy": (C.c_int, [C.c_void_p]),
    "bg_last_error": (C.c_char_p, [C.c_void_p]),
    "bg_set_option": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int64]),
    "bg_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_int64), C.c_int, C.c_int,
                            C.POINTER(C.c_int64)]),
    "bg_materialize": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t]),
    "bg_release": (C.c_int, [C.c_void_p, C.c_int64]),
    "bg_handle_nbytes": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_int64)]),
    "bg_matmul": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                            C.POINTER(C.c_int64)]),
    "bg_fused_elementwise": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int, C.POINTER(C.c_int32), C.c_int,
                                       C.POINTER(C.c_int64), C.c_int, C.c_int, C.POINTER(C.c_int64)]),
    "bg_cast": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_int64), C.c_int,
                          C.POINTER(C.c_int64)]),
    "bg_flash_attention": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.POINTER(C.c_int64),
                                     C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_double, C.c_int,
                                     C.POINTER(C.c_int64)]),
    "bg_run_tensor_plan": (C.c_int, [C.c_void_p, C.POINTER(Plan), C.POINTER(PlanInput), C.c_int, C.c_void_p,
                                     C.c_size_t]),
    "bg_run_tensor_plan_resident": (C.c_int, [C.c_void_p, C.POINTER(Plan), C.POINTER(PlanInput), C.c_int,
                                              C.POINTER(C.c_int64)]),
    "bg_alive_handle_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
    "bg_resource_snapshot": (C.c_int, [C.c_void_p, C.POINTER(ResourceStats)]),
    "bg_flush_profiles": (C.c_int, [C.c_void_p, C.POINTER(ProfileEntry), C.c_int, C.POINTER(C.c_int)]),
    "bg_last_plan_trace": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "bg_compile_plan_dry": (C.c_int, [C.POINTER(Plan), C.c_int, C.c_char_p, C.c_size_t]),
    "bg_cross_entropy_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                                           C.c_int64, C.c_void_p, C.c_char_p, C.c_size_t]),
    "bg_selftest_wait_timeout": (C.c_int, [C.c_void_p, C.c_int64]),
    "bg_alloc": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int, C.c_int, C.POINTER(C.c_int64)]),
    "bg_stream": (C.c_void_p, [C.c_void_p]),
    "bg_device_pointer": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p)]),
}

_LIB = None


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libbgcuda.so")


def load() -> C.CDLL:
    """Load the shared library and bind every declared symbol.  Raises if it was not built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"CUDA bridge: {path} is missing. Build it with `make -C browsergrad_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`); there is no CPU fallback.")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib
