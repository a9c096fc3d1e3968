"""ctypes binding of libraf_b200.so (the C ABI declared in include/raf_b200.h).

There is no CPU or PyTorch fallback behind these functions: if the shared
library cannot be loaded, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("RAFB200_LIB") or os.path.join(HERE, "libraf_b200.so")  # an installed copy elsewhere

F32, F16, BF16 = 0, 1, 2
OPT_SGD, OPT_ADAM, OPT_LANS = 0, 1, 2

STATUS_NAMES = {
    0: "OK", 1: "INVALID_ARGUMENT", 2: "CUDA_ERROR", 3: "NCCL_ERROR", 4: "TIMEOUT",
    5: "DEVICE_WAIT_EXPIRED", 6: "UNSUPPORTED", 7: "IO_ERROR",
}


class RafB200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"raf_b200 status {status} ({STATUS_NAMES.get(status, '?')}): {message}")
        self.status = status


class Hyper(C.Structure):
    """struct rafb200_hyper."""
    _fields_ = [
        ("optimizer", C.c_int), ("learning_rate", C.c_float), ("mu", C.c_float),
        ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
        ("weight_decay", C.c_float), ("bias_correction", C.c_int), ("grad_averaging", C.c_int),
        ("mode", C.c_int), ("normalize_grad", C.c_int), ("grad_scale", C.c_float),
        ("average", C.c_int),
    ]


_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
_P = C.POINTER

# name -> (restype, argtypes); every symbol include/raf_b200.h declares
SIGNATURES = {
    "rafb200_last_error": (C.c_char_p, []),
    "rafb200_version": (_i, []),
    "rafb200_tensor_list_create": (_i, [_i, _vp, _i, _i, _P(_vp)]),
    "rafb200_tensor_list_bind": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "rafb200_tensor_list_destroy": (_i, [_vp]),
    "rafb200_tensor_list_total_elems": (_i64, [_vp]),
    "rafb200_tensor_list_tune": (_i, [_vp, _i64, _i, _i]),
    "rafb200_sgd": (_i, [_vp, _vp, _i, _vp, _i64, _f, _f, _f, _f, _vp, _i, _vp]),
    "rafb200_sgd_list": (_i, [_vp, _f, _f, _f, _f, _vp]),
    "rafb200_lans_workspace_bytes": (_sz, [_vp]),
    "rafb200_lans": (_i, [_vp, _i, _vp, _f, _f, _f, _f, _i, _f, _i, _i, _i, _f, _vp, _sz, _vp]),
    "rafb200_lans_schedule": (_i, [_i, _vp, _i, _i, _i, _i64, _i, _vp, _sz, _P(_sz)]),
    "rafb200_tensor_list_set_wait_limit": (_i, [_vp, _i]),
    "rafb200_tensor_list_set_lans_items": (_i, [_vp, _vp, _sz]),
    "rafb200_lans_partition": (_i, [_i, _vp, _i, _i, _i, _i64, _i, _vp, _vp, _sz, _P(_sz), _P(_i), _P(_i)]),
    "rafb200_tensor_list_set_symmetric": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "rafb200_lans_status": (_i, [_vp, _vp, _vp, _vp]),
    "rafb200_lans_tensor_static": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i64, _i, _f, _f, _f, _f,
                                        _i, _f, _i, _i, _i, _f, _vp]),
    "rafb200_adam": (_i, [_vp, _i, _vp, _f, _f, _f, _f, _i, _f, _i, _f, _vp]),
    "rafb200_cast": (_i, [_vp, _i, _vp, _i, _i64, _vp]),
    "rafb200_group_cast": (_i, [_i, _vp, _i, _vp, _i, _vp, _vp]),
    "rafb200_fuse_tensor": (_i, [_i, _vp, _vp, _vp, _i, _vp, _vp]),
    "rafb200_defuse_tensor": (_i, [_i, _vp, _vp, _vp, _i, _vp, _vp]),
    "rafb200_comm_create": (_i, [_i, _i, _i, C.c_char_p, _i, _P(_vp)]),
    "rafb200_unique_id": (_i, [_vp]),
    "rafb200_comm_create_with_id": (_i, [_i, _i, _i, _vp, _i, _P(_vp)]),
    "rafb200_store_exchange": (_i, [_i, C.c_char_p, _i, _vp, _sz, _i]),
    "rafb200_comm_adopt": (_i, [_vp, _i, _i, _P(_vp)]),
    "rafb200_comm_destroy": (_i, [_vp]),
    "rafb200_comm_alloc": (_i, [_vp, _sz, _P(_vp)]),
    "rafb200_comm_free": (_i, [_vp, _vp]),
    "rafb200_comm_sub": (_i, [_vp, _i, _vp, _vp, _P(_vp)]),
    "rafb200_dist_config_get": (_i, [_vp]),
    "rafb200_dist_config_set": (_i, [_vp]),
    "rafb200_stream_get": (_i, [_i, _i, _i, _P(_vp)]),
    "rafb200_stream_release_all": (_i, []),
    "rafb200_zero_set_fused": (_i, [_vp, _i]),
    "rafb200_symm_alloc": (_i, [_i, _i, _i, C.c_size_t, C.c_char_p, _i, _i, _P(_vp)]),
    "rafb200_symm_bytes": (C.c_size_t, [_vp]),
    "rafb200_symm_pointers": (_i, [_vp, _vp, _P(_vp)]),
    "rafb200_symm_free": (_i, [_vp]),
    "rafb200_comm_size": (_i, [_vp]),
    "rafb200_comm_rank": (_i, [_vp]),
    "rafb200_comm_check": (_i, [_vp]),
    "rafb200_allreduce": (_i, [_vp, _vp, _vp, _i64, _i, C.c_char_p, _vp]),
    "rafb200_reduce_scatter": (_i, [_vp, _vp, _vp, _i64, _i, C.c_char_p, _vp]),
    "rafb200_group_reduce_scatter": (_i, [_vp, _i, _vp, _vp, _vp, _i, C.c_char_p, _vp]),
    "rafb200_allgather": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "rafb200_group_allgather": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp]),
    "rafb200_plan_create": (_i, [_i, _vp, _vp, _i, _i, _i64, _P(_vp)]),
    "rafb200_plan_destroy": (_i, [_vp]),
    "rafb200_plan_num_buckets": (_i, [_vp]),
    "rafb200_plan_query": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "rafb200_plan_totals": (_i, [_vp, _P(_i64), _P(_i64), _P(_i64)]),
    "rafb200_zero_create": (_i, [_vp, _vp, _i, _i, _i, _P(_vp)]),
    "rafb200_zero_destroy": (_i, [_vp]),
    "rafb200_zero_bind": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "rafb200_zero_step": (_i, [_vp, _P(Hyper), _i, _vp, _vp]),
    "rafb200_zero_flat_bytes": (_i, [_vp, _P(_sz), _P(_sz), _P(_sz)]),
    "rafb200_zero_attach_symmetric": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "rafb200_zero_arena_offsets": (_i, [_vp, _vp, _vp]),
    "rafb200_zero_status": (_i, [_vp]),
    "rafb200_zero_set_stage_mask": (_i, [_vp, _i]),
    "rafb200_zero_set_wait_limit": (_i, [_vp, _i]),
    "rafb200_zero_set_host_output": (_i, [_vp, _i]),
    "rafb200_zero_declare_arena": (_i, [_vp, _vp, _sz]),
    "rafb200_zero_shard_grad": (_i, [_vp, _i, _P(_vp)]),
    "rafb200_zero_launch_counts": (_i, [_vp, _P(_i), _P(_i)]),
    "rafb200_zero_set_update_blocks": (_i, [_vp, _i]),
    "rafb200_zero_step_host": (_i, [_vp, _P(Hyper), _i, _vp, _vp, _vp, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load libraf_b200.so, building it first when it is missing and nvcc is available."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build  # raises when nvcc is missing
        _build.build()
    # torch bundles its own libnccl.so.2; importing it first makes this library
    # resolve NCCL to that same copy instead of pulling a second one into the process.
    import torch  # noqa: F401
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise RafB200Error(status, load().rafb200_last_error().decode("utf-8", "replace"))


def ptr_array(ptrs) -> C.Array:
    return (C.c_void_p * len(ptrs))(*[C.c_void_p(p) if p else None for p in ptrs])


def i64_array(vals) -> C.Array:
    return (C.c_int64 * len(vals))(*[int(v) for v in vals])
