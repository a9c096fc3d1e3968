"""numpy front end of the CPU oracle (test infrastructure, never the product path).

Loads ``libzero_oracle.so`` (built from ``zero_oracle.c`` by ``oracle/Makefile``)
and adds the integer / collective restatements that are simplest in numpy.
Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module.

bf16 arrays are carried as ``numpy.uint16`` bit patterns (numpy has no bf16);
fp16 arrays are ``numpy.float16``.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess

import numpy as np

F32, F16, BF16 = 0, 1, 2
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libzero_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C restatement (gcc, OpenMP, no fp contraction)."""
    src = os.path.join(_HERE, "zero_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libzero_oracle.so"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_bf16_to_f32.restype = C.c_float
        L.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_bf16.restype = C.c_uint16
        L.oracle_f32_to_bf16.argtypes = [C.c_float]
        L.oracle_cast.restype = None
        L.oracle_cast.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64]
        L.oracle_sgd.restype = None
        L.oracle_sgd.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_float,
                                 C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_int]
        L.oracle_l2norm_ref_order.restype = C.c_float
        L.oracle_l2norm_ref_order.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_int, C.c_int]
        L.oracle_l2norm_f64.restype = C.c_double
        L.oracle_l2norm_f64.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_float]
        L.oracle_lans_bias_corrections.restype = None
        L.oracle_lans_bias_corrections.argtypes = [C.c_float, C.c_float, C.c_int, C.c_int,
                                                   C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.oracle_lans.restype = None
        L.oracle_lans.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float, C.c_float,
                                  C.c_int, C.c_float, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int,
                                  C.c_void_p, C.c_int, C.c_void_p]
        L.oracle_adam.restype = None
        L.oracle_adam.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_int, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int,
                                  C.c_float, C.c_int, C.c_float, C.c_void_p, C.c_int]
        L.oracle_shard_rows.restype = C.c_int64
        L.oracle_shard_rows.argtypes = [C.c_int64, C.c_int]
        L.oracle_plan_buckets.restype = C.c_int
        L.oracle_plan_buckets.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p]
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_num_threads.restype = C.c_int
        L.oracle_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def num_threads() -> int:
    return lib().oracle_num_threads()


def use_all_host_threads() -> int:
    """Thread count = the cores this process may run on, whatever OMP_NUM_THREADS a
    launcher exported (torch.distributed.run sets it to 1); returns the count in use."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover
        n = os.cpu_count() or 1
    return lib().oracle_set_num_threads(n)


# --------------------------------------------------------------------------- dtypes
def np_dtype(code: int):
    return {F32: np.float32, F16: np.float16, BF16: np.uint16}[code]


def code_of(arr: np.ndarray, bf16: bool = False) -> int:
    if arr.dtype == np.float32:
        return F32
    if arr.dtype == np.float16:
        return F16
    if arr.dtype == np.uint16:
        return BF16
    raise TypeError(f"unsupported dtype {arr.dtype}")


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def cast(src: np.ndarray, dst_code: int) -> np.ndarray:
    """raf.op.cast (round to nearest even)."""
    src = np.ascontiguousarray(src)
    dst = np.empty(src.shape, np_dtype(dst_code))
    lib().oracle_cast(_ptr(src), code_of(src), _ptr(dst), dst_code, src.size)
    return dst


def to_f32(a: np.ndarray) -> np.ndarray:
    return a if a.dtype == np.float32 else cast(a, F32)


# --------------------------------------------------------------------------- optimizers
def sgd(x, dx, v, lr, mu, weight_decay=0.0, grad_scale=1.0, out_code=None):
    """In-place raf.op.sgd on fp32 ``x`` and ``v``; returns cast(x1) when out_code is given."""
    assert x.dtype == np.float32 and v.dtype == np.float32 and x.size == dx.size == v.size
    out = np.empty(x.shape, np_dtype(out_code)) if out_code is not None else None
    lib().oracle_sgd(_ptr(x), _ptr(dx), code_of(dx), _ptr(v), x.size, lr, mu, weight_decay,
                     grad_scale, _ptr(out) if out is not None else None, out_code or 0)
    return out


def bias_corrections(beta1, beta2, step, bias_correction=1):
    a, b = C.c_float(), C.c_float()
    lib().oracle_lans_bias_corrections(beta1, beta2, step, int(bias_correction), C.byref(a), C.byref(b))
    return a.value, b.value


def _ptr_array(arrs):
    return (C.c_void_p * len(arrs))(*[_ptr(a) for a in arrs])


def lans(gs, ps, ms, vs, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, bias_correction=1,
         weight_decay=0.01, grad_averaging=1, mode=1, normalize_grad=1, grad_scale=1.0,
         norm_mode=0, out_code=None):
    """In-place raf.op.lans over tensor lists; returns (outs or None, norms[k,4])."""
    k = len(gs)
    assert k == len(ps) == len(ms) == len(vs)
    gcode = code_of(gs[0]) if k else F32
    numel = np.array([p.size for p in ps], np.int64)
    outs = [np.empty(p.shape, np_dtype(out_code)) for p in ps] if out_code is not None else None
    norms = np.zeros((k, 4), np.float32)
    lib().oracle_lans(k, _ptr_array(gs), gcode, _ptr_array(ps), _ptr_array(ms), _ptr_array(vs),
                      _ptr(numel), int(step), lr, beta1, beta2, eps, int(bias_correction),
                      weight_decay, int(grad_averaging), int(mode), int(normalize_grad), grad_scale,
                      norm_mode, _ptr_array(outs) if outs is not None else None, out_code or 0,
                      _ptr(norms))
    return outs, norms


def adam(g, p, m, v, step, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, bias_correction=1,
         weight_decay=0.1, mode=1, grad_scale=1.0, out_code=None):
    """In-place Adam (parity unpinned: defined by this repository)."""
    out = np.empty(p.shape, np_dtype(out_code)) if out_code is not None else None
    lib().oracle_adam(_ptr(g), code_of(g), _ptr(p), _ptr(m), _ptr(v), p.size, int(step), lr, beta1,
                      beta2, eps, int(bias_correction), weight_decay, int(mode), grad_scale,
                      _ptr(out) if out is not None else None, out_code or 0)
    return out


def l2norm_ref_order(x, scale=1.0, max_chunks=0, fused=False) -> float:
    x = np.ascontiguousarray(x)
    return lib().oracle_l2norm_ref_order(_ptr(x), code_of(x), x.size, scale, max_chunks, int(fused))


def l2norm_f64(x, scale=1.0) -> float:
    x = np.ascontiguousarray(x)
    return lib().oracle_l2norm_f64(_ptr(x), code_of(x), x.size, scale)


# --------------------------------------------------------------------------- geometry
def shard_rows(d0: int, n_part: int) -> int:
    return lib().oracle_shard_rows(d0, n_part)


def plan_buckets(sizes, bucket_size: int, rule: int = 0):
    sizes = np.asarray(sizes, np.int64)
    out = np.zeros(len(sizes), np.int32)
    nb = lib().oracle_plan_buckets(_ptr(sizes), len(sizes), bucket_size, rule, _ptr(out))
    return nb, out


def split_with_padding(inp: np.ndarray, n_part: int):
    """python/raf/optim/utils.py:35-52: zero-pad dim 0 to a multiple of n_part, split evenly."""
    part = math.ceil(inp.shape[0] / n_part)
    padded = part * n_part
    if padded > inp.shape[0]:
        width = [(0, 0) for _ in inp.shape]
        width[0] = (0, padded - inp.shape[0])
        inp = np.pad(inp, width)
    return np.split(inp, n_part)


# --------------------------------------------------------------------------- collectives
# Semantics of src/op/declare/collective_comm.cc:26-158 and the NCCL calls of
# src/op/dialect/nccl/nccl.cc:40-399, simulated for all ranks in one process.
# Reductions are carried out in the tensor's own dtype, left to right over ranks
# (exact for the integer-valued data the reference's tests use).
def _reduce(parts, computation):
    acc = parts[0].copy()
    for x in parts[1:]:
        if computation in ("sum", "avg"):
            acc = (acc + x).astype(acc.dtype)
        elif computation == "prod":
            acc = (acc * x).astype(acc.dtype)
        elif computation == "min":
            acc = np.minimum(acc, x)
        elif computation == "max":
            acc = np.maximum(acc, x)
        else:
            raise ValueError(f"Invalid computation {computation}")
    if computation == "avg":
        acc = (acc / acc.dtype.type(len(parts))).astype(acc.dtype)
    return acc


def allreduce(per_rank, computation="sum"):
    """per_rank[r] = that rank's tensor; every rank receives the reduction."""
    red = _reduce(per_rank, computation)
    return [red.copy() for _ in per_rank]


def reduce_scatter(per_rank, computation="sum"):
    """Rank r receives rows [r*d0/n, (r+1)*d0/n) of the reduction (dim 0 must divide)."""
    n = len(per_rank)
    assert per_rank[0].shape[0] % n == 0, "dim 0 must be divisible by the communicator size"
    red = _reduce(per_rank, computation)
    return [s.copy() for s in np.split(red, n)]


def allgather(per_rank, axis=0):
    full = np.concatenate(per_rank, axis=axis)
    return [full.copy() for _ in per_rank]
