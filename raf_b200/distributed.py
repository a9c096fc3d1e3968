"""Python mirror of ``raf.distributed`` for the ZeRO path: DistConfig, the global
communicator and the collective wrappers (``python/raf/distributed/{config,
communicator,op}.py``).  Collectives forward to the NCCL entry points of the C
ABI on the communication stream; there is no host implementation.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch

from . import _lib
from ._lib import check
from .op import _check_cuda, stream_ptr
from .op import dtype_code as _float_code

# collectives also move the integer and double types of the reference's NCCL map
# (src/op/dialect/nccl/communication_utils.h:31-48)
_COMM_CODES = {torch.float64: 3, torch.int8: 4, torch.uint8: 5, torch.int64: 6}


def dtype_code(dtype) -> int:
    return _COMM_CODES[dtype] if dtype in _COMM_CODES else _float_code(dtype)


class _CDistConfig(C.Structure):
    _fields_ = [("scheduling_param", C.c_int), ("iteration", C.c_int),
                ("enable_data_parallel", C.c_int), ("zero_opt_level", C.c_int),
                ("enable_auto_dp_profiling", C.c_int), ("auto_dp_profiling_start_iter", C.c_int),
                ("auto_dp_profiling_end_iter", C.c_int), ("group_bucket_size", C.c_int64)]


class DistConfig:
    """include/raf/dist_config.h:17-35 (same field names and defaults).  The values live in
    the library's process-wide record, the one its C++ operator glue reads, so that setting
    ``zero_opt_level`` here is seen there as DistConfig::Global() is in the reference."""
    _names = [f[0] for f in _CDistConfig._fields_]
    _bools = ("enable_data_parallel", "enable_auto_dp_profiling")

    def _read(self):
        c = _CDistConfig()
        check(_lib.load().rafb200_dist_config_get(C.byref(c)))
        return c

    def __getattr__(self, name):
        if name in DistConfig._names:
            v = getattr(self._read(), name)
            return bool(v) if name in DistConfig._bools else int(v)
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if name not in DistConfig._names:
            raise AttributeError(name)
        c = self._read()
        setattr(c, name, int(value))
        check(_lib.load().rafb200_dist_config_set(C.byref(c)))

    def dumps(self):
        c = self._read()
        return {n: (bool(getattr(c, n)) if n in DistConfig._bools else int(getattr(c, n)))
                for n in DistConfig._names}

    def loads(self, config_dict):
        for key in config_dict:
            if key not in DistConfig._names:
                raise KeyError(key)
        for key, val in config_dict.items():
            setattr(self, key, val)


_config = DistConfig()
_comm: Optional["Communicator"] = None


def get_config() -> DistConfig:
    return _config


class Communicator:
    """The global NCCL communicator (one process per GPU).

    ``size``/``rank``/``local_rank`` mirror CommunicatorObj (include/raf/communicator.h:52-62).
    """

    def __init__(self, size=1, rank=0, local_rank=0, store_path=None, unique_id=None,
                 timeout_ms=60000):
        self.size, self.rank, self.local_rank = size, rank, local_rank
        self.local_size = size
        self.world_size, self.world_rank, self.root_rank = size, rank, 0
        h = C.c_void_p()
        lib = _lib.load()
        if unique_id is not None:
            buf = (C.c_uint8 * 128).from_buffer_copy(bytes(unique_id))
            check(lib.rafb200_comm_create_with_id(size, rank, local_rank, buf, timeout_ms, C.byref(h)))
        else:
            path = store_path.encode() if store_path else None
            check(lib.rafb200_comm_create(size, rank, local_rank, path, timeout_ms, C.byref(h)))
        self.handle = h

    def check(self):
        check(_lib.load().rafb200_comm_check(self.handle))

    def close(self):
        if self.handle:
            torch.cuda.synchronize()
            check(_lib.load().rafb200_comm_destroy(self.handle))
            self.handle = None


def unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    check(_lib.load().rafb200_unique_id(buf))
    return bytes(buf)


def set_communicator(comm: Optional[Communicator]):
    global _comm
    _comm = comm


def get_communicator() -> Communicator:
    """Global communicator; a world of one (the reference's VoidCommunicator) by default."""
    global _comm
    if _comm is None:
        _comm = Communicator(1, 0, torch.cuda.current_device())
    return _comm


def init_from_env(timeout_ms=120000) -> Communicator:
    """Create the global communicator from RANK / WORLD_SIZE / LOCAL_RANK (torchrun style);
    the id travels through the file store at $RAF_FILE_STORE_PATH as in the reference."""
    size = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    comm = Communicator(size, rank, local_rank, store_path=os.environ.get("RAF_FILE_STORE_PATH"),
                        timeout_ms=timeout_ms)
    set_communicator(comm)
    return comm


STREAM_TAGS = {"compute": 1, "mem_cpy_cpu_to_cuda": 2, "mem_cpy_cuda_to_cpu": 3, "communicate": 4,
               "fuse": 5, "defuse": 6}  # include/raf/stream_pool.h:35-44


def get_stream(tag="compute", index=0, device=None) -> torch.cuda.ExternalStream:
    """Stream::Get(device, tag, index) (src/impl/stream_pool.cc:53-98): the library's stream
    for the tag, created on first use; the same arguments give the same stream."""
    device = torch.cuda.current_device() if device is None else device
    h = C.c_void_p()
    check(_lib.load().rafb200_stream_get(int(device), STREAM_TAGS[tag] if isinstance(tag, str) else int(tag),
                                         int(index), C.byref(h)))
    return torch.cuda.ExternalStream(h.value, device=device)


def comm_stream(device=None) -> torch.cuda.ExternalStream:
    """The communication stream (tag CudaCommunicate = 4, include/raf/stream_pool.h:40)."""
    return get_stream("communicate", 0, device)


def _group_comm(rank_list):
    """(handle, size, rank) of the communicator a collective with this ``rank_list`` runs on:
    the global one when rank_list is empty, else the group that names this rank - or a world
    of one when none does (src/distributed/common/communicator.cc:21-84)."""
    comm = get_communicator()
    if not rank_list:
        return comm.handle, comm.size, comm.rank
    groups = [[int(r) for r in g] for g in rank_list]
    sizes = (C.c_int * len(groups))(*[len(g) for g in groups])
    flat = [r for g in groups for r in g]
    ranks = (C.c_int * len(flat))(*flat)
    sub = C.c_void_p()
    lib = _lib.load()
    check(lib.rafb200_comm_sub(comm.handle, len(groups), sizes, ranks, C.byref(sub)))
    return sub, lib.rafb200_comm_size(sub), lib.rafb200_comm_rank(sub)


def allreduce(x, computation="sum", rank_list=None, stream=None):
    """raf.op._allreduce: in place on every tensor of x (TRAFInplaceUpdate {0:0})."""
    is_list = isinstance(x, (tuple, list))
    xs = list(x) if is_list else [x]
    handle, _, _ = _group_comm(rank_list)
    lib = _lib.load()
    for t in xs:
        _check_cuda(t)
        check(lib.rafb200_allreduce(handle, t.data_ptr(), t.data_ptr(), t.numel(),
                                    dtype_code(t.dtype), computation.encode(), stream_ptr(stream)))
    return xs if is_list else xs[0]


def reduce_scatter(x, computation="sum", rank_list=None, stream=None):
    """raf.op._reduce_scatter: dim 0 is split over the ranks of the group (must divide)."""
    return group_reduce_scatter([x], computation, rank_list=rank_list, stream=stream)[0]


def group_reduce_scatter(tensor_list, computation="sum", rank_list=None, stream=None):
    """raf.op._group_reduce_scatter: one grouped launch for the whole list."""
    handle, size, _ = _group_comm(rank_list)
    outs = []
    for t in tensor_list:
        _check_cuda(t)
        if t.shape[0] % size != 0:
            raise ValueError("reduce_scatter: dim 0 must be divisible by the communicator size")
        outs.append(torch.empty((t.shape[0] // size,) + tuple(t.shape[1:]), dtype=t.dtype,
                                device=t.device))
    if tensor_list:
        check(_lib.load().rafb200_group_reduce_scatter(
            handle, len(tensor_list), _lib.ptr_array([t.data_ptr() for t in tensor_list]),
            _lib.ptr_array([t.data_ptr() for t in outs]), _lib.i64_array([t.numel() for t in outs]),
            dtype_code(tensor_list[0].dtype), computation.encode(), stream_ptr(stream)))
    return outs


def allgather(x, axis=0, rank_list=None, stream=None):
    """raf.distributed.allgather: concatenation across the ranks of the group on ``axis``
    (NCCL gathers on axis 0; other axes are swapped in and out as the reference does)."""
    is_list = isinstance(x, (tuple, list))
    xs = list(x) if is_list else [x]
    _, size, _ = _group_comm(rank_list)
    ins = [t if axis == 0 else t.transpose(0, axis).contiguous() for t in xs]
    outs = [torch.empty((t.shape[0] * size,) + tuple(t.shape[1:]), dtype=t.dtype,
                        device=t.device) for t in ins]
    group_allgather(ins, 0, outs, rank_list=rank_list, stream=stream)
    outs = [o if axis == 0 else o.transpose(0, axis).contiguous() for o in outs]
    return outs if is_list else outs[0]


def group_allgather(tensor_list, axis, out, rank_list=None, stream=None):
    """raf.op._group_allgather: writes into the caller's ``out`` tensors (TRAFInplaceUpdate {2:0})."""
    if axis != 0:
        raise NotImplementedError("group_allgather gathers on axis 0, as NCCL does")
    handle, size, _ = _group_comm(rank_list)
    assert len(tensor_list) == len(out)
    for t, o in zip(tensor_list, out):
        _check_cuda(t, o)
        assert o.numel() == t.numel() * size and o.dtype == t.dtype
    if tensor_list:
        check(_lib.load().rafb200_group_allgather(
            handle, len(tensor_list), _lib.ptr_array([t.data_ptr() for t in tensor_list]),
            _lib.ptr_array([t.data_ptr() for t in out]),
            _lib.i64_array([t.numel() for t in tensor_list]), dtype_code(tensor_list[0].dtype),
            stream_ptr(stream)))
    return out
