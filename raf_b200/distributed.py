"""Python mirror of ``raf.distributed`` for the ZeRO path: DistConfig, the global
communicator and the collective wrappers (``python/raf/distributed/{config,
communicator,op}.py``).  Collectives forward to the NCCL entry points of the C
ABI on the communication stream; there is no host implementation.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _lib
from ._lib import check
from .op import _check_cuda, dtype_code, stream_ptr


@dataclass
class DistConfig:
    """include/raf/dist_config.h:17-35 (same field names and defaults)."""
    enable_data_parallel: bool = False
    zero_opt_level: int = 0
    enable_auto_dp_profiling: bool = False
    auto_dp_profiling_start_iter: int = 2
    auto_dp_profiling_end_iter: int = 4
    group_bucket_size: int = 5000000000  # in elements

    def dumps(self):
        return dict(self.__dict__)

    def loads(self, config_dict):
        for key, val in config_dict.items():
            if not hasattr(self, key):
                raise KeyError(key)
            setattr(self, key, val)


_config = DistConfig()
_comm: Optional["Communicator"] = None
_comm_stream = {}


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


def comm_stream(device=None) -> torch.cuda.Stream:
    """The communication stream (tag CudaCommunicate = 4, include/raf/stream_pool.h:40)."""
    device = torch.cuda.current_device() if device is None else device
    if device not in _comm_stream:
        _comm_stream[device] = torch.cuda.Stream(device=device)
    return _comm_stream[device]


def _reject_rank_list(rank_list):
    if rank_list:
        raise NotImplementedError("sub-communicators (rank_list) are outside the ZeRO path")


def allreduce(x, computation="sum", rank_list=None, stream=None):
    """raf.op._allreduce: in place on every tensor of x (TRAFInplaceUpdate {0:0})."""
    _reject_rank_list(rank_list)
    is_list = isinstance(x, (tuple, list))
    xs = list(x) if is_list else [x]
    comm = get_communicator()
    lib = _lib.load()
    for t in xs:
        _check_cuda(t)
        check(lib.rafb200_allreduce(comm.handle, t.data_ptr(), t.data_ptr(), t.numel(),
                                    dtype_code(t.dtype), computation.encode(), stream_ptr(stream)))
    return xs if is_list else xs[0]


def reduce_scatter(x, computation="sum", rank_list=None, stream=None):
    """raf.op._reduce_scatter: dim 0 is split over ranks (must divide)."""
    _reject_rank_list(rank_list)
    return group_reduce_scatter([x], computation, stream=stream)[0]


def group_reduce_scatter(tensor_list, computation="sum", stream=None):
    """raf.op._group_reduce_scatter: one grouped launch for the whole list."""
    comm = get_communicator()
    outs = []
    for t in tensor_list:
        _check_cuda(t)
        if t.shape[0] % comm.size != 0:
            raise ValueError("reduce_scatter: dim 0 must be divisible by the communicator size")
        outs.append(torch.empty((t.shape[0] // comm.size,) + tuple(t.shape[1:]), dtype=t.dtype,
                                device=t.device))
    if tensor_list:
        check(_lib.load().rafb200_group_reduce_scatter(
            comm.handle, len(tensor_list), _lib.ptr_array([t.data_ptr() for t in tensor_list]),
            _lib.ptr_array([t.data_ptr() for t in outs]), _lib.i64_array([t.numel() for t in outs]),
            dtype_code(tensor_list[0].dtype), computation.encode(), stream_ptr(stream)))
    return outs


def allgather(x, axis=0, rank_list=None, stream=None):
    """raf.distributed.allgather: concatenation across ranks on ``axis``
    (NCCL gathers on axis 0; other axes are swapped in and out as the reference does)."""
    _reject_rank_list(rank_list)
    is_list = isinstance(x, (tuple, list))
    xs = list(x) if is_list else [x]
    comm = get_communicator()
    ins = [t if axis == 0 else t.transpose(0, axis).contiguous() for t in xs]
    outs = [torch.empty((t.shape[0] * comm.size,) + tuple(t.shape[1:]), dtype=t.dtype,
                        device=t.device) for t in ins]
    group_allgather(ins, 0, outs, stream=stream)
    outs = [o if axis == 0 else o.transpose(0, axis).contiguous() for o in outs]
    return outs if is_list else outs[0]


def group_allgather(tensor_list, axis, out, stream=None):
    """raf.op._group_allgather: writes into the caller's ``out`` tensors (TRAFInplaceUpdate {2:0})."""
    if axis != 0:
        raise NotImplementedError("group_allgather gathers on axis 0, as NCCL does")
    comm = get_communicator()
    assert len(tensor_list) == len(out)
    for t, o in zip(tensor_list, out):
        _check_cuda(t, o)
        assert o.numel() == t.numel() * comm.size and o.dtype == t.dtype
    if tensor_list:
        check(_lib.load().rafb200_group_allgather(
            comm.handle, len(tensor_list), _lib.ptr_array([t.data_ptr() for t in tensor_list]),
            _lib.ptr_array([t.data_ptr() for t in out]),
            _lib.i64_array([t.numel() for t in tensor_list]), dtype_code(tensor_list[0].dtype),
            stream_ptr(stream)))
    return out
