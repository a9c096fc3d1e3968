"""ZeRO plan and step driver bindings."""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import OPT_ADAM, OPT_LANS, OPT_SGD, Hyper, check
from .op import dtype_code, stream_ptr, torch_dtype


def _dim0_row(shape) -> Tuple[int, int]:
    shape = tuple(int(s) for s in shape)
    if len(shape) == 0:
        return 1, 1
    row = 1
    for s in shape[1:]:
        row *= s
    return shape[0], row


class Plan:
    """Shard geometry and buckets of a parameter list (host only; no GPU needed).

    Follows GradientPartitioner / CommGrouper of the reference
    (src/pass/partition_gradient.cc:177-205,289-300; src/pass/group_allgather.cc:110-145).
    """

    def __init__(self, shapes: Sequence[Sequence[int]], n_ranks: int, rank: int, bucket_elems: int):
        self.shapes = [tuple(int(x) for x in s) for s in shapes]
        self.k = len(self.shapes)
        self.n_ranks, self.rank, self.bucket_elems = n_ranks, rank, bucket_elems
        d0r = [_dim0_row(s) for s in self.shapes]
        h = C.c_void_p()
        lib = _lib.load()
        check(lib.rafb200_plan_create(self.k, _lib.i64_array([d for d, _ in d0r]),
                                      _lib.i64_array([r for _, r in d0r]), n_ranks, rank,
                                      int(bucket_elems), C.byref(h)))
        self.handle = h
        rows = np.zeros(self.k, np.int64)
        elems = np.zeros(self.k, np.int64)
        padded = np.zeros(self.k, np.int64)
        bucket = np.zeros(self.k, np.int32)
        check(lib.rafb200_plan_query(h, rows.ctypes.data, elems.ctypes.data, padded.ctypes.data,
                                     bucket.ctypes.data))
        self.shard_rows, self.shard_elems, self.padded_elems, self.bucket_of = rows, elems, padded, bucket
        self.num_buckets = lib.rafb200_plan_num_buckets(h)
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        check(lib.rafb200_plan_totals(h, C.byref(a), C.byref(b), C.byref(c)))
        self.total_elems, self.total_padded, self.total_shard = a.value, b.value, c.value

    def shard_shape(self, i: int) -> Tuple[int, ...]:
        s = self.shapes[i]
        return (int(self.shard_rows[i]),) + s[1:] if len(s) else (1,)

    def close(self):
        if self.handle:
            _lib.load().rafb200_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_hyper(optimizer: str, **kw) -> Hyper:
    opt = {"sgd": OPT_SGD, "adam": OPT_ADAM, "lans": OPT_LANS}[optimizer]
    h = Hyper()
    h.optimizer = opt
    h.learning_rate = kw.get("learning_rate", kw.get("lr", 1e-3))
    h.mu = kw.get("mu", kw.get("momentum", 0.0))
    h.beta1 = kw.get("beta1", 0.9)
    h.beta2 = kw.get("beta2", 0.999)
    h.eps = kw.get("eps", 1e-6)
    h.weight_decay = kw.get("weight_decay", 0.0)
    h.bias_correction = int(kw.get("bias_correction", 1))
    h.grad_averaging = int(kw.get("grad_averaging", 1))
    h.mode = int(kw.get("mode", 1))
    h.normalize_grad = int(kw.get("normalize_grad", 1))
    h.grad_scale = kw.get("grad_scale", 1.0)
    h.average = int(kw.get("average", 1))
    return h


class _DevMem:
    """Exposes a raw device range through __cuda_array_interface__ (no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


def _device_view(ptr: int, nbytes: int, dtype) -> torch.Tensor:
    return torch.as_tensor(_DevMem(ptr, nbytes), device="cuda").view(dtype)


class ZeroStep:
    """reduce-scatter -> shard update -> all-gather over a Plan (rafb200_zero_*)."""

    def __init__(self, plan: Plan, comm, g_dtype, param_dtype, optimizer: str):
        self.plan, self.comm = plan, comm
        self.g_dtype, self.param_dtype = torch_dtype(g_dtype), torch_dtype(param_dtype)
        self.optimizer = optimizer
        h = C.c_void_p()
        opt = {"sgd": OPT_SGD, "adam": OPT_ADAM, "lans": OPT_LANS}[optimizer]
        check(_lib.load().rafb200_zero_create(plan.handle, comm.handle, dtype_code(self.g_dtype),
                                              dtype_code(self.param_dtype), opt, C.byref(h)))
        self.handle = h
        self._keep = None

    def bind(self, grads, params, p, m, v=None):
        pa = _lib.ptr_array
        for ts, dt in ((grads, self.g_dtype), (params, self.param_dtype), (p, torch.float32),
                       (m, torch.float32), (v, torch.float32)):
            if ts is None:
                continue
            assert len(ts) == self.plan.k
            for t in ts:
                assert t.is_cuda and t.is_contiguous() and t.dtype == dt, (t.dtype, dt)
        check(_lib.load().rafb200_zero_bind(
            self.handle, pa([t.data_ptr() for t in grads]), pa([t.data_ptr() for t in params]),
            pa([t.data_ptr() for t in p]), pa([t.data_ptr() for t in m]),
            pa([t.data_ptr() for t in v]) if v is not None else None))
        self._keep = (grads, params, p, m, v)

    def step(self, hyper: Hyper, step: int, compute_stream=None, comm_stream=None):
        from .distributed import comm_stream as default_comm_stream

        cs = compute_stream if compute_stream is not None else torch.cuda.current_stream()
        ms = comm_stream if comm_stream is not None else default_comm_stream()
        check(_lib.load().rafb200_zero_step(self.handle, C.byref(hyper), int(step), cs.cuda_stream,
                                            ms.cuda_stream))

    def step_host(self, hyper: Hyper, step: int, grads_host, params_host, compute_stream=None,
                  comm_stream=None):
        """Host-buffer form: gradients come from (pinned) host tensors, the updated
        model-dtype parameters are copied back into host tensors."""
        from .distributed import comm_stream as default_comm_stream

        cs = compute_stream if compute_stream is not None else torch.cuda.current_stream()
        ms = comm_stream if comm_stream is not None else default_comm_stream()
        pa = _lib.ptr_array
        check(_lib.load().rafb200_zero_step_host(
            self.handle, C.byref(hyper), int(step), pa([t.data_ptr() for t in grads_host]),
            pa([t.data_ptr() for t in params_host]), cs.cuda_stream, ms.cuda_stream))

    def launch_counts(self) -> Tuple[int, int]:
        a, b = C.c_int(), C.c_int()
        check(_lib.load().rafb200_zero_launch_counts(self.handle, C.byref(a), C.byref(b)))
        return a.value, b.value

    def attach_symmetric(self, group=None, comm_blocks: int = 0, multicast: bool = True,
                         allocator: str = "library", key: Optional[str] = None, timeout_ms: int = 60000):
        """Switch the collectives of this step from NCCL to the library's own kernels over
        symmetric memory: one allocation mapped into every rank plus, with ``multicast``, its
        NVSwitch multicast address.  ``allocator="library"`` takes the memory from
        rafb200_symm_alloc (``key``: a string common to the ranks of this job, default
        MASTER_ADDR:MASTER_PORT); ``allocator="torch"`` from torch.distributed._symmetric_memory
        on ``group`` (default: the world group, which must be initialised).  Call on every
        rank, before :meth:`bind`."""
        lib = _lib.load()
        gb, pb, sb = C.c_size_t(), C.c_size_t(), C.c_size_t()
        check(lib.rafb200_zero_flat_bytes(self.handle, C.byref(gb), C.byref(pb), C.byref(sb)))

        def up(x):
            return (x + 4095) & ~4095

        sig_off, g_off = 0, up(sb.value)
        p_off = g_off + up(gb.value)
        total = p_off + up(pb.value)
        n, rank = self.comm.size, self.comm.rank
        if allocator == "library":
            if key is None:
                key = f"{os.environ.get('MASTER_ADDR', 'local')}:{os.environ.get('MASTER_PORT', '0')}"
            h = C.c_void_p()
            check(lib.rafb200_symm_alloc(n, rank, torch.cuda.current_device(), total, key.encode(),
                                         1 if multicast else 0, int(timeout_ms), C.byref(h)))
            ptrs = (C.c_void_p * n)()
            mcp = C.c_void_p()
            check(lib.rafb200_symm_pointers(h, ptrs, C.byref(mcp)))
            bases = [int(ptrs[q]) for q in range(n)]
            mc = int(mcp.value or 0)
            buf = _device_view(bases[rank], total, torch.uint8)
            buf.zero_()  # padding rows, alignment gaps and barrier words all start at zero
            torch.cuda.synchronize()
            if n > 1:  # every rank has cleared its memory before any rank's kernels touch it
                from . import distributed as dist

                token = torch.zeros(1, device="cuda")
                check(lib.rafb200_allreduce(self.comm.handle, token.data_ptr(), token.data_ptr(), 1,
                                            dist.dtype_code(token.dtype), b"sum", None))
                torch.cuda.synchronize()
            self._symm = (buf, h)
            self._symm_lib = h
        elif allocator == "torch":
            import torch.distributed as td
            import torch.distributed._symmetric_memory as symm

            buf = symm.empty(total, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
            handle = symm.rendezvous(buf, group if group is not None else td.group.WORLD)
            buf.zero_()
            torch.cuda.synchronize()
            handle.barrier()
            torch.cuda.synchronize()
            bases = [int(x) for x in handle.buffer_ptrs]
            mc = int(handle.multicast_ptr) if multicast else 0
            self._symm = (buf, handle)  # keeps the mapping alive
        else:
            raise ValueError(f"unknown allocator {allocator!r}")
        pa = _lib.ptr_array
        check(lib.rafb200_zero_attach_symmetric(
            self.handle, pa([b + g_off for b in bases]), (mc + g_off) if mc else None,
            pa([b + p_off for b in bases]), (mc + p_off) if mc else None,
            pa([b + sig_off for b in bases]), int(comm_blocks)))
        self.declare_arena(buf)
        self._arena = (g_off, p_off)
        self.multicast = bool(mc)

    def set_fused(self, mode: int):
        """LANS with the collectives inside the update kernel: 1 = reduce-scatter, 2 = all-gather
        too (rafb200_zero_set_fused).  After attach_symmetric, before bind, on every rank."""
        check(_lib.load().rafb200_zero_set_fused(self.handle, int(mode)))

    def arena_views(self):
        """(grads, params): per tensor a view of its region of the symmetric gradient /
        parameter buffer in the tensor's own shape, or None where the shard size is not a
        multiple of 8 elements.  Binding these tensors makes the step copy-free for them."""
        import numpy as np

        k = self.plan.k
        off = np.zeros(k, np.int64)
        nat = np.zeros(k, np.int32)
        check(_lib.load().rafb200_zero_arena_offsets(self.handle, off.ctypes.data, nat.ctypes.data))
        buf = self._symm[0]
        g_off, p_off = self._arena
        grads, params = [], []
        for i, shape in enumerate(self.plan.shapes):
            n = numel(shape)
            if not nat[i]:
                grads.append(None)
                params.append(None)
                continue
            for out, base, dt in ((grads, g_off, self.g_dtype), (params, p_off, self.param_dtype)):
                es = torch.empty((), dtype=dt).element_size()
                lo = base + int(off[i]) * es
                out.append(buf[lo:lo + n * es].view(dt).view(shape if len(shape) else ()))
        return grads, params

    def status(self):
        """Synchronise the device; raise if a bounded cross-GPU wait of a step ran out."""
        check(_lib.load().rafb200_zero_status(self.handle))

    def set_wait_limit(self, limit_ms: int):
        """Bound of every cross-GPU wait of the symmetric mode (default 10 s)."""
        check(_lib.load().rafb200_zero_set_wait_limit(self.handle, int(limit_ms)))

    def declare_arena(self, tensor: torch.Tensor):
        """Declare the memory of ``tensor`` (host or device) to be one allocation, so that
        step_host may merge the copies of adjacent tensors inside it."""
        check(_lib.load().rafb200_zero_declare_arena(self.handle, tensor.data_ptr(),
                                                     tensor.numel() * tensor.element_size()))

    def set_host_output(self, mode: int):
        """step_host copies back 0: every parameter in full, 1: this rank's rows only."""
        check(_lib.load().rafb200_zero_set_host_output(self.handle, int(mode)))

    def shard_grad(self, i: int) -> torch.Tensor:
        """The gradient block the update of tensor ``i`` reads (this rank's reduced row
        block when there is more than one rank), as a 1-D view of device memory."""
        ptr = C.c_void_p()
        check(_lib.load().rafb200_zero_shard_grad(self.handle, int(i), C.byref(ptr)))
        n = int(self.plan.shard_elems[i])
        es = torch.empty((), dtype=self.g_dtype).element_size()
        if n == 0 or not ptr.value:
            return torch.empty(0, dtype=self.g_dtype, device="cuda")
        return _device_view(ptr.value, n * es, self.g_dtype)

    def set_stage_mask(self, mask: int):
        """Measurement aid: bit 0 pack, 1 reduce-scatter, 2 update, 3 all-gather, 4 unpack."""
        check(_lib.load().rafb200_zero_set_stage_mask(self.handle, int(mask)))

    def set_update_blocks(self, max_blocks: int):
        check(_lib.load().rafb200_zero_set_update_blocks(self.handle, int(max_blocks)))

    def close(self):
        if self.handle:
            torch.cuda.synchronize()
            _lib.load().rafb200_zero_destroy(self.handle)
            self.handle = None
        if getattr(self, "_symm_lib", None):
            # the peers may still be reading this rank's memory: leave together
            if self.comm.size > 1:
                token = torch.zeros(1, device="cuda")
                check(_lib.load().rafb200_allreduce(self.comm.handle, token.data_ptr(), token.data_ptr(), 1, 0,
                                                    b"sum", None))
                torch.cuda.synchronize()
            self._symm = None
            _lib.load().rafb200_symm_free(self._symm_lib)
            self._symm_lib = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n
