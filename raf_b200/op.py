"""Python mirror of the RAF operators on the ZeRO optimizer path.

Same names, argument order and dtype rules as ``raf.op.*`` / ``raf._op.imp``
in the reference (``scripts/src_codegen/def_schema.py:525-536,671-738``), on
``torch`` CUDA tensors.  Every function forwards device pointers to the C ABI
(``include/raf_b200.h``); nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib
from ._lib import BF16, F16, F32, check

_CODES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
_NAMES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def dtype_code(dtype) -> int:
    if isinstance(dtype, str):
        dtype = _NAMES[dtype]
    try:
        return _CODES[dtype]
    except KeyError as exc:
        raise TypeError(f"NotImplementedError: {dtype}") from exc


def torch_dtype(dtype):
    return _NAMES[dtype] if isinstance(dtype, str) else dtype


def _check_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("raf_b200 operators need CUDA tensors; there is no CPU path")
        if not t.is_contiguous():
            raise ValueError("tensors must be compact (contiguous), as in the reference")


def stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


# --------------------------------------------------------------------------- lists
class TensorList:
    """Device-resident tensor list ([g..., p..., m..., v...] of raf.op.lans)."""

    def __init__(self, numels: Sequence[int], g_dtype, out_dtype=torch.float32):
        self.k = len(numels)
        self.numels = [int(n) for n in numels]
        self.g_dtype = torch_dtype(g_dtype)
        self.out_dtype = torch_dtype(out_dtype)
        h = C.c_void_p()
        check(_lib.load().rafb200_tensor_list_create(
            self.k, _lib.i64_array(self.numels), dtype_code(self.g_dtype),
            dtype_code(self.out_dtype), C.byref(h)))
        self.handle = h
        self._keep = None
        self._ws = None

    def bind(self, g, p, m, v=None, out=None, stream=None):
        def ptrs(ts, dtype):
            if ts is None:
                return None
            assert len(ts) == self.k
            res = []
            for t, n in zip(ts, self.numels):
                if t is None:
                    res.append(0)
                    continue
                _check_cuda(t)
                assert t.numel() == n and t.dtype == dtype, (t.shape, t.dtype, n, dtype)
                res.append(t.data_ptr())
            return _lib.ptr_array(res)

        check(_lib.load().rafb200_tensor_list_bind(
            self.handle, ptrs(g, self.g_dtype), ptrs(p, torch.float32), ptrs(m, torch.float32),
            ptrs(v, torch.float32), ptrs(out, self.out_dtype), stream_ptr(stream)))
        self._keep = (g, p, m, v, out)  # the device table holds raw pointers

    def tune(self, lead_elems=8 << 20, gap_items=0, max_blocks=0):
        """Scheduling knobs of the LANS kernel (rafb200_tensor_list_tune); the defaults are
        the ones a list is created with."""
        check(_lib.load().rafb200_tensor_list_tune(self.handle, int(lead_elems), int(gap_items),
                                                   int(max_blocks)))

    def set_wait_limit(self, limit_ms: int):
        """Bound of every wait inside the LANS kernel (default 2 s)."""
        check(_lib.load().rafb200_tensor_list_set_wait_limit(self.handle, int(limit_ms)))

    def set_symmetric(self, rank, g_peers, p_peers, g_offsets_bytes, g_mc=0, p_mc=0, reduce_scatter=True,
                      all_gather=True):
        """The collectives inside the update kernels (rafb200_tensor_list_set_symmetric):
        ``g_peers`` / ``p_peers`` = every rank's gradient / parameter buffer as addressable here
        (device addresses), ``g_offsets_bytes`` = each tensor's offset inside the gradient buffer."""
        world = len(g_peers)
        off = _lib.i64_array([int(x) for x in g_offsets_bytes])
        check(_lib.load().rafb200_tensor_list_set_symmetric(
            self.handle, world, int(rank), _lib.ptr_array([int(x) for x in g_peers]), int(g_mc) or None,
            _lib.ptr_array([int(x) for x in p_peers]), int(p_mc) or None, off, int(bool(reduce_scatter)),
            int(bool(all_gather))))

    def set_lans_items(self, items):
        """Replace the LANS work-item table: ``items`` is an (n, 2) uint32 array."""
        import numpy as np

        a = np.ascontiguousarray(items, np.uint32).reshape(-1, 2)
        check(_lib.load().rafb200_tensor_list_set_lans_items(self.handle, a.ctypes.data, a.shape[0]))

    def lans_workspace(self) -> torch.Tensor:
        if self._ws is None:
            n = _lib.load().rafb200_lans_workspace_bytes(self.handle)
            self._ws = torch.empty(max(n, 16), dtype=torch.uint8, device="cuda")
        return self._ws

    def close(self):
        if self.handle:
            torch.cuda.synchronize()
            _lib.load().rafb200_tensor_list_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass


# --------------------------------------------------------------------------- optimizers
def sgd(x, dx, v, learning_rate, mu):
    """raf.op.sgd: returns (v1, x1) as NEW tensors (src/op/declare/optimizer.cc:22-44)."""
    _check_cuda(x, dx, v)
    if x.shape != dx.shape or x.shape != v.shape:
        raise ValueError("sgd: x, dx and v must have the same shape")
    x1 = x.clone()
    v1 = v.clone()
    sgd_(x1, dx, v1, learning_rate, mu)
    return v1, x1


def sgd_(x, dx, v, learning_rate, mu, weight_decay=0.0, grad_scale=1.0, out=None, stream=None):
    """In-place fused form: x, v fp32; dx fp32/fp16/bf16; out (optional) receives cast(x1)."""
    _check_cuda(x, dx, v)
    assert x.dtype == torch.float32 and v.dtype == torch.float32
    if out is not None:
        _check_cuda(out)
        assert out.numel() == x.numel()
    check(_lib.load().rafb200_sgd(
        x.data_ptr(), dx.data_ptr(), dtype_code(dx.dtype), v.data_ptr(), x.numel(),
        float(learning_rate), float(mu), float(weight_decay), float(grad_scale),
        out.data_ptr() if out is not None else None,
        dtype_code(out.dtype) if out is not None else F32, stream_ptr(stream)))
    return x, v


def sgd_list_(tl: TensorList, learning_rate, mu, weight_decay=0.0, grad_scale=1.0, stream=None):
    check(_lib.load().rafb200_sgd_list(tl.handle, float(learning_rate), float(mu),
                                       float(weight_decay), float(grad_scale), stream_ptr(stream)))


def lans_list_(tl: TensorList, step, learning_rate, beta1, beta2, eps, bias_correction,
               weight_decay, grad_averaging, mode, normalize_grad, grad_scale=1.0, stream=None):
    """raf.op.lans on a bound TensorList; ``step`` is an int or a 0-d fp32 CUDA tensor."""
    ws = tl.lans_workspace()
    step_dev = None
    if isinstance(step, torch.Tensor):
        assert step.is_cuda and step.dtype == torch.float32 and step.dim() == 0
        step_dev, step = step.data_ptr(), 0
    check(_lib.load().rafb200_lans(
        tl.handle, int(step), step_dev, float(learning_rate), float(beta1), float(beta2),
        float(eps), int(bias_correction), float(weight_decay), int(grad_averaging), int(mode),
        int(bool(normalize_grad)), float(grad_scale), ws.data_ptr(), ws.numel(),
        stream_ptr(stream)))


def lans_status(tl: TensorList, want_norms=False, stream=None):
    """Waits for the stream; raises if a bounded device wait expired; returns norms[k,4] or None."""
    import numpy as np

    norms = np.zeros((tl.k, 4), np.float32) if want_norms else None
    check(_lib.load().rafb200_lans_status(
        tl.handle, tl.lans_workspace().data_ptr(),
        norms.ctypes.data if norms is not None else None, stream_ptr(stream)))
    return norms


def lans(tensor_list: List[torch.Tensor], step, learning_rate, beta1, beta2, eps, bias_correction,
         weight_decay, grad_averaging, mode, normalize_grad):
    """raf.op.lans (python/raf/optim/lans.py:87-99): tensor_list = g + p + m + v, updated in place.

    Like the reference (src/op/dialect/cuda/lans.cc:38-40) it takes fp32 tensors only;
    16-bit gradients go through :class:`TensorList` / :func:`lans_list_`.
    """
    n = len(tensor_list)
    if n % 4 != 0:
        raise ValueError("lans: tensor_list must hold g, p, m and v lists of equal length")
    k = n // 4
    for t in tensor_list:
        _check_cuda(t)
        if t.dtype != torch.float32:
            raise TypeError("LANS only takes FP32 inputs")
    g, p, m, v = (tensor_list[i * k:(i + 1) * k] for i in range(4))
    tl = TensorList([t.numel() for t in p], torch.float32, torch.float32)
    try:
        tl.bind(g, p, m, v)
        lans_list_(tl, step, learning_rate, beta1, beta2, eps, bias_correction, weight_decay,
                   grad_averaging, mode, normalize_grad)
        lans_status(tl)
    finally:
        tl.close()
    return tensor_list


def adam_list_(tl: TensorList, step, learning_rate, beta1, beta2, eps, bias_correction,
               weight_decay, mode, grad_scale=1.0, stream=None):
    """Adam / AdamW on a bound TensorList (no reference operator; see include/raf_b200.h)."""
    check(_lib.load().rafb200_adam(
        tl.handle, int(step), None, float(learning_rate), float(beta1), float(beta2), float(eps),
        int(bias_correction), float(weight_decay), int(mode), float(grad_scale),
        stream_ptr(stream)))


# --------------------------------------------------------------------------- casts, packing
def cast(data, dtype, out=None, stream=None):
    """raf.op.cast."""
    _check_cuda(data)
    dtype = torch_dtype(dtype)
    if out is None:
        out = torch.empty_like(data, dtype=dtype)
    check(_lib.load().rafb200_cast(data.data_ptr(), dtype_code(data.dtype), out.data_ptr(),
                                   dtype_code(dtype), data.numel(), stream_ptr(stream)))
    return out


def group_cast(tensor_list, dtype, stream=None):
    """raf.op.group_cast: one launch for the whole tuple."""
    dtype = torch_dtype(dtype)
    if not tensor_list:
        return []
    _check_cuda(*tensor_list)
    src_dtype = tensor_list[0].dtype
    assert all(t.dtype == src_dtype for t in tensor_list)
    outs = [torch.empty_like(t, dtype=dtype) for t in tensor_list]
    check(_lib.load().rafb200_group_cast(
        len(tensor_list), _lib.ptr_array([t.data_ptr() for t in tensor_list]),
        dtype_code(src_dtype), _lib.ptr_array([t.data_ptr() for t in outs]), dtype_code(dtype),
        _lib.i64_array([t.numel() for t in tensor_list]), stream_ptr(stream)))
    return outs


def fuse_tensor(tensor_list, stream=None):
    """raf.op.fuse_tensor: concatenate a tuple into one flat buffer."""
    _check_cuda(*tensor_list)
    dtype = tensor_list[0].dtype
    numels = [t.numel() for t in tensor_list]
    offsets = [0]
    for n in numels[:-1]:
        offsets.append(offsets[-1] + n)
    flat = torch.empty(sum(numels), dtype=dtype, device=tensor_list[0].device)
    check(_lib.load().rafb200_fuse_tensor(
        len(tensor_list), _lib.ptr_array([t.data_ptr() for t in tensor_list]),
        _lib.i64_array(numels), _lib.i64_array(offsets), flat.element_size(), flat.data_ptr(),
        stream_ptr(stream)))
    return flat


def defuse_tensor(data, sizes, shapes, shape_indices, stream=None):
    """raf.op.defuse_tensor (schema DefuseTensorArgs{data, sizes, shapes, shape_indices})."""
    _check_cuda(data)
    outs, offsets, start = [], [], 0
    off = 0
    for i, n in enumerate(sizes):
        shape = tuple(shapes[start:shape_indices[i]])
        start = shape_indices[i]
        outs.append(torch.empty(shape, dtype=data.dtype, device=data.device))
        assert outs[-1].numel() == n
        offsets.append(off)
        off += n
    check(_lib.load().rafb200_defuse_tensor(
        len(outs), _lib.ptr_array([t.data_ptr() for t in outs]), _lib.i64_array(sizes),
        _lib.i64_array(offsets), data.element_size(), data.data_ptr(), stream_ptr(stream)))
    return outs
