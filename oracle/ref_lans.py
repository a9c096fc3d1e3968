"""ctypes front end of oracle/_ref/libraf_ref_lans.so: the reference's own
multi_tensor_lans_cuda<float>, compiled unchanged from the reference tree by
oracle/Makefile.  Test infrastructure (it needs a GPU); used to pin the CPU
oracle, to produce tests/golden/lans_ref_*.npz and as "the existing kernel" timed
beside this repository's kernel.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libraf_ref_lans.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(LIB_PATH)
        L.ref_lans_workspace_floats.restype = C.c_size_t
        L.ref_lans_workspace_floats.argtypes = [C.c_int, C.c_void_p, C.POINTER(C.c_int)]
        L.ref_lans.restype = C.c_int
        L.ref_lans.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                               C.c_int, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int,
                               C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                               C.c_void_p, C.c_void_p]
        _lib = L
    return _lib


class RefLans:
    """Runs raf.op.cuda.lans' kernel sequence on lists of fp32 CUDA tensors."""

    def __init__(self, numels, q_layout=0):
        self.k = len(numels)
        self.numels = (C.c_int * self.k)(*[int(n) for n in numels])
        self.q_layout = q_layout
        mc = C.c_int()
        nfloats = lib().ref_lans_workspace_floats(self.k, self.numels, C.byref(mc))
        self.workspace = torch.zeros(max(nfloats, 1), dtype=torch.float32, device="cuda")
        self.norms = torch.zeros(4 * max(self.k, 1), dtype=torch.float32, device="cuda")

    def __call__(self, g, p, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6,
                 bias_correction=1, weight_decay=0.01, grad_averaging=1, mode=1, normalize_grad=1,
                 stream=None):
        def arr(ts):
            return (C.c_void_p * self.k)(*[t.data_ptr() for t in ts])

        s = (stream or torch.cuda.current_stream()).cuda_stream
        rc = lib().ref_lans(self.k, arr(g), arr(p), arr(m), arr(v), self.numels, int(step), lr,
                            beta1, beta2, eps, int(bias_correction), weight_decay,
                            int(grad_averaging), int(mode), int(normalize_grad),
                            self.workspace.data_ptr(), self.q_layout, self.norms.data_ptr(), s)
        if rc != 0:
            raise RuntimeError(f"reference LANS kernel failed with CUDA error {rc}")

    def norms_host(self):
        """[k, 4]: ||g||, ||p||, ||update_m||, ||update_g||."""
        return self.norms[: 4 * self.k].view(4, self.k).t().contiguous().cpu().numpy()
