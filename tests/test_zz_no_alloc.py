"""rafb200_lans_tensor_static: the one-tensor LANS entry point that allocates nothing.

Called through the C ABI with raw device pointers and compared with the existing
entry point (rafb200_lans on a one-tensor list) on the same inputs, for two calls in
a row - the second call finds the shared static array as the first one left it.
Tolerance: 1e-5 relative, the LANS bar of this suite (the two entry points run the
same kernel, so in practice they agree far more closely).

The file name sorts last on purpose: this test must pass both alone and after every
other GPU test has used the library in the same process.
"""
import numpy as np
import pytest
import torch

from tests.util import TORCH, make_grad, rel_err, to_numpy, to_torch

pytestmark = pytest.mark.gpu

MAX_ELEMS = 4 << 20
HYPER = dict(learning_rate=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, bias_correction=1,
             weight_decay=0.01, grad_averaging=1)


def _static_call(lib, g, p, m, v, out, step, mode, normalize_grad, grad_scale=1.0):
    from raf_b200 import op

    return lib.rafb200_lans_tensor_static(
        g.data_ptr(), op.dtype_code(g.dtype), p.data_ptr(), m.data_ptr(), v.data_ptr(),
        out.data_ptr() if out is not None else None,
        op.dtype_code(out.dtype) if out is not None else 0, p.numel(), step,
        HYPER["learning_rate"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"],
        HYPER["bias_correction"], HYPER["weight_decay"], HYPER["grad_averaging"], mode,
        int(normalize_grad), grad_scale, op.stream_ptr())


@pytest.mark.parametrize("n,g_dtype,out_dtype,mode,normalize_grad", [
    (1, "float32", None, 1, True),
    (4097, "float32", "float32", 1, True),
    (300007, "float16", "float16", 1, True),
    (1 << 20, "bfloat16", "bfloat16", 0, False),
    (MAX_ELEMS, "float32", "float16", 1, True),
])
def test_static_entry_matches_list_entry_twice(n, g_dtype, out_dtype, mode, normalize_grad):
    from raf_b200 import _lib, op

    lib = _lib.load()
    rng = np.random.default_rng(n)
    p0 = (rng.standard_normal(n) * 0.02).astype(np.float32)
    scale = 2.0 ** -7 if g_dtype != "float32" else 1.0

    def state():
        return (to_torch(p0, "float32"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"),
                torch.zeros(n, dtype=TORCH[out_dtype], device="cuda") if out_dtype else None)

    pa, ma, va, oa = state()   # existing entry point
    pb, mb, vb, ob = state()   # static-scratch entry point
    tl = op.TensorList([n], g_dtype, out_dtype or "float32")
    try:
        for step in (1, 2):
            g = to_torch(make_grad(np.random.default_rng(100 + step), n, g_dtype,
                                   loss_scale=1.0 / scale), g_dtype)
            tl.bind([g], [pa], [ma], [va], [oa] if oa is not None else None)
            op.lans_list_(tl, step, HYPER["learning_rate"], HYPER["beta1"], HYPER["beta2"],
                          HYPER["eps"], HYPER["bias_correction"], HYPER["weight_decay"],
                          HYPER["grad_averaging"], mode, normalize_grad, grad_scale=scale)
            op.lans_status(tl)
            _lib.check(_static_call(lib, g, pb, mb, vb, ob, step, mode, normalize_grad, scale))
            torch.cuda.synchronize()
            for a, b, name in ((pa, pb, "p"), (ma, mb, "m"), (va, vb, "v")):
                err = rel_err(to_numpy(b), to_numpy(a))
                assert err < 1e-5, (name, step, err)
            if oa is not None:
                err = rel_err(to_numpy(ob.float()), to_numpy(oa.float()))
                assert err < (1e-5 if out_dtype == "float32" else 1e-2), ("out", step, err)
            assert float((pb - to_torch(p0, "float32")).abs().max()) > 0  # it did update
    finally:
        tl.close()


def test_static_entry_rejects_oversize_and_bad_arguments():
    from raf_b200 import _lib

    lib = _lib.load()
    x = torch.zeros(16, device="cuda")
    # Nothing is launched for a refused call, so the small buffers are never touched.
    rc = lib.rafb200_lans_tensor_static(
        x.data_ptr(), 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 0, MAX_ELEMS + 1, 1,
        1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, 1.0, None)
    assert rc == 1  # RAFB200_INVALID_ARGUMENT
    msg = lib.rafb200_last_error().decode()
    assert "exceed" in msg and str(MAX_ELEMS) in msg
    rc = lib.rafb200_lans_tensor_static(
        x.data_ptr(), 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 0, 16, 0,
        1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, 1.0, None)
    assert rc == 1  # RAFB200_INVALID_ARGUMENT
    # numel == 0 is a no-op, as for the list entry point
    rc = lib.rafb200_lans_tensor_static(
        None, 0, None, None, None, None, 0, 0, 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, 1.0,
        None)
    assert rc == 0
