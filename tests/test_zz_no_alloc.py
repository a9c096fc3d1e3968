"""rafb200_lans_tensor_static: the one-tensor LANS entry point that allocates nothing.

Called through the C ABI with raw device pointers and compared with the existing
entry point (rafb200_lans on a one-tensor list) AND with the CPU oracle on the same
inputs, for two calls in a row - the second call finds the shared static array as the
first one left it.  Tolerance: 1e-5 relative, the LANS bar of this suite (the two entry
points run the same kernel, so in practice they agree far more closely).  The free
device memory reported by the driver must be the same before and after the calls.

The file name sorts last on purpose: this test must pass both alone and after every
other GPU test has used the library in the same process.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import CODES, TORCH, make_grad, rel_err, to_numpy, to_torch

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
    po, mo, vo = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)  # CPU oracle
    tl = op.TensorList([n], g_dtype, out_dtype or "float32")
    grads = [make_grad(np.random.default_rng(100 + step), n, g_dtype, loss_scale=1.0 / scale)
             for step in (1, 2)]
    tgrads = [to_torch(g, g_dtype) for g in grads]
    # the first call on a device resolves the address of the static array: make it here, then
    # compare the driver's free-memory figure right before and right after each call under test
    # (nothing of torch allocates in between)
    _lib.check(_static_call(lib, tgrads[0], *state()[:3], None, 1, mode, normalize_grad, scale))
    torch.cuda.synchronize()
    try:
        for step in (1, 2):
            g = tgrads[step - 1]
            tl.bind([g], [pa], [ma], [va], [oa] if oa is not None else None)
            op.lans_list_(tl, step, HYPER["learning_rate"], HYPER["beta1"], HYPER["beta2"],
                          HYPER["eps"], HYPER["bias_correction"], HYPER["weight_decay"],
                          HYPER["grad_averaging"], mode, normalize_grad, grad_scale=scale)
            op.lans_status(tl)
            free_mid = torch.cuda.mem_get_info()[0]
            _lib.check(_static_call(lib, g, pb, mb, vb, ob, step, mode, normalize_grad, scale))
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_mid, "the call changed the free device memory"
            O.lans([grads[step - 1]], [po], [mo], [vo], step, HYPER["learning_rate"], HYPER["beta1"],
                   HYPER["beta2"], HYPER["eps"], HYPER["bias_correction"], HYPER["weight_decay"],
                   HYPER["grad_averaging"], mode, int(normalize_grad), scale)
            for a, b, ref, name in ((pa, pb, po, "p"), (ma, mb, mo, "m"), (va, vb, vo, "v")):
                err = rel_err(to_numpy(b), to_numpy(a))
                assert err < 1e-5, (name, step, err)
                err = rel_err(to_numpy(b), ref)
                assert err < 1e-5, ("against the oracle", name, step, err)
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
