"""The RAF-side glue (raf_b200/csrc/raf_dialect/b200_ops.cc), compiled against the raf_compat
stand-in for RAF's headers: what it registers (CPU), and its OpEnvs driven the way RAF's
executors drive them - schema struct from raw device pointers, dispatch by priority level,
requests fulfilled, Execute - against the CPU oracle (GPU)."""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_vp, _i, _i64, _f, _d = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double


def glue():
    from raf_b200 import _lib

    _lib.load()  # libraf_b200.so first: the glue links against it
    lib = C.CDLL(os.path.join(ROOT, "raf_b200", "libraf_b200_glue.so"))
    lib.rafcompat_last_error.restype = C.c_char_p
    lib.rafcompat_list_ops.argtypes = [C.c_char_p, C.c_size_t]
    lib.rafcompat_run_sgd.argtypes = [_vp, _vp, _i, _vp, _vp, _vp, _i64, _d, _d, _vp]
    lib.rafcompat_run_lans.argtypes = [_i, _vp, _vp, _i, _vp, _f, _f, _f, _f, _i, _f, _i, _i, _i, _vp]
    lib.rafcompat_run_cast.argtypes = [_vp, _i, _vp, _i, _i64, _vp]
    lib.rafcompat_run_fuse_defuse.argtypes = [_i, _vp, _vp, _vp, _vp, _i, _vp]
    lib.rafcompat_run_collective.argtypes = [_i, _i, _vp, _vp, _vp, _vp, _i, C.c_char_p, _vp, _i, _i, _vp]
    return lib


def ok(lib, rc):
    assert rc == 0, lib.rafcompat_last_error().decode()


def test_registry_names_and_levels():
    """One dialect "b200", enabled for CUDA; one dialect op with a maker per base operator of
    the path, at levels above the stock implementations (nccl ops 10, cuda.lans 20, tvm 10:
    src/op/dialect/nccl/nccl.cc:154-155, src/op/dialect/cuda/lans.cc:164-165)."""
    lib = glue()
    buf = C.create_string_buffer(8192)
    lib.rafcompat_list_ops(buf, len(buf))
    lines = [ln.split() for ln in buf.value.decode().splitlines()]
    assert ["dialect", "b200", "cuda"] in lines
    ops = {ln[0]: ln for ln in lines if ln[0].startswith("raf.op.")}
    want = {"raf.op.lans": 30, "raf.op.sgd": 20, "raf.op.cast": 20, "raf.op.group_cast": 20,
            "raf.op.fuse_tensor": 20, "raf.op.defuse_tensor": 20, "raf.op._allreduce": 20,
            "raf.op._allgather": 20, "raf.op._group_allgather": 20, "raf.op._reduce_scatter": 20,
            "raf.op._group_reduce_scatter": 20}
    assert set(ops) == set(want)
    for base, level in want.items():
        _, dialect, dialect_op, plevel, maker = ops[base]
        assert dialect == "b200" and dialect_op == base.replace("raf.op.", "raf.op.b200.")
        assert int(plevel) == level and maker == "maker"


@pytest.mark.gpu
@pytest.mark.parametrize("inplace", [False, True])
def test_sgd_openv(inplace):
    """SgdB200::Execute: (v1, x1) in new buffers, or - as the InplaceUpdate pass arranges -
    in the inputs' own buffers; bit-exact against the oracle either way."""
    import torch
    from oracle import oracle as O

    lib = glue()
    n = 70001
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(n) * 0.02).astype(np.float32)
    v = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    dx = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    tx, tv, tdx = (torch.from_numpy(a.copy()).cuda() for a in (x, v, dx))
    tv1, tx1 = (tv, tx) if inplace else (torch.zeros_like(tv), torch.zeros_like(tx))
    ok(lib, lib.rafcompat_run_sgd(tx.data_ptr(), tdx.data_ptr(), 0, tv.data_ptr(), tv1.data_ptr(), tx1.data_ptr(),
                                  n, 0.1, 0.9, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    x_ref, v_ref = x.copy(), v.copy()
    O.sgd(x_ref, dx, v_ref, 0.1, 0.9)
    assert tx1.cpu().numpy().tobytes() == x_ref.tobytes() and tv1.cpu().numpy().tobytes() == v_ref.tobytes()
    if not inplace:  # the inputs were left alone
        assert tx.cpu().numpy().tobytes() == x.tobytes() and tv.cpu().numpy().tobytes() == v.tobytes()


@pytest.mark.gpu
def test_lans_openv_three_steps():
    """LansB200: list built in the constructor, workspace requested and re-allocated for every
    Execute, `step` read on the device; fp32 tensors as the reference op requires."""
    import torch
    from oracle import oracle as O
    from tests.util import rel_err

    lib = glue()
    numels = [5, 4096, 70001, 1]
    k = len(numels)
    rng = np.random.default_rng(3)
    p = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in numels]
    m = [np.zeros(n, np.float32) for n in numels]
    v = [np.zeros(n, np.float32) for n in numels]
    tp, tm, tv = ([torch.from_numpy(a.copy()).cuda() for a in xs] for xs in (p, m, v))
    nm = (C.c_int64 * k)(*numels)
    for step in (1, 2, 3):
        g = [(rng.standard_normal(n) * 1e-3).astype(np.float32) for n in numels]
        tg = [torch.from_numpy(a).cuda() for a in g]
        ptrs = (C.c_void_p * (4 * k))(*[t.data_ptr() for t in tg + tp + tm + tv])
        tstep = torch.tensor(float(step), device="cuda")
        ok(lib, lib.rafcompat_run_lans(k, ptrs, nm, 0, tstep.data_ptr(), 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1,
                                       torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        O.lans(g, p, m, v, step)
    for i in range(k):
        for ours, ref in ((tp[i], p[i]), (tm[i], m[i]), (tv[i], v[i])):
            assert rel_err(ours.cpu().numpy(), ref) < 1e-5


@pytest.mark.gpu
def test_cast_fuse_defuse_openvs():
    import torch
    from oracle import oracle as O

    lib = glue()
    s = torch.cuda.current_stream().cuda_stream
    x = np.random.default_rng(4).standard_normal(10007).astype(np.float32)
    tx = torch.from_numpy(x).cuda()
    ty = torch.zeros(x.size, dtype=torch.float16, device="cuda")
    ok(lib, lib.rafcompat_run_cast(tx.data_ptr(), 0, ty.data_ptr(), 1, x.size, s))
    torch.cuda.synchronize()
    assert ty.cpu().numpy().tobytes() == O.cast(x, O.F16).tobytes()
    numels = [3, 1000, 17, 4096]
    src = [torch.randn(n, device="cuda") for n in numels]
    dst = [torch.zeros(n, device="cuda") for n in numels]
    flat = torch.zeros(sum(numels), device="cuda")
    k = len(numels)
    ok(lib, lib.rafcompat_run_fuse_defuse(k, (C.c_void_p * k)(*[t.data_ptr() for t in src]),
                                          (C.c_void_p * k)(*[t.data_ptr() for t in dst]),
                                          (C.c_int64 * k)(*numels), flat.data_ptr(), 0, s))
    torch.cuda.synchronize()
    assert torch.equal(flat, torch.cat(src)) and all(torch.equal(a, b) for a, b in zip(src, dst))


@pytest.mark.gpu
def test_collective_openvs_on_the_void_communicator():
    """A world of one (RAF's VoidCommunicator): every collective of the path degenerates to a
    copy of its input, through the OpEnvs and the C ABI's communicator entry points."""
    import torch

    lib = glue()
    s = torch.cuda.current_stream().cuda_stream
    for dtype, code in ((torch.float32, 0), (torch.float16, 1), (torch.bfloat16, 2)):
        xs = [torch.randn(n, device="cuda").to(dtype) for n in (8, 1024, 33)]
        k = len(xs)
        nm = (C.c_int64 * k)(*[x.numel() for x in xs])
        pin = (C.c_void_p * k)(*[x.data_ptr() for x in xs])
        for which in (2, 4):  # _group_reduce_scatter, _group_allgather
            outs = [torch.zeros_like(x) for x in xs]
            pout = (C.c_void_p * k)(*[o.data_ptr() for o in outs])
            ok(lib, lib.rafcompat_run_collective(which, k, pin, pout, nm, nm, code, b"sum", None, 1, 0, s))
            torch.cuda.synchronize()
            assert all(torch.equal(a, b) for a, b in zip(xs, outs))
        for which in (1, 3):  # _reduce_scatter, _allgather
            out = torch.zeros_like(xs[1])
            ok(lib, lib.rafcompat_run_collective(which, 1, (C.c_void_p * 1)(xs[1].data_ptr()),
                                                 (C.c_void_p * 1)(out.data_ptr()), (C.c_int64 * 1)(xs[1].numel()),
                                                 (C.c_int64 * 1)(xs[1].numel()), code, b"avg" if which == 1 else b"sum",
                                                 None, 1, 0, s))
            torch.cuda.synchronize()
            assert torch.equal(out, xs[1])
        before = [x.clone() for x in xs]
        ok(lib, lib.rafcompat_run_collective(0, k, pin, pin, nm, nm, code, b"max", None, 1, 0, s))  # _allreduce
        torch.cuda.synchronize()
        assert all(torch.equal(a, b) for a, b in zip(xs, before))
