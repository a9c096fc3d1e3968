"""Parity of the CUDA kernels with the CPU oracle, through the C ABI (ctypes).

Bar: SGD and Adam bit-exact against the oracle (same operations, none fused);
LANS within 1e-5 (its trust ratios depend on the order of the norm reductions) and,
given identical norms, bit-exact element-wise; casts bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import CODES, EDGE_NUMELS, TORCH, bits_equal, make_grad, rel_err, to_numpy, to_torch

pytestmark = pytest.mark.gpu

G_DTYPES = ["float32", "float16", "bfloat16"]


@pytest.fixture(scope="module")
def rb():
    import raf_b200.op as op

    return op


def _params(rng, n):
    return ((rng.standard_normal(n) * 0.02).astype(np.float32), np.zeros(n, np.float32),
            np.zeros(n, np.float32))


# --------------------------------------------------------------------------- sgd
@pytest.mark.parametrize("n", EDGE_NUMELS)
def test_sgd_edge_sizes_bit_exact(rb, n):
    rng = np.random.default_rng(n + 1)
    p, v, _ = _params(rng, n)
    v = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    g = make_grad(rng, n, "float32")
    tp, tv, tg = to_torch(p, "float32"), to_torch(v, "float32"), to_torch(g, "float32")
    rb.sgd_(tp, tg, tv, 0.1, 0.9)
    O.sgd(p, g, v, 0.1, 0.9)
    torch.cuda.synchronize()
    assert bits_equal(to_numpy(tp), p) and bits_equal(to_numpy(tv), v)


@pytest.mark.parametrize("g_dtype", G_DTYPES)
@pytest.mark.parametrize("out_dtype", G_DTYPES)
def test_sgd_ten_steps_dtypes_bit_exact(rb, g_dtype, out_dtype):
    """BASELINE config 1 at reduced size: 10 steps, lr 0.1, momentum 0.9, wd 1e-4."""
    n = 300007
    rng = np.random.default_rng(0)
    p, v, _ = _params(rng, n)
    tp, tv = to_torch(p, "float32"), to_torch(v, "float32")
    tout = torch.zeros(n, dtype=TORCH[out_dtype], device="cuda")
    scale = 2.0 ** -7 if g_dtype != "float32" else 1.0
    for step in range(10):
        g = make_grad(np.random.default_rng(1 + step), n, g_dtype, loss_scale=1.0 / scale)
        tg = to_torch(g, g_dtype)
        rb.sgd_(tp, tg, tv, 0.1, 0.9, weight_decay=1e-4, grad_scale=scale, out=tout)
        out = O.sgd(p, g, v, 0.1, 0.9, weight_decay=1e-4, grad_scale=scale, out_code=CODES[out_dtype])
    torch.cuda.synchronize()
    assert bits_equal(to_numpy(tp), p)
    assert bits_equal(to_numpy(tv), v)
    assert bits_equal(to_numpy(tout), out)


def test_sgd_unaligned_views(rb):
    """Pointers that are only element-aligned take the scalar path."""
    n = 10001
    rng = np.random.default_rng(3)
    base_p = torch.zeros(n + 3, device="cuda")
    base_v = torch.zeros(n + 3, device="cuda")
    base_g = torch.zeros(n + 3, device="cuda", dtype=torch.float16)
    p, v, _ = _params(rng, n)
    g = make_grad(rng, n, "float16")
    tp, tv, tg = base_p[1:n + 1], base_v[3:n + 3], base_g[1:n + 1]
    tp.copy_(torch.from_numpy(p))
    tg.copy_(torch.from_numpy(g))
    rb.sgd_(tp, tg, tv, 0.05, 0.5)
    O.sgd(p, g, v, 0.05, 0.5)
    torch.cuda.synchronize()
    assert bits_equal(to_numpy(tp), p) and bits_equal(to_numpy(tv), v)
    assert base_p[0].item() == 0 and base_p[n + 1].item() == 0  # neighbours untouched


def test_sgd_op_returns_new_tensors(rb):
    """raf.op.sgd returns (v1, x1) and leaves its inputs alone
    (tests/python/op/tvm/test_tvm_loss.py::test_sgd)."""
    rng = np.random.default_rng(4)
    x0 = rng.standard_normal((4, 4)).astype(np.float32)
    dx = rng.standard_normal((4, 4)).astype(np.float32)
    v0 = rng.standard_normal((4, 4)).astype(np.float32)
    mu = float(np.float32(rng.standard_normal()))
    n_v1 = np.float32(mu) * v0 + dx
    n_x1 = x0 - np.float32(0.01) * n_v1
    tx, tdx, tv = (torch.from_numpy(a).cuda() for a in (x0, dx, v0))
    m_v1, m_x1 = rb.sgd(tx, tdx, tv, 0.01, mu)
    np.testing.assert_allclose(m_v1.cpu().numpy(), n_v1, 1e-4, 1e-4)
    np.testing.assert_allclose(m_x1.cpu().numpy(), n_x1, 1e-4, 1e-4)
    assert bits_equal(tx.cpu().numpy(), x0) and bits_equal(tv.cpu().numpy(), v0)
    with pytest.raises(ValueError):
        rb.sgd(tx, tdx[:2], tv, 0.01, mu)


def test_sgd_list_multi_tensor(rb):
    rng = np.random.default_rng(5)
    numels = [0, 1, 5, 4096, 4097, 70001, 64, 256 * 1024 + 1]
    ps, vs, gs = [], [], []
    for n in numels:
        p, v, _ = _params(rng, n)
        ps.append(p)
        vs.append(v)
        gs.append(make_grad(rng, n, "bfloat16"))
    tps = [to_torch(p, "float32") for p in ps]
    tvs = [to_torch(v, "float32") for v in vs]
    tgs = [to_torch(g, "bfloat16") for g in gs]
    touts = [torch.zeros(n, dtype=torch.float16, device="cuda") for n in numels]
    tl = rb.TensorList(numels, "bfloat16", "float16")
    tl.bind(tgs, tps, tvs, None, touts)
    for _ in range(3):
        rb.sgd_list_(tl, 0.1, 0.9, weight_decay=1e-4)
        outs = [O.sgd(p, g, v, 0.1, 0.9, weight_decay=1e-4, out_code=O.F16) for p, g, v in zip(ps, gs, vs)]
    torch.cuda.synchronize()
    for i in range(len(numels)):
        assert bits_equal(to_numpy(tps[i]), ps[i]), i
        assert bits_equal(to_numpy(tvs[i]), vs[i]), i
        assert bits_equal(to_numpy(touts[i]), outs[i]), i
    tl.close()


# --------------------------------------------------------------------------- adam
@pytest.mark.parametrize("g_dtype", G_DTYPES)
@pytest.mark.parametrize("mode", [0, 1])
def test_adam_bit_exact(rb, g_dtype, mode):
    rng = np.random.default_rng(6)
    numels = [3, 4096, 100001, 1 << 18]
    ps, ms, vs = zip(*[_params(rng, n) for n in numels])
    tps = [to_torch(p, "float32") for p in ps]
    tms = [to_torch(m, "float32") for m in ms]
    tvs = [to_torch(v, "float32") for v in vs]
    touts = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for n in numels]
    tl = rb.TensorList(numels, g_dtype, "bfloat16")
    for step in range(1, 11):
        gs = [make_grad(np.random.default_rng(50 * step + i), n, g_dtype) for i, n in enumerate(numels)]
        tgs = [to_torch(g, g_dtype) for g in gs]
        tl.bind(tgs, tps, tms, tvs, touts)
        rb.adam_list_(tl, step, 1e-4, 0.9, 0.95, 1e-8, 1, 0.1, mode)
        torch.cuda.synchronize()
        outs = [O.adam(g, p, m, v, step, 1e-4, 0.9, 0.95, 1e-8, 1, 0.1, mode, out_code=O.BF16)
                for g, p, m, v in zip(gs, ps, ms, vs)]
    for i in range(len(numels)):
        assert bits_equal(to_numpy(tps[i]), ps[i]), i
        assert bits_equal(to_numpy(tms[i]), ms[i]), i
        assert bits_equal(to_numpy(tvs[i]), vs[i]), i
        assert bits_equal(to_numpy(touts[i]), outs[i]), i
    tl.close()


# --------------------------------------------------------------------------- lans
LANS_HYPER = dict(learning_rate=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, bias_correction=1,
                  weight_decay=0.01, grad_averaging=1, mode=1, normalize_grad=1)


def _run_lans_case(rb, numels, g_dtype, out_dtype, hyper, steps, grad_scale=1.0, tune=None,
                   step_on_device=False):
    rng = np.random.default_rng(7)
    ps, ms, vs = zip(*[_params(rng, n) for n in numels])
    ps64 = [[p.copy(), m.copy(), v.copy()] for p, m, v in zip(ps, ms, vs)]  # double-norm oracle
    tps = [to_torch(p, "float32") for p in ps]
    tms = [to_torch(m, "float32") for m in ms]
    tvs = [to_torch(v, "float32") for v in vs]
    touts = [torch.zeros(n, dtype=TORCH[out_dtype], device="cuda") for n in numels]
    tl = rb.TensorList(numels, g_dtype, out_dtype)
    if tune:
        tl.tune(**tune)
    okw = dict(lr=hyper["learning_rate"], **{k: v for k, v in hyper.items() if k != "learning_rate"})
    for step in range(1, steps + 1):
        gs = [make_grad(np.random.default_rng(70 * step + i), n, g_dtype, loss_scale=1.0 / grad_scale)
              for i, n in enumerate(numels)]
        tgs = [to_torch(g, g_dtype) for g in gs]
        tl.bind(tgs, tps, tms, tvs, touts)
        dev_step = torch.tensor(float(step), device="cuda") if step_on_device else step
        rb.lans_list_(tl, dev_step, grad_scale=grad_scale, **hyper)
        norms = rb.lans_status(tl, want_norms=True)
        outs, onorms = O.lans(gs, list(ps), list(ms), list(vs), step, grad_scale=grad_scale,
                              norm_mode=0, out_code=CODES[out_dtype], **okw)
        O.lans(gs, [a[0] for a in ps64], [a[1] for a in ps64], [a[2] for a in ps64], step,
               grad_scale=grad_scale, norm_mode=2, **okw)
        nz = [i for i, n in enumerate(numels) if n > 0]
        # ||g|| is only computed (phase A) when gradients are normalised.  ||update_m|| of a
        # tiny tensor can be the difference of two O(1) terms (m/denom and wd*p cancel), which
        # amplifies the 1-ulp differences of the kernel's reciprocal arithmetic: 2e-5 here,
        # while p, m and v below are held to 1e-5 and, in practice, sit near 1e-7.
        cols = [0, 1, 2, 3] if hyper["normalize_grad"] else [1, 2, 3]
        big = [i for i in nz if numels[i] >= 1000]
        assert np.allclose(norms[big][:, cols], onorms[big][:, cols], rtol=2e-5, atol=0), (step, norms, onorms)
        assert np.allclose(norms[nz][:, :2], onorms[nz][:, :2], rtol=2e-6, atol=0) or not hyper["normalize_grad"]
    worst = 0.0
    for i, n in enumerate(numels):
        for ours, ref, ref64 in ((tps[i], ps[i], ps64[i][0]), (tms[i], ms[i], ps64[i][1]),
                                 (tvs[i], vs[i], ps64[i][2])):
            e = rel_err(to_numpy(ours), ref)
            worst = max(worst, e)
            assert e < 1e-5, (i, n, e)
            assert rel_err(to_numpy(ours), ref64) < 1e-5  # also inside the band of the exact-norm oracle
        if n:
            # the 16-bit copy is the cast of the fp32 value this kernel produced
            want = O.cast(to_numpy(tps[i]), CODES[out_dtype]) if out_dtype != "float32" else to_numpy(tps[i])
            assert bits_equal(to_numpy(touts[i]), want)
    tl.close()
    return worst


@pytest.mark.parametrize("g_dtype,out_dtype", [("float32", "float32"), ("float16", "float16"),
                                               ("bfloat16", "bfloat16")])
def test_lans_ten_steps(rb, g_dtype, out_dtype):
    numels = [0, 1, 3, 5, 1024, 4096, 4097, 65537, 300001, 2]
    scale = 2.0 ** -15 if g_dtype == "float16" else 1.0
    _run_lans_case(rb, numels, g_dtype, out_dtype, LANS_HYPER, 10, grad_scale=scale)


@pytest.mark.parametrize("hyper_delta", [dict(mode=0), dict(normalize_grad=0), dict(bias_correction=0),
                                         dict(grad_averaging=0), dict(weight_decay=0.0)])
def test_lans_flags(rb, hyper_delta):
    hyper = dict(LANS_HYPER)
    hyper.update(hyper_delta)
    _run_lans_case(rb, [7, 5000, 123457], "float32", "float32", hyper, 3)


@pytest.mark.parametrize("n", EDGE_NUMELS[1:])
def test_lans_edge_sizes(rb, n):
    _run_lans_case(rb, [n], "float16", "float16", LANS_HYPER, 2, grad_scale=2.0 ** -15)


def test_lans_schedules_give_identical_bits(rb):
    """The order of the work items (lead, gap, grid size - and with it which chunks stay on chip
    and which are streamed twice) must not change a single bit."""
    numels = [100, 9000, 70000, 400003, 1, 33000]
    results = []
    for tune in (dict(lead_elems=8 << 20, gap_items=0, max_blocks=0),
                 dict(lead_elems=0, gap_items=1, max_blocks=0),
                 dict(lead_elems=1 << 20, gap_items=50, max_blocks=7),
                 dict(lead_elems=1 << 30, gap_items=100000, max_blocks=1)):
        rng = np.random.default_rng(8)
        ps, ms, vs = zip(*[_params(rng, n) for n in numels])
        tps = [to_torch(p, "float32") for p in ps]
        tms = [to_torch(m, "float32") for m in ms]
        tvs = [to_torch(v, "float32") for v in vs]
        tl = rb.TensorList(numels, "float32", "float32")
        tl.tune(**tune)
        for step in range(1, 4):
            tgs = [to_torch(make_grad(np.random.default_rng(90 * step + i), n, "float32"), "float32")
                   for i, n in enumerate(numels)]
            tl.bind(tgs, tps, tms, tvs, None)
            rb.lans_list_(tl, step, **LANS_HYPER)
            rb.lans_status(tl)
        results.append([to_numpy(t) for t in tps + tms + tvs])
        tl.close()
    for other in results[1:]:
        for a, b in zip(results[0], other):
            assert bits_equal(a, b)


def test_lans_unaligned_views(rb):
    """Tensors that are only element-aligned cannot use bulk copies: the kernel reads them
    with plain loads.  Mixed with aligned tensors in one list."""
    rng = np.random.default_rng(21)
    numels = [5000, 4096, 9001, 70000]
    offs = [1, 0, 3, 2]
    ps, ms, vs = zip(*[_params(rng, n) for n in numels])
    gs = [make_grad(rng, n, "float16", loss_scale=2.0 ** 15) for n in numels]

    def view(arr, off, dtype):
        base = torch.zeros(arr.size + 8, dtype=dtype, device="cuda")
        v = base[off:off + arr.size]
        v.copy_(torch.from_numpy(arr))
        return base, v

    keep, tg, tp, tm, tv, to = [], [], [], [], [], []
    for g, p, m, v, off in zip(gs, ps, ms, vs, offs):
        for lst, arr, dt in ((tg, g, torch.float16), (tp, p, torch.float32), (tm, m, torch.float32),
                             (tv, v, torch.float32)):
            b, vw = view(arr, off, dt)
            keep.append((b, off, arr.size))
            lst.append(vw)
        b, vw = view(np.zeros(p.size, np.float16), off, torch.float16)
        keep.append((b, off, p.size))
        to.append(vw)
    tl = rb.TensorList(numels, "float16", "float16")
    tl.bind(tg, tp, tm, tv, to)
    rb.lans_list_(tl, 1, grad_scale=2.0 ** -15, **LANS_HYPER)
    rb.lans_status(tl)
    okw = dict(lr=LANS_HYPER["learning_rate"], **{k: v for k, v in LANS_HYPER.items() if k != "learning_rate"})
    outs, _ = O.lans(gs, list(ps), list(ms), list(vs), 1, grad_scale=2.0 ** -15, out_code=O.F16, **okw)
    for i in range(len(numels)):
        assert rel_err(to_numpy(tp[i]), ps[i]) < 1e-5
        assert rel_err(to_numpy(tm[i]), ms[i]) < 1e-5
        assert rel_err(to_numpy(tv[i]), vs[i]) < 1e-5
        assert bits_equal(to_numpy(to[i]), O.cast(to_numpy(tp[i]), O.F16))
    for b, off, n in keep:  # canaries: the words on either side of every view are still zero
        assert int(torch.count_nonzero(b[:off])) == 0 and int(torch.count_nonzero(b[off + n:])) == 0
    tl.close()


def test_lans_step_on_device(rb):
    """step as a 0-d fp32 device tensor (python/raf/optim/lans.py:239), no host round trip."""
    _run_lans_case(rb, [4099, 65536], "float32", "float32", LANS_HYPER, 4, step_on_device=True)


def test_lans_op_fp32_only_like_reference(rb):
    """src/op/dialect/cuda/lans.cc:38-40: "LANS only takes FP32 inputs"; list length % 4."""
    t = [torch.zeros(8, device="cuda", dtype=torch.float16) for _ in range(4)]
    with pytest.raises(TypeError):
        rb.lans(t, 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1)
    with pytest.raises(ValueError):
        rb.lans([torch.zeros(8, device="cuda")] * 3, 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1)


def test_lans_op_eager_simple(rb):
    """tests/python/optim/test_lans.py::test_traced_lans_simple shape: a (2,2) parameter, 4 steps."""
    rng = np.random.default_rng(9)
    p = rng.standard_normal((2, 2)).astype(np.float32)
    m = np.zeros((2, 2), np.float32)
    v = np.zeros((2, 2), np.float32)
    tp, tm, tv = (torch.from_numpy(a.copy()).cuda() for a in (p, m, v))
    for step in range(1, 5):
        g = rng.standard_normal((2, 2)).astype(np.float32)
        rb.lans([torch.from_numpy(g).cuda(), tp, tm, tv], step, 1e-3, 0.9, 0.999, 1e-6, True, 0.01,
                True, True, True)
        O.lans([g], [p], [m], [v], step)
    np.testing.assert_allclose(tp.cpu().numpy(), p, rtol=1e-4, atol=1e-4)  # the reference's tolerance
    assert rel_err(tp.cpu().numpy(), p) < 1e-5


def test_lans_workspace_too_small_is_rejected(rb):
    import ctypes as C

    from raf_b200 import _lib

    tl = rb.TensorList([4096], "float32", "float32")
    t = [torch.zeros(4096, device="cuda") for _ in range(4)]
    tl.bind([t[0]], [t[1]], [t[2]], [t[3]], None)
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = _lib.load().rafb200_lans(tl.handle, 1, None, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, 1.0,
                                  ws.data_ptr(), 16, None)
    assert rc == 1 and b"workspace" in _lib.load().rafb200_last_error()
    tl.close()


# --------------------------------------------------------------------------- reference kernel on the GPU
def test_lans_against_reference_kernel(rb):
    """The reference's own multi_tensor_lans_cuda<float> (oracle/_ref) on the same device
    buffers: pins the CPU oracle AND this repository's kernel to the real implementation."""
    from oracle import ref_lans

    if not ref_lans.available():
        pytest.skip("oracle/_ref/libraf_ref_lans.so was not built (reference tree absent at build time)")
    numels = [5, 1027, 4099, 66001, 131072, 300000]
    rng = np.random.default_rng(10)
    ps, ms, vs = zip(*[_params(rng, n) for n in numels])
    ours = [[to_torch(a, "float32") for a in xs] for xs in (ps, ms, vs)]
    theirs = [[to_torch(a, "float32") for a in xs] for xs in (ps, ms, vs)]
    cpu = [[a.copy() for a in xs] for xs in (ps, ms, vs)]
    ref = ref_lans.RefLans(numels)
    tl = rb.TensorList(numels, "float32", "float32")
    for step in range(1, 6):
        gs = [make_grad(np.random.default_rng(110 * step + i), n, "float32") for i, n in enumerate(numels)]
        tg_ours = [to_torch(g, "float32") for g in gs]
        tg_ref = [to_torch(g, "float32") for g in gs]
        tl.bind(tg_ours, ours[0], ours[1], ours[2], None)
        rb.lans_list_(tl, step, **LANS_HYPER)
        norms = rb.lans_status(tl, want_norms=True)
        ref(tg_ref, theirs[0], theirs[1], theirs[2], step)
        torch.cuda.synchronize()
        _, onorms = O.lans(gs, cpu[0], cpu[1], cpu[2], step, norm_mode=1)
        rnorms = ref.norms_host()
        assert np.allclose(norms, rnorms, rtol=2e-6)
        assert np.allclose(onorms, rnorms, rtol=2e-6)
    for a in range(3):
        for i in range(len(numels)):
            r = to_numpy(theirs[a][i])
            assert rel_err(to_numpy(ours[a][i]), r) < 1e-5, (a, i)
            assert rel_err(cpu[a][i], r) < 1e-5, (a, i)
    tl.close()


# --------------------------------------------------------------------------- casts, packing
@pytest.mark.parametrize("src", G_DTYPES)
@pytest.mark.parametrize("dst", G_DTYPES)
def test_cast_bit_exact(rb, src, dst):
    rng = np.random.default_rng(11)
    for n in (0, 1, 7, 4096, 100003):
        x = make_grad(rng, n, src, std=1.0)
        out = rb.cast(to_torch(x, src), dst)
        torch.cuda.synchronize()
        want = O.cast(x, CODES[dst]) if src != dst else x
        assert bits_equal(to_numpy(out), want), (n,)


def test_group_cast_many_tensors(rb):
    rng = np.random.default_rng(12)
    numels = [int(x) for x in rng.integers(0, 5000, size=230)] + [200003]
    xs = [make_grad(rng, n, "float16", std=1.0) for n in numels]
    outs = rb.group_cast([to_torch(x, "float16") for x in xs], "float32")
    torch.cuda.synchronize()
    for x, o in zip(xs, outs):
        assert bits_equal(to_numpy(o), O.cast(x, O.F32))


def test_fuse_defuse_round_trip(rb):
    rng = np.random.default_rng(13)
    shapes = [(3, 5), (7,), (128, 33), (1,), (64, 3, 3, 3)]
    ts = [torch.from_numpy(rng.standard_normal(s).astype(np.float32)).cuda() for s in shapes]
    flat = rb.fuse_tensor(ts)
    torch.cuda.synchronize()
    assert torch.equal(flat, torch.cat([t.reshape(-1) for t in ts]))
    sizes = [t.numel() for t in ts]
    flat_shapes = [d for s in shapes for d in s]
    idx = list(np.cumsum([len(s) for s in shapes]))
    back = rb.defuse_tensor(flat, sizes, flat_shapes, idx)
    torch.cuda.synchronize()
    for a, b in zip(ts, back):
        assert a.shape == b.shape and torch.equal(a, b)


def test_lans_bounded_wait_reports_instead_of_hanging(rb):
    """A work-item table whose only item is a streamed update (kind 2): the norms it waits for
    are never produced.  The kernel must give up after the wait limit, report
    RAFB200_DEVICE_WAIT_EXPIRED through rafb200_lans_status, and leave the context usable:
    with the built-in order restored the same list updates correctly."""
    from raf_b200 import _lib

    n = 5000
    rng = np.random.default_rng(31)
    p, m, v = _params(rng, n)
    g = make_grad(rng, n, "float32")
    tp, tm, tv, tg = (to_torch(a, "float32") for a in (p, m, v, g))
    tl = rb.TensorList([n], "float32", "float32")
    tl.bind([tg], [tp], [tm], [tv], None)
    tl.set_wait_limit(50)
    tl.set_lans_items(np.array([[2 << 30, 0]], np.uint32))
    rb.lans_list_(tl, 1, **LANS_HYPER)
    with pytest.raises(_lib.RafB200Error) as err:
        rb.lans_status(tl)
    assert err.value.status == 5  # RAFB200_DEVICE_WAIT_EXPIRED
    assert bits_equal(to_numpy(tp), p)  # nothing was written
    tl.tune()  # back to the built-in order
    rb.lans_list_(tl, 1, **LANS_HYPER)
    rb.lans_status(tl)
    okw = dict(lr=LANS_HYPER["learning_rate"], **{k: v for k, v in LANS_HYPER.items() if k != "learning_rate"})
    O.lans([g], [p], [m], [v], 1, **okw)
    assert rel_err(to_numpy(tp), p) < 1e-5 and rel_err(to_numpy(tm), m) < 1e-5
    tl.close()
