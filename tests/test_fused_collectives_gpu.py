"""The update kernels with the collectives inside (rafb200_tensor_list_set_symmetric), on ONE GPU:
the buffers of three "ranks" are three allocations on the same device, and the kernel of "rank" r
is a single launch over them - nothing waits for another launch.  Checked: the gradient the
kernel wrote back is the sum over the ranks (fp32 accumulation, one rounding), the state equals
the oracle's on that sum (bit for bit for SGD and Adam, 1e-5 for LANS), and the model-dtype copy
arrived in every rank's parameter buffer.  The real multi-GPU runs (with the NVSwitch multicast
forms, which one GPU cannot emulate) are tests/test_dist_gpu.py."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import CODES, TORCH, bits_equal, rel_err, to_numpy

pytestmark = pytest.mark.gpu

WORLD = 3
# element counts of the "shards": ragged, below and above one chunk, one above an A item of LANS
NUMELS = [5, 1024, 4099, 7168 + 13, 40000, 1, 0, 12288]


def layout(numels, elem_size):
    """Byte offset of every tensor inside the symmetric buffer: regions padded to 16 bytes."""
    offs, at = [], 0
    for n in numels:
        offs.append(at)
        at += ((n * elem_size + 15) // 16) * 16
    return offs, max(at, 16)


def setup(g_dtype, p_dtype, rank, seed):
    rng = np.random.default_rng(seed)
    gs, ps = torch.empty((), dtype=TORCH[g_dtype]).element_size(), torch.empty((), dtype=TORCH[p_dtype]).element_size()
    g_off, g_bytes = layout(NUMELS, gs)
    p_off, p_bytes = layout(NUMELS, ps)
    # every rank's gradient buffer: small integers times 2^-10, so that sums are exact in any dtype
    gbufs = [torch.zeros(g_bytes // gs, dtype=TORCH[g_dtype], device="cuda") for _ in range(WORLD)]
    total = []
    for i, n in enumerate(NUMELS):
        acc = np.zeros(n, np.float32)
        for q in range(WORLD):
            k = rng.integers(-15, 16, size=n).astype(np.float32) * np.float32(2.0 ** -10)
            gbufs[q][g_off[i] // gs:g_off[i] // gs + n] = torch.from_numpy(k).to(TORCH[g_dtype]).cuda()
            acc += k
        total.append(acc)
    pbufs = [torch.zeros(p_bytes // ps, dtype=TORCH[p_dtype], device="cuda") for _ in range(WORLD)]
    gred = torch.full((g_bytes // gs,), 7.0, dtype=TORCH[g_dtype], device="cuda")  # the kernel overwrites it
    p = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in NUMELS]
    tp = [torch.from_numpy(x.copy()).cuda() for x in p]
    tm = [torch.zeros(n, device="cuda") for n in NUMELS]
    tv = [torch.zeros(n, device="cuda") for n in NUMELS]
    g_views = [gred[g_off[i] // gs:g_off[i] // gs + n] for i, n in enumerate(NUMELS)]
    out_views = [pbufs[rank][p_off[i] // ps:p_off[i] // ps + n] for i, n in enumerate(NUMELS)]
    return dict(gbufs=gbufs, pbufs=pbufs, gred=gred, g_off=g_off, p_off=p_off, gs=gs, ps=ps, total=total, p=p,
                tp=tp, tm=tm, tv=tv, g_views=g_views, out_views=out_views)


def make_list(s, g_dtype, p_dtype, rank, with_v, all_gather=True):
    from raf_b200 import op

    tl = op.TensorList(NUMELS, g_dtype, p_dtype)
    tl.set_symmetric(rank, [b.data_ptr() for b in s["gbufs"]], [b.data_ptr() for b in s["pbufs"]], s["g_off"],
                     reduce_scatter=True, all_gather=all_gather)
    tl.bind(s["g_views"], s["tp"], s["tm"], s["tv"] if with_v else None, s["out_views"])
    return tl


def check_common(s, g_dtype, p_dtype, rank, want_p, copies_everywhere=True):
    for i, n in enumerate(NUMELS):
        want_g = O.cast(s["total"][i], CODES[g_dtype]) if g_dtype != "float32" else s["total"][i]
        assert bits_equal(to_numpy(s["g_views"][i]), want_g), ("reduced gradient", i)
        want_out = O.cast(want_p[i], CODES[p_dtype]) if p_dtype != "float32" else want_p[i]
        lo = s["p_off"][i] // s["ps"]
        for q in range(WORLD):
            got = to_numpy(s["pbufs"][q][lo:lo + n])
            if q == rank or copies_everywhere:
                assert bits_equal(got, want_out), ("parameter copy", i, q)
            else:
                assert not got.any(), ("a copy reached rank", q, "although the all-gather is off")


@pytest.mark.parametrize("g_dtype,p_dtype", [("float32", "float32"), ("float16", "float16"), ("bfloat16", "bfloat16")])
@pytest.mark.parametrize("rank", [0, 2])
def test_sgd_and_adam_read_the_sum_and_store_everywhere(g_dtype, p_dtype, rank):
    from raf_b200 import op

    for optimizer in ("sgd", "adam"):
        s = setup(g_dtype, p_dtype, rank, seed=11)
        tl = make_list(s, g_dtype, p_dtype, rank, with_v=(optimizer == "adam"))
        m = [np.zeros(n, np.float32) for n in NUMELS]
        v = [np.zeros(n, np.float32) for n in NUMELS]
        p = [x.copy() for x in s["p"]]
        gscale = 1.0 / WORLD
        if optimizer == "sgd":
            op.sgd_list_(tl, 0.1, 0.9, weight_decay=0.01, grad_scale=gscale)
        else:
            op.adam_list_(tl, 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, grad_scale=gscale)
        torch.cuda.synchronize()
        for i in range(len(NUMELS)):
            g = O.cast(s["total"][i], CODES[g_dtype]) if g_dtype != "float32" else s["total"][i]
            if optimizer == "sgd":
                O.sgd(p[i], g, m[i], 0.1, 0.9, 0.01, gscale)
            else:
                O.adam(g, p[i], m[i], v[i], 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, gscale)
            assert bits_equal(to_numpy(s["tp"][i]), p[i]) and bits_equal(to_numpy(s["tm"][i]), m[i]), (optimizer, i)
            if optimizer == "adam":
                assert bits_equal(to_numpy(s["tv"][i]), v[i])
        check_common(s, g_dtype, p_dtype, rank, p)
        tl.close()


@pytest.mark.parametrize("g_dtype,p_dtype", [("float16", "float16"), ("float32", "float32")])
@pytest.mark.parametrize("all_gather", [True, False])
def test_lans_reads_the_sum_in_its_norm_pass_and_stores_everywhere(g_dtype, p_dtype, all_gather):
    from raf_b200 import op

    rank = 1
    s = setup(g_dtype, p_dtype, rank, seed=12)
    tl = make_list(s, g_dtype, p_dtype, rank, with_v=True, all_gather=all_gather)
    m = [np.zeros(n, np.float32) for n in NUMELS]
    v = [np.zeros(n, np.float32) for n in NUMELS]
    p = [x.copy() for x in s["p"]]
    gscale = 1.0 / WORLD
    for step in (1, 2):  # the gradient buffers stay as they are: the kernel writes only its own block
        op.lans_list_(tl, step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, grad_scale=gscale)
        op.lans_status(tl)
        g = [O.cast(t, CODES[g_dtype]) if g_dtype != "float32" else t for t in s["total"]]
        O.lans(g, p, m, v, step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, gscale)
    for i in range(len(NUMELS)):
        assert rel_err(to_numpy(s["tp"][i]), p[i]) < 1e-5 and rel_err(to_numpy(s["tm"][i]), m[i]) < 1e-5, i
        assert rel_err(to_numpy(s["tv"][i]), v[i]) < 1e-5, i
    # the copies are cast(p) of what the kernel itself computed
    check_common(s, g_dtype, p_dtype, rank, [to_numpy(t) for t in s["tp"]], copies_everywhere=all_gather)
    tl.close()


def test_lans_without_the_norm_pass_is_refused():
    from raf_b200 import _lib, op

    s = setup("float16", "float16", 0, seed=13)
    tl = make_list(s, "float16", "float16", 0, with_v=True)
    with pytest.raises(_lib.RafB200Error):
        op.lans_list_(tl, 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 0)
    tl.close()
