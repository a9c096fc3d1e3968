"""Parity at the full sizes of the benchmark configurations.

Config 1 (one flat fp32 tensor of 25,557,032 elements, SGD-momentum, 10 steps): every element
is compared, bit for bit.  Config 3 (the BERT-large LANS list, 335,141,888 elements) and config 4
(the GPT-2-medium Adam list, 354,823,168 elements): one step over the whole list, every element
compared.  Config 5: one flat tensor of 64 Mi and of 512 Mi elements, windows and strided samples.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import bits_equal, make_grad, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def test_config1_flat_sgd_ten_steps_full_size():
    from raf_b200 import op

    n = 25557032
    rng = np.random.default_rng(0)
    p = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02))
    v = np.zeros(n, np.float32)
    tp, tv = to_torch(p, "float32"), to_torch(v, "float32")
    for step in range(10):
        g = (np.random.default_rng(1 + step).standard_normal(n, dtype=np.float32) * np.float32(1e-3))
        tg = to_torch(g, "float32")
        op.sgd_(tp, tg, tv, 0.1, 0.9, weight_decay=1e-4)
        O.sgd(p, g, v, 0.1, 0.9, weight_decay=1e-4)
    torch.cuda.synchronize()
    assert bits_equal(to_numpy(tp), p)
    assert bits_equal(to_numpy(tv), v)


def test_config3_bert_large_lans_one_step_full_size():
    from raf_b200 import op
    from bench import bert_large_shapes, numel
    from tests.test_kernels_gpu import LANS_HYPER, _run_lans_case

    numels = [numel(s) for s in bert_large_shapes()]
    assert sum(numels) == 335141888
    worst = _run_lans_case(op, numels, "float16", "float16", LANS_HYPER, 1, grad_scale=2.0 ** -15)
    assert worst < 1e-5


def test_config4_gpt2_medium_adam_one_step_full_size():
    from raf_b200 import op
    from bench import gpt2_medium_shapes, numel

    numels = [numel(s) for s in gpt2_medium_shapes()]
    assert sum(numels) == 354823168
    rng = np.random.default_rng(6)
    ps = [(rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)) for n in numels]
    ms = [np.zeros(n, np.float32) for n in numels]
    vs = [np.zeros(n, np.float32) for n in numels]
    tps = [to_torch(x, "float32") for x in ps]
    tms = [to_torch(x, "float32") for x in ms]
    tvs = [to_torch(x, "float32") for x in vs]
    touts = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for n in numels]
    tl = op.TensorList(numels, "bfloat16", "bfloat16")
    gs = [make_grad(np.random.default_rng(50 + i), n, "bfloat16") for i, n in enumerate(numels)]
    tgs = [to_torch(g, "bfloat16") for g in gs]
    tl.bind(tgs, tps, tms, tvs, touts)
    op.adam_list_(tl, 1, 1e-4, 0.9, 0.95, 1e-8, 1, 0.1, 1)
    torch.cuda.synchronize()
    for i, n in enumerate(numels):
        out = O.adam(gs[i], ps[i], ms[i], vs[i], 1, 1e-4, 0.9, 0.95, 1e-8, 1, 0.1, 1, out_code=O.BF16)
        assert bits_equal(to_numpy(tps[i]), ps[i]), i
        assert bits_equal(to_numpy(tms[i]), ms[i]), i
        assert bits_equal(to_numpy(tvs[i]), vs[i]), i
        assert bits_equal(to_numpy(touts[i]), out), i
    tl.close()


@pytest.mark.parametrize("mi", [64, 512])
def test_config5_flat_adam_one_step_full_size(mi):
    """One flat fp32 tensor of 64 Mi / 512 Mi elements (the largest is 131,072 work items in one
    tensor, 2 GiB per array).  Adam is element-wise, so three windows of 4 Mi elements (start,
    an odd offset in the middle, end) are compared bit for bit with the oracle, and float64
    sums over strided samples of p, m, v catch anything that went wrong in between."""
    from raf_b200 import op

    n = mi << 20
    torch.cuda.empty_cache()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(mi)
    tp = torch.randn(n, generator=gen, device="cuda") * 0.02
    tg = torch.randn(n, generator=gen, device="cuda") * 1e-3
    tm = torch.randn(n, generator=gen, device="cuda") * 1e-4
    tv = torch.rand(n, generator=gen, device="cuda") * 1e-6
    win = 4 << 20
    mid = (n // 2 + 12345) | 1
    windows = [(0, win), (mid, mid + win), (n - win, n)]
    stride = 4099  # prime: samples fall on every position of the 4096-element work items
    before = [[to_numpy(t[lo:hi]) for t in (tg, tp, tm, tv)] for lo, hi in windows]
    samp = [to_numpy(t[::stride]) for t in (tg, tp, tm, tv)]
    tl = op.TensorList([n], "float32", "float32")
    tl.bind([tg], [tp], [tm], [tv], None)
    op.adam_list_(tl, 3, 1e-4, 0.9, 0.95, 1e-8, 1, 0.1, 1)
    torch.cuda.synchronize()
    for (lo, hi), (g, p, m, v) in zip(windows, before):
        O.adam(g, p, m, v, 3, 1e-4, 0.9, 0.95, 1e-8, 1, 0.1, 1)
        assert bits_equal(to_numpy(tp[lo:hi]), p), (mi, lo)
        assert bits_equal(to_numpy(tm[lo:hi]), m), (mi, lo)
        assert bits_equal(to_numpy(tv[lo:hi]), v), (mi, lo)
    g, p, m, v = samp
    O.adam(g, p, m, v, 3, 1e-4, 0.9, 0.95, 1e-8, 1, 0.1, 1)
    for ours, want in ((tp, p), (tm, m), (tv, v)):
        got = to_numpy(ours[::stride])
        assert bits_equal(got, want), mi
        assert float(got.astype(np.float64).sum()) == float(want.astype(np.float64).sum())
    tl.close()
    del tp, tg, tm, tv
    torch.cuda.empty_cache()
