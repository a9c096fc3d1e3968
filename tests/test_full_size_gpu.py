"""Parity at the full sizes of the benchmark configurations.

Config 1 (one flat fp32 tensor of 25,557,032 elements, SGD-momentum, 10 steps) runs always: the
oracle needs a fraction of a second per step, so every element is compared, bit for bit.
The BERT-large LANS and GPT-2-medium Adam lists at full size (about 10 GB of host arrays and half
a minute each) run when RAFB200_FULL_SIZE_TESTS=1.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import bits_equal, make_grad, to_numpy, to_torch

pytestmark = pytest.mark.gpu
FULL = pytest.mark.skipif(os.environ.get("RAFB200_FULL_SIZE_TESTS") != "1",
                          reason="set RAFB200_FULL_SIZE_TESTS=1 (10 GB of host memory, ~1 minute)")


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


@FULL
def test_config3_bert_large_lans_one_step_full_size():
    from raf_b200 import op
    from raf_b200.zero import bert_large_shapes, numel
    from tests.test_kernels_gpu import LANS_HYPER, _run_lans_case

    numels = [numel(s) for s in bert_large_shapes()]
    assert sum(numels) == 335141888
    worst = _run_lans_case(op, numels, "float16", "float16", LANS_HYPER, 1, grad_scale=2.0 ** -15)
    assert worst < 1e-5


@FULL
def test_config4_gpt2_medium_adam_one_step_full_size():
    from raf_b200 import op
    from raf_b200.zero import gpt2_medium_shapes, numel

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
