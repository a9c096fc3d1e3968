"""The ZeRO step driver on one GPU (world of one: collectives degenerate, the update
runs as one launch over all tensors) against the oracle, device- and host-buffer forms."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import CODES, TORCH, bits_equal, make_grad, rel_err, to_numpy, to_torch

pytestmark = pytest.mark.gpu

SHAPES = [(30, 16), (16,), (7, 3, 3), (1,), (129, 65), (4096,), (50, 1024)]


def _setup(optimizer, g_dtype, p_dtype):
    from raf_b200 import distributed as dist
    from raf_b200.zero import Plan, ZeroStep, numel

    comm = dist.get_communicator()
    plan = Plan(SHAPES, 1, 0, 5000)
    z = ZeroStep(plan, comm, g_dtype, p_dtype, optimizer)
    rng = np.random.default_rng(0)
    p = [(rng.standard_normal(numel(s)) * 0.02).astype(np.float32) for s in SHAPES]
    m = [np.zeros_like(x) for x in p]
    v = [np.zeros_like(x) for x in p]
    return plan, z, p, m, v


@pytest.mark.parametrize("optimizer,g_dtype,p_dtype", [("sgd", "float32", "float32"),
                                                       ("adam", "bfloat16", "bfloat16"),
                                                       ("lans", "float16", "float16")])
def test_zero_step_single_rank(optimizer, g_dtype, p_dtype):
    from raf_b200.zero import make_hyper, numel

    plan, z, p, m, v = _setup(optimizer, g_dtype, p_dtype)
    tp = [to_torch(x, "float32") for x in p]
    tm = [to_torch(x, "float32") for x in m]
    tv = [to_torch(x, "float32") for x in v]
    params = [torch.zeros(numel(s), dtype=TORCH[p_dtype], device="cuda") for s in SHAPES]
    scale = 2.0 ** -15 if g_dtype == "float16" else 1.0
    kw = dict(learning_rate=0.1 if optimizer == "sgd" else 1e-3, mu=0.9, beta1=0.9, beta2=0.999,
              eps=1e-6, weight_decay=0.01, grad_scale=scale)
    hyper = make_hyper(optimizer, **kw)
    for step in range(1, 6):
        g = [make_grad(np.random.default_rng(100 * step + i), numel(s), g_dtype, loss_scale=1 / scale)
             for i, s in enumerate(SHAPES)]
        tg = [to_torch(x, g_dtype) for x in g]
        z.bind(tg, params, tp, tm, tv)
        z.step(hyper, step)
        torch.cuda.synchronize()
        if optimizer == "sgd":
            outs = [O.sgd(p[i], g[i], m[i], 0.1, 0.9, 0.01, scale, out_code=CODES[p_dtype]) for i in range(len(p))]
        elif optimizer == "adam":
            outs = [O.adam(g[i], p[i], m[i], v[i], step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, scale,
                           out_code=CODES[p_dtype]) for i in range(len(p))]
        else:
            outs, _ = O.lans(g, p, m, v, step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, scale,
                             out_code=CODES[p_dtype])
    kernels, collectives = z.launch_counts()
    assert kernels == 1 and collectives == 0
    for i in range(len(p)):
        if optimizer == "lans":
            assert rel_err(to_numpy(tp[i]), p[i]) < 1e-5
            assert rel_err(to_numpy(tm[i]), m[i]) < 1e-5
            assert rel_err(to_numpy(tv[i]), v[i]) < 1e-5
        else:
            assert bits_equal(to_numpy(tp[i]), p[i])
            assert bits_equal(to_numpy(tm[i]), m[i])
            assert bits_equal(to_numpy(params[i]), outs[i])
    z.close()


def test_zero_step_host_buffers():
    """Gradients from pinned host memory in, model-dtype parameters back out."""
    from raf_b200.zero import make_hyper, numel

    plan, z, p, m, v = _setup("lans", "float16", "float16")
    tp = [to_torch(x, "float32") for x in p]
    tm = [to_torch(x, "float32") for x in m]
    tv = [to_torch(x, "float32") for x in v]
    grads_dev = [torch.zeros(numel(s), dtype=torch.float16, device="cuda") for s in SHAPES]
    params_dev = [torch.zeros(numel(s), dtype=torch.float16, device="cuda") for s in SHAPES]
    z.bind(grads_dev, params_dev, tp, tm, tv)
    hyper = make_hyper("lans", learning_rate=1e-3, weight_decay=0.01, grad_scale=2.0 ** -15)
    g = [make_grad(np.random.default_rng(7 + i), numel(s), "float16", loss_scale=2.0 ** 15)
         for i, s in enumerate(SHAPES)]
    grads_host = [torch.from_numpy(x.copy()).pin_memory() for x in g]
    params_host = [torch.zeros(numel(s), dtype=torch.float16).pin_memory() for s in SHAPES]
    z.step_host(hyper, 1, grads_host, params_host)
    torch.cuda.synchronize()
    outs, _ = O.lans(g, p, m, v, 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, 2.0 ** -15, out_code=O.F16)
    for i in range(len(p)):
        assert rel_err(params_host[i].numpy().astype(np.float32), outs[i].astype(np.float32)) < 2e-3
        assert rel_err(to_numpy(tp[i]), p[i]) < 1e-5
        assert torch.equal(params_host[i], params_dev[i].cpu())
    z.close()
