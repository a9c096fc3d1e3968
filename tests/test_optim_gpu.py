"""The optimizer classes mirrored from raf.optim, checked the way the reference checks its own:
SGD against torch.optim.SGD(lr=0.1, momentum=0.01) (tests/python/optim/test_sgd.py:80-125, 1e-4
there; the kernel is exact, so the bar here is 1e-6), LANS against the CPU oracle, and the
ZeRO-aware wrappers for their state names and shard shapes (test_sgd.py:283-302,
test_lans.py:247-266)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import rel_err, to_numpy

pytestmark = pytest.mark.gpu

SHAPES = [(64, 3, 3, 3), (64,), (10, 64), (10,), (7, 5)]


def _params(seed=0):
    rng = np.random.default_rng(seed)
    return [torch.from_numpy((rng.standard_normal(s) * 0.1).astype(np.float32)).cuda() for s in SHAPES]


def test_sgd_matches_torch_sgd():
    from raf_b200.optim import SGD

    ours = _params()
    theirs = [p.clone().requires_grad_(True) for p in ours]
    opt = SGD(ours, 0.1, 0.01)
    ref = torch.optim.SGD(theirs, lr=0.1, momentum=0.01)
    assert sorted(opt.state()) == sorted(f"sgd.{i}.v" for i in range(len(SHAPES)))
    for step in range(5):
        rng = np.random.default_rng(100 + step)
        for a, b in zip(ours, theirs):
            g = torch.from_numpy(rng.standard_normal(tuple(a.shape)).astype(np.float32) * 1e-2).cuda()
            a.grad = g
            b.grad = g.clone()
        opt.step()
        ref.step()
    for a, b in zip(ours, theirs):
        assert rel_err(to_numpy(a), to_numpy(b)) < 1e-6
    with pytest.raises(ValueError):
        SGD(ours, -1.0)
    with pytest.raises(ValueError):
        SGD(ours, 0.1, -0.5)


def test_lans_matches_oracle_and_counts_steps_from_one():
    from raf_b200.optim import LANS

    ours = _params(1)
    p = [to_numpy(x).reshape(-1) for x in ours]
    m = [np.zeros_like(x) for x in p]
    v = [np.zeros_like(x) for x in p]
    opt = LANS(ours)
    assert opt._step == 1
    for step in range(1, 4):
        rng = np.random.default_rng(200 + step)
        g = [(rng.standard_normal(x.size) * 1e-2).astype(np.float32) for x in p]
        for a, gi in zip(ours, g):
            a.grad = torch.from_numpy(gi).cuda().reshape(a.shape)
        opt.step()
        O.lans(g, p, m, v, step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, 1.0)
    assert opt._step == 4
    for a, b in zip(ours, p):
        assert rel_err(to_numpy(a).reshape(-1), b) < 1e-5
    for i, b in enumerate(m):
        assert rel_err(to_numpy(opt.state()[f"lans.{i}.m"]).reshape(-1), b) < 1e-5
    with pytest.raises(TypeError):
        half = [x.half() for x in ours]
        for h in half:
            h.grad = torch.zeros_like(h)
        LANS(half).step()


@pytest.mark.parametrize("which", ["sgd", "lans"])
def test_zero_wrappers_state_names_and_update(which):
    from raf_b200 import distributed as dist
    from raf_b200.optim import with_lans, with_sgd

    dist.get_config().zero_opt_level = 1
    try:
        names = [f"layer{i}.w" for i in range(len(SHAPES))]
        model = dict(zip(names, _params(2)))
        before = [to_numpy(x).reshape(-1) for x in model.values()]
        wrap = (with_sgd(0.1, 0.01) if which == "sgd" else with_lans())(model)
        want = {f"{n}.sgd_w" for n in names} | {f"{n}.sgd_v" for n in names} if which == "sgd" else \
            {f"{n}.lans_w" for n in names} | {f"{n}.m" for n in names} | {f"{n}.v" for n in names}
        assert set(wrap.state) == want
        for n, s in zip(names, SHAPES):  # a world of one: the shard is the whole tensor
            assert wrap.state[f"{n}.{which}_w"].numel() == int(np.prod(s))
        rng = np.random.default_rng(5)
        g = [(rng.standard_normal(x.size) * 1e-2).astype(np.float32) for x in before]
        wrap.step([torch.from_numpy(x).cuda() for x in g])
        torch.cuda.synchronize()
        p = [x.copy() for x in before]
        m = [np.zeros_like(x) for x in p]
        v = [np.zeros_like(x) for x in p]
        if which == "sgd":
            for i in range(len(p)):
                O.sgd(p[i], g[i], m[i], 0.1, 0.01)
        else:
            O.lans(g, p, m, v, 1, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, 1.0)
        for x, b in zip(model.values(), p):
            assert rel_err(to_numpy(x).reshape(-1), b) < 1e-5  # the model's own tensors were updated
        wrap.close()
    finally:
        dist.get_config().zero_opt_level = 0
