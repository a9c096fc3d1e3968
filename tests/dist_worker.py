"""One rank of the multi-GPU tests (started by tests/test_dist_gpu.py, one process per GPU).

Environment: RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR, MASTER_PORT, RAF_FILE_STORE_PATH (id
exchange), OUT_DIR.
Part 1 checks the collectives against the known answers of the reference's own tests
(tests/python/distributed/test_collective_communication.py:73-121,230-255,637-754:
rank-valued inputs whose reductions are exact integers).  Part 2 runs the ZeRO step
for three steps per optimizer and writes what this rank ended with (state shards,
gathered parameters) to OUT_DIR for the parent to check against the oracle.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from raf_b200 import distributed as dist  # noqa: E402
from raf_b200.zero import Plan, ZeroStep, make_hyper, numel  # noqa: E402

SHAPES = [(30, 16), (16,), (7, 3, 3), (1,), (129, 65), (4096,), (50, 1024), (2, 8)]
BUCKET = 5000
CASES = [("sgd", "float32", "float32"), ("adam", "bfloat16", "bfloat16"), ("lans", "float16", "float16"),
         ("lans", "float32", "float32")]
TORCH = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
STEPS = 3


def local_grad(rank, step, i, n, dtype, loss_scale):
    """Rank-local gradient k * 2^-10 * loss_scale with integer |k| <= 15, a different seed per
    rank: sums over up to 8 ranks are exact in fp32, fp16 and bf16 whatever order NCCL adds in,
    so the parent can state the reduced gradient exactly."""
    rng = np.random.default_rng(1000 * rank + 100 * step + i)
    k = rng.integers(-15, 16, size=n).astype(np.float32)
    return torch.from_numpy(k * np.float32(2.0 ** -10 * loss_scale)).to(TORCH[dtype])


def check_collectives(comm):
    n, r = comm.size, comm.rank
    s = dist.comm_stream()
    with torch.cuda.stream(s):
        # _allreduce: every rank contributes ones * (rank + 1)
        for dtype in (torch.float32, torch.float16):
            x = torch.full((4, 4), float(r + 1), dtype=dtype, device="cuda")
            dist.allreduce(x, "sum", stream=s)
            assert torch.all(x == n * (n + 1) / 2), x
        x = torch.full((4, 4), float(r + 1), device="cuda")
        dist.allreduce(x, "avg", stream=s)
        assert torch.allclose(x, torch.full_like(x, (n + 1) / 2))
        pair = [torch.full((4, 4), float(r + 1), device="cuda"), torch.full((3,), float(-(r + 1)), device="cuda")]
        dist.allreduce(pair, "max", stream=s)
        assert torch.all(pair[0] == n) and torch.all(pair[1] == -1)
        # _allgather on axis 0 and 1
        x = torch.full((2, 3), float(r + 1), device="cuda")
        y = dist.allgather(x, 0, stream=s)
        assert y.shape == (2 * n, 3)
        assert torch.equal(y[:, 0].cpu(), torch.arange(1, n + 1).repeat_interleave(2).float())
        y = dist.allgather(x, 1, stream=s)
        assert y.shape == (2, 3 * n)
        assert torch.equal(y[0].cpu(), torch.arange(1, n + 1).repeat_interleave(3).float())
        # _reduce_scatter: rank j receives row block j of the sum
        x = (torch.arange(n * 2, device="cuda").float().reshape(n * 2, 1) + 1) * (r + 1)
        y = dist.reduce_scatter(x.expand(n * 2, 4).contiguous(), "sum", stream=s)
        want = (torch.arange(2 * r, 2 * r + 2).float() + 1) * (n * (n + 1) / 2)
        assert y.shape == (2, 4) and torch.equal(y[:, 0].cpu(), want), (y, want)
        for comp, red in (("min", min), ("max", max), ("prod", None)):
            x = torch.full((n, 2), float(r + 1), device="cuda")
            y = dist.reduce_scatter(x, comp, stream=s)
            if red is not None:
                assert torch.all(y == red(range(1, n + 1)))
            else:
                assert torch.all(y == float(np.prod(np.arange(1, n + 1))))
        # _group_reduce_scatter / _group_allgather on lists of different sizes, fp16 too
        for dtype in (torch.float32, torch.float16):
            xs = [torch.full((n * k, 3), float(r + 1), dtype=dtype, device="cuda") for k in (1, 2, 5)]
            ys = dist.group_reduce_scatter(xs, "sum", stream=s)
            for k, y in zip((1, 2, 5), ys):
                assert y.shape == (k, 3) and torch.all(y == n * (n + 1) / 2)
            ys = dist.group_reduce_scatter(xs, "avg", stream=s)
            for y in ys:
                assert torch.allclose(y.float(), torch.full(y.shape, (n + 1) / 2, device="cuda"))
            shards = [torch.full((k, 3), float(r + 1), dtype=dtype, device="cuda") for k in (1, 2, 5)]
            outs = [torch.zeros((n * k, 3), dtype=dtype, device="cuda") for k in (1, 2, 5)]
            dist.group_allgather(shards, 0, outs, stream=s)
            for k, o in zip((1, 2, 5), outs):
                assert torch.equal(o[:, 0].float().cpu(), torch.arange(1, n + 1).repeat_interleave(k).float())
        # rank_list: every group reduces / gathers among its own ranks; a rank that no group
        # names works alone (test_collective_communication.py:124-227, communicator.cc:21-84)
        groups = [[0], list(range(1, n))] if n > 2 else [[0], [1]]
        mine = groups[0] if r == 0 else groups[1]
        x = torch.full((4, 4), float(r + 1), device="cuda")
        dist.allreduce(x, "sum", rank_list=groups, stream=s)
        assert torch.all(x == float(sum(q + 1 for q in mine))), x
        y = dist.allgather(torch.full((2, 3), float(r + 1), device="cuda"), 0, rank_list=groups, stream=s)
        assert torch.equal(y[:, 0].cpu(), torch.tensor([q + 1.0 for q in mine]).repeat_interleave(2))
        x = torch.full((len(mine) * 2, 2), float(r + 1), device="cuda")
        y = dist.reduce_scatter(x, "sum", rank_list=groups, stream=s)
        assert y.shape == (2, 2) and torch.all(y == float(sum(q + 1 for q in mine)))
        x = torch.full((3,), float(r + 1), device="cuda")
        dist.allreduce(x, "sum", rank_list=[[0]], stream=s)  # ranks other than 0 are named nowhere
        assert torch.all(x == float(r + 1))
        x = torch.full((3,), float(r + 1), device="cuda")
        dist.allreduce(x, "sum", rank_list=groups, stream=s)  # the same list again: the cached group
        assert torch.all(x == float(sum(q + 1 for q in mine)))
        whole = [list(range(n))]  # one group of every rank: a communicator split off the global one
        x = torch.full((3,), float(r + 1), device="cuda")
        dist.allreduce(x, "sum", rank_list=whole, stream=s)
        assert torch.all(x == n * (n + 1) / 2)
        y = dist.allgather(torch.full((1, 2), float(r + 1), device="cuda"), 0, rank_list=whole, stream=s)
        assert torch.equal(y[:, 0].cpu(), torch.arange(1, n + 1).float())
        # the integer and double types of the reference's NCCL type map
        for dtype in (torch.int64, torch.uint8, torch.int8, torch.float64):
            x = torch.full((5,), r + 1, dtype=dtype, device="cuda")
            dist.allreduce(x, "sum", stream=s)
            assert torch.all(x == n * (n + 1) // 2), (dtype, x)
            y = dist.allgather(torch.full((2,), r + 1, dtype=dtype, device="cuda"), 0, stream=s)
            assert torch.equal(y.cpu().double(), torch.arange(1, n + 1).repeat_interleave(2).double())
        try:
            dist.reduce_scatter(torch.zeros(n + 1, 2, device="cuda"), "sum", stream=s)
            raise AssertionError("reduce_scatter accepted a dim 0 that does not divide")
        except ValueError:
            pass
    s.synchronize()
    comm.check()


# collectives by NCCL / own kernels with / without multicast / own kernels on gradients and
# parameters that live inside the symmetric buffer (no pack and unpack copies) - these three on
# memory from rafb200_symm_alloc - / own kernels with multicast on memory from
# torch.distributed._symmetric_memory / LANS with the collectives inside the update kernel:
# reduce-scatter only, both with multicast, both with peer loads and stores, reduction through
# the switch with peer stores
MODES = ["nccl", "multimem", "peer", "view", "torch", "fusedrs", "fusedm", "fusedp", "fusedx"]
FUSED = {"fusedrs": 1, "fusedm": 2, "fusedp": 2, "fusedx": 3}  # the collectives inside the update kernel
# ... and each of them again with all steps queued back to back: no host synchronisation and no
# status read between steps, so the values also cover the ordering ACROSS steps (the fence at the
# start of a step, barrier epochs, the all-gather of step s overlapping the reduce-scatter of
# step s + 1, gradients rewritten inside the symmetric buffer)
MODES = MODES + [m + "_q" for m in MODES]


def run_zero(comm, out_dir, tag):
    n, r = comm.size, comm.rank
    queued = tag.endswith("_q")
    mode = tag[:-2] if queued else tag
    for case, (optimizer, g_dtype, p_dtype) in enumerate(CASES):
        plan = Plan(SHAPES, n, r, BUCKET)
        z = ZeroStep(plan, comm, g_dtype, p_dtype, optimizer)
        gviews = pviews = None
        if mode != "nccl":
            z.attach_symmetric(multicast=(mode not in ("peer", "fusedp")),
                               allocator="torch" if mode == "torch" else "library")
            if mode not in ("peer", "fusedp"):
                assert z.multicast, "no multicast address available"
            if mode in FUSED:
                z.set_fused(FUSED[mode])
            if mode == "view" or mode in FUSED:
                gviews, pviews = z.arena_views()
                assert any(x is not None for x in gviews) and any(x is None for x in gviews)
        rng = np.random.default_rng(0)
        full_p = [(rng.standard_normal(numel(s)) * 0.02).astype(np.float32) for s in SHAPES]
        tp, tm, tv = [], [], []
        for i, s in enumerate(SHAPES):
            se = int(plan.shard_elems[i])
            padded = np.zeros(se * n, np.float32)
            padded[:numel(s)] = full_p[i]
            tp.append(torch.from_numpy(padded[r * se:(r + 1) * se].copy()).cuda())
            tm.append(torch.zeros(se, device="cuda"))
            tv.append(torch.zeros(se, device="cuda"))
        params = [torch.zeros(numel(s), dtype=TORCH[p_dtype], device="cuda") for s in SHAPES]
        if pviews is not None:
            params = [pv.reshape(-1) if pv is not None else own for pv, own in zip(pviews, params)]
        scale = 2.0 ** -15 if g_dtype == "float16" else 1.0
        hyper = make_hyper(optimizer, learning_rate=0.1 if optimizer == "sgd" else 1e-3, mu=0.9,
                           beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.01, grad_scale=scale,
                           average=1)
        saved = {}
        keep = []  # the library's streams read the gradients: they stay allocated until the last status
        for step in range(1, STEPS + 1):
            grads = [local_grad(r, step, i, numel(s), g_dtype, 1 / scale).cuda() for i, s in enumerate(SHAPES)]
            keep.append(list(grads))
            if gviews is not None:  # "backward" writes straight into the symmetric buffer
                for i, gv in enumerate(gviews):
                    if gv is not None:
                        gv.reshape(-1).copy_(grads[i])
                        grads[i] = gv.reshape(-1)
            z.bind(grads, params, tp, tm, tv)
            z.step(hyper, step)
            if queued:
                continue
            z.status()
            if step == 1:  # the caller's gradients are inputs only: the step must not modify them
                for i, s in enumerate(SHAPES):
                    again = local_grad(r, step, i, numel(s), g_dtype, 1 / scale)
                    assert torch.equal(grads[i].cpu(), again), ("gradient modified", i)
        z.status()
        for i in range(len(SHAPES)):
            saved[f"p_{i}"] = tp[i].cpu().numpy()
            saved[f"m_{i}"] = tm[i].cpu().numpy()
            saved[f"v_{i}"] = tv[i].cpu().numpy()
            saved[f"param_{i}"] = params[i].float().cpu().numpy()
        kernels, collectives = z.launch_counts()
        if mode == "view" or mode in FUSED:
            assert kernels <= 7 * plan.num_buckets
        saved["counts"] = np.array([kernels, collectives, plan.num_buckets])
        np.savez(os.path.join(out_dir, f"case{case}_{tag}_rank{r}.npz"), **saved)
        z.close()
        plan.close()


def check_plain_data_parallel(comm):
    """zero_opt_level 0 on several ranks: gradients averaged by _allreduce, unsharded update
    (python/raf/optim/sgd.py:118-150 with the data-parallel pass instead of the ZeRO one)."""
    from raf_b200 import optim

    n, r = comm.size, comm.rank
    cfg = dist.get_config()
    before = cfg.dumps()
    cfg.zero_opt_level = 0
    cfg.enable_data_parallel = True
    try:
        rng = np.random.default_rng(5)
        x0 = {f"w{i}": torch.from_numpy((rng.standard_normal(s) * 0.02).astype(np.float32)).cuda()
              for i, s in enumerate([(33, 7), (5,), (1024,)])}
        want = {k: v.clone() for k, v in x0.items()}
        opt = optim.with_sgd(learning_rate=0.1, momentum=0.01)(x0)
        grads = [local_grad(r, 1, i, v.numel(), "float32", 1.0).cuda().reshape(v.shape) for i, v in enumerate(x0.values())]
        opt.step(grads)
        torch.cuda.synchronize()
        for i, (k, v) in enumerate(want.items()):
            total = sum(local_grad(q, 1, i, v.numel(), "float32", 1.0) for q in range(n)).reshape(v.shape) / n
            assert torch.allclose(grads[i].cpu(), total, rtol=0, atol=0), "gradients are averaged in place"
            exp = v.cpu() - 0.1 * total  # v1 = 0.01 * 0 + g ; x1 = x0 - lr * v1
            assert torch.allclose(x0[k].cpu(), exp, rtol=1e-7, atol=1e-9), (k, (x0[k].cpu() - exp).abs().max())
        opt.close()
    finally:
        cfg.loads(before)


def check_wait_expiry(comm):
    """A rank that never joins a step: the others' cross-GPU barrier gives up after its (short)
    limit, the step reports RAFB200_DEVICE_WAIT_EXPIRED instead of hanging, the next step is
    refused on the host, and the context stays usable.  Plain peer loads, no multicast."""
    import time

    from raf_b200._lib import RafB200Error

    n, r = comm.size, comm.rank
    plan = Plan(SHAPES, n, r, BUCKET)
    z = ZeroStep(plan, comm, "float32", "float32", "sgd")
    z.attach_symmetric(multicast=False)
    z.set_wait_limit(200)
    ses = [int(x) for x in plan.shard_elems]
    grads = [torch.zeros(numel(s), device="cuda") for s in SHAPES]
    params = [torch.zeros(numel(s), device="cuda") for s in SHAPES]
    tp = [torch.zeros(se, device="cuda") for se in ses]
    tm = [torch.zeros(se, device="cuda") for se in ses]
    z.bind(grads, params, tp, tm, None)
    hyper = make_hyper("sgd", learning_rate=0.1, mu=0.9, weight_decay=0.0, grad_scale=1.0, average=1)
    dist.allreduce(torch.zeros(1, device="cuda"))
    torch.cuda.synchronize()
    if r != n - 1:
        z.step(hyper, 1)
        try:
            z.status()
            raise AssertionError("the step completed although one rank never joined it")
        except RafB200Error as e:
            assert e.status == 5, e  # RAFB200_DEVICE_WAIT_EXPIRED
        try:
            z.step(hyper, 2)
            raise AssertionError("a step was queued after a wait had expired")
        except RafB200Error as e:
            assert e.status == 5, e
        # the context is intact: ordinary work still runs
        assert float((torch.ones(1000, device="cuda") * 2).sum()) == 2000.0
    else:
        time.sleep(1.0)  # takes no part in the step; leaves only when the others are done waiting
    dist.allreduce(torch.zeros(1, device="cuda"))
    torch.cuda.synchronize()
    z.close()
    plan.close()


def main():
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    import torch.distributed as td

    comm = dist.init_from_env(timeout_ms=120000)
    check_collectives(comm)
    check_plain_data_parallel(comm)
    # torch.distributed only carries the symmetric-memory rendezvous of the two non-NCCL modes
    td.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    for mode in MODES:
        run_zero(comm, os.environ["OUT_DIR"], mode)
    torch.cuda.synchronize()
    td.barrier()
    torch.cuda.synchronize()
    check_wait_expiry(comm)
    comm.close()
    td.destroy_process_group()
    print(f"rank {comm.rank}: ok", flush=True)


if __name__ == "__main__":
    main()
