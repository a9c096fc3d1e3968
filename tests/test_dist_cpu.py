"""World-size-2 tests of the host side of the multi-rank path, on CPU (gloo, no GPU).

What they cover: (1) the file-store rendezvous of the C library between two real
processes, including the failure case of a root that never arrives (bounded, reported
as RAFB200_TIMEOUT); (2) that the shard geometry each rank derives from its own Plan
tiles the padded tensors without gaps or overlap, using gloo's all_gather / reduce_scatter
as an independent implementation of the exchange; (3) that shard-wise oracle updates on
gloo-reduced gradients reproduce the unsharded oracle bit for bit for the element-wise
optimizers (the property the GPU path relies on when it shards).
"""
import ctypes as C
import os
import sys
import tempfile
import time

import numpy as np
import torch
import torch.distributed as td
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHAPES = [(30, 16), (16,), (7, 3, 3), (1,), (129, 65), (50, 64)]


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    td.init_process_group("gloo", rank=rank, world_size=world)


def _free_port():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_store(rank, world, port, store, result):
    sys.path.insert(0, ROOT)
    from raf_b200 import _lib

    _init(rank, world, port)
    lib = _lib.load()
    payload = bytes(range(128))
    buf = (C.c_uint8 * 128)(*(payload if rank == 0 else bytes(128)))
    if rank != 0:
        time.sleep(0.3)  # the root publishes first or later: both orders must work
    rc = lib.rafb200_store_exchange(rank, store.encode(), 7, buf, 128, 20000)
    assert rc == 0, lib.rafb200_last_error()
    assert bytes(buf) == payload
    td.barrier()
    # a key nobody publishes: the non-root rank gives up after the deadline and says so
    if rank == 1:
        t0 = time.time()
        rc = lib.rafb200_store_exchange(1, store.encode(), 8, buf, 128, 300)
        assert rc == 4, rc  # RAFB200_TIMEOUT
        assert 0.25 < time.time() - t0 < 5.0
        assert b"after 300 ms" in lib.rafb200_last_error()
    td.barrier()
    result[rank] = 1
    td.destroy_process_group()


def _worker_shards(rank, world, port, result):
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    from raf_b200.zero import Plan, numel

    _init(rank, world, port)
    plan = Plan(SHAPES, world, rank, 2000)
    rng = np.random.default_rng(0)
    full_p = [(rng.standard_normal(numel(s)) * 0.02).astype(np.float32) for s in SHAPES]
    # unsharded oracle on the mean gradient (what one process would compute)
    ref_p = [x.copy() for x in full_p]
    ref_v = [np.zeros_like(x) for x in full_p]
    my_p, my_v = [], []
    for i, s in enumerate(SHAPES):
        se = int(plan.shard_elems[i])
        assert int(plan.padded_elems[i]) == se * world and se * world >= numel(s)
        padded = np.zeros(se * world, np.float32)
        padded[:numel(s)] = full_p[i]
        my_p.append(padded[rank * se:(rank + 1) * se].copy())
        my_v.append(np.zeros(se, np.float32))
    for step in range(1, 4):
        for i, s in enumerate(SHAPES):
            se = int(plan.shard_elems[i])
            local = [np.random.default_rng(1000 * q + 10 * step + i).integers(-15, 16, numel(s)).astype(np.float32)
                     * np.float32(2.0 ** -10) for q in range(world)]
            # exchange through gloo: pad, reduce-scatter (sum), later all-gather
            padded = torch.zeros(se * world)
            padded[:numel(s)] = torch.from_numpy(local[rank])
            shard = torch.zeros(se)
            td.reduce_scatter(shard, list(padded.split(se)), op=td.ReduceOp.SUM)
            O.sgd(my_p[i], shard.numpy().copy(), my_v[i], 0.1, 0.9, 1e-4, 1.0 / world)
            O.sgd(ref_p[i], sum(local).astype(np.float32), ref_v[i], 0.1, 0.9, 1e-4, 1.0 / world)
    for i, s in enumerate(SHAPES):
        se = int(plan.shard_elems[i])
        gathered = [torch.zeros(se) for _ in range(world)]
        td.all_gather(gathered, torch.from_numpy(my_p[i]))
        full = torch.cat(gathered).numpy()
        assert full[:numel(s)].tobytes() == ref_p[i].tobytes(), (rank, i)
        assert not full[numel(s):].any()  # padding rows stay zero
    result[rank] = 1
    td.destroy_process_group()


def _run(fn, *args):
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=fn, args=(r, 2, port) + args + (result,)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        if p.is_alive():
            p.terminate()  # exactly the child started above
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(result) == {0: 1, 1: 1}


def test_file_store_rendezvous_two_processes_and_timeout():
    with tempfile.TemporaryDirectory() as tmp:
        _run(_worker_store, os.path.join(tmp, "store"))


def test_sharded_update_equals_unsharded_two_processes():
    _run(_worker_shards)
