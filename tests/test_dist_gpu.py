"""Multi-GPU tests: NCCL collectives and the ZeRO step on 2 (and 4) GPUs, one process per
GPU, against the reference's known answers and the CPU oracle.  Skipped on a box with one GPU.

The children (tests/dist_worker.py) exchange the NCCL id through the file store, check the
collectives themselves, and write what each rank ended with; this process then replays the
same three steps per rank shard on the oracle.  Rank-local gradients are small integers
times a power of two, so their sum over ranks is exact in every dtype and in any order:
the reduced gradient is known exactly and SGD / Adam must match the oracle bit for bit at
any world size; LANS within 1e-5.  Each case runs four times: collectives by NCCL, by the
library's own kernels over symmetric memory with the NVSwitch multicast address
(multimem.ld_reduce / multimem.st), by the same kernels over plain peer pointers, and with the
gradients and parameters living inside the symmetric buffer (no pack / unpack copies).
"""
import itertools
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import CODES, bits_equal, rel_err

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spawn(world, out_dir, store):
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                   RAF_FILE_STORE_PATH=store, OUT_DIR=out_dir, NCCL_NVLS_ENABLE="0",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "dist_worker.py")],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                      text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()  # exactly the child this test started
            out, _ = p.communicate()
            out += "\n[timeout]"
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-4000:]}"


@pytest.mark.parametrize("world", [2, 4])
def test_collectives_and_zero_step_multi_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import dist_worker as W
    from raf_b200.zero import numel

    with tempfile.TemporaryDirectory() as tmp:
        store = os.path.join(tmp, "store")
        os.makedirs(store)
        _spawn(world, tmp, store)
        for mode, (case, (optimizer, g_dtype, p_dtype)) in itertools.product(W.MODES, enumerate(W.CASES)):
            ranks = [np.load(os.path.join(tmp, f"case{case}_{mode}_rank{r}.npz")) for r in range(world)]
            scale = 2.0 ** -15 if g_dtype == "float16" else 1.0
            gscale = scale / world  # the mean over ranks folded into the gradient scale
            rng = np.random.default_rng(0)
            full_p = [(rng.standard_normal(numel(s)) * 0.02).astype(np.float32) for s in W.SHAPES]
            for r in range(world):
                p, m, v = [], [], []
                rows = [O.shard_rows(s[0], world) for s in W.SHAPES]
                ses = [rows[i] * (numel(s) // s[0]) for i, s in enumerate(W.SHAPES)]
                for i, s in enumerate(W.SHAPES):
                    padded = np.zeros(ses[i] * world, np.float32)
                    padded[:numel(s)] = full_p[i]
                    p.append(padded[r * ses[i]:(r + 1) * ses[i]].copy())
                    m.append(np.zeros(ses[i], np.float32))
                    v.append(np.zeros(ses[i], np.float32))
                outs = None
                for step in range(1, W.STEPS + 1):
                    g = []
                    for i, s in enumerate(W.SHAPES):
                        total = np.zeros(ses[i] * world, np.float32)
                        for q in range(world):
                            total[:numel(s)] += W.local_grad(q, step, i, numel(s), "float32", 1 / scale).numpy()
                        shard = total[r * ses[i]:(r + 1) * ses[i]].copy()
                        g.append(O.cast(shard, CODES[g_dtype]) if g_dtype != "float32" else shard)
                    if optimizer == "sgd":
                        outs = [O.sgd(p[i], g[i], m[i], 0.1, 0.9, 0.01, gscale, out_code=CODES[p_dtype])
                                for i in range(len(p))]
                    elif optimizer == "adam":
                        outs = [O.adam(g[i], p[i], m[i], v[i], step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1,
                                       gscale, out_code=CODES[p_dtype]) for i in range(len(p))]
                    else:
                        outs, _ = O.lans(g, p, m, v, step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, 1, gscale,
                                         out_code=CODES[p_dtype])
                for i, s in enumerate(W.SHAPES):
                    got_p, got_m, got_v = ranks[r][f"p_{i}"], ranks[r][f"m_{i}"], ranks[r][f"v_{i}"]
                    if optimizer == "lans":
                        assert rel_err(got_p, p[i]) < 1e-5 and rel_err(got_m, m[i]) < 1e-5
                        assert rel_err(got_v, v[i]) < 1e-5
                    else:
                        assert bits_equal(got_p, p[i]) and bits_equal(got_m, m[i]), (mode, case, r, i)
                        if optimizer == "adam":
                            assert bits_equal(got_v, v[i])
                    # every rank's gathered parameter holds this rank's block (padding rows dropped)
                    lo, hi = r * ses[i], min((r + 1) * ses[i], numel(s))
                    if hi > lo:
                        if p_dtype == "float32":
                            want = np.asarray(outs[i], np.float32)[:hi - lo]
                        elif p_dtype == "float16":
                            want = np.asarray(outs[i]).astype(np.float32)[:hi - lo]
                        else:
                            want = (np.asarray(outs[i]).astype(np.uint32) << 16).view(np.float32)[:hi - lo]
                        for q in range(world):
                            got = ranks[q][f"param_{i}"][lo:hi]
                            if optimizer == "lans":
                                assert rel_err(got, want) < (1e-5 if p_dtype == "float32" else 2e-3)
                            else:
                                assert bits_equal(got, want), (mode, case, r, q, i)
                kernels, collectives, nb = ranks[r]["counts"]
                mode = mode.split("_")[0]  # the "_q" runs queue their steps back to back
                # per bucket: pack, update, unpack kernels and ONE reduce-scatter + ONE all-gather,
                # which are NCCL calls or two more kernels of the library plus two barrier kernels
                if mode == "nccl":
                    assert kernels == 3 * nb and collectives == 2 * nb
                else:
                    assert collectives == 0 and (kernels == 7 * nb or mode == "view" or mode.startswith("fused"))
