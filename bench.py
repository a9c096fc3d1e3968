#!/usr/bin/env python
"""Benchmark of the ZeRO optimizer step (reduce-scatter -> shard update -> all-gather).

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

N > 1 is launched by torch.distributed.run (one rank per GPU).  Rank 0 prints ONE
JSON line.  A step is one pass of the hot path over one batch of synthetic
gradients:
  value  whole-job parameter-elements/s with the gradients already resident in HBM
         (K steps timed as one region with CUDA events, max over ranks);
  e2e    the same metric through the host-buffer entry point: gradients copied in
         from pinned host memory and the updated model-dtype parameters copied back
         inside the timed region; `frac_of_pcie` compares it with a plain pinned copy
         of the same bytes in both directions;
  roofline  algorithmic bytes of the update kernel / its duration, against the
         measured HBM copy bandwidth;
  step_roofline  (N > 1) the slower of update bytes at the measured HBM peak and
         collective bytes per direction at 900 GB/s, over the measured step time;
  verified  one more step after the timed region, checked against the CPU oracle on
         the largest tensor, a mid-sized one and the small tail of the list (every
         rank checks its own row blocks from the reduced gradients; the gathered
         parameters must equal the cast of every rank's master block);
  cpu_baseline  (N = 1) the CPU oracle (a restatement of the reference's math,
         OpenMP, all host threads) timed on the same tensors;
  existing_kernel  (LANS) the reference's own multi_tensor_lans_cuda, compiled
         unchanged for sm_100a, on the same shards.
Workloads (BASELINE.json configs): bert_lans (default, config 3), rn50_sgd (2),
gpt2_adam (4), flat_adam:<Mi elements> (5), flat_sgd (1).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from typing import List, Tuple

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 << 20
NVLINK_NOMINAL_GBS = 900.0   # per direction per GPU: the figure the step roofline is defined on
NVLINK_PEER_COPY_GBS = 770.0  # a peer copy measured on B200 / NVSwitch: reported beside it, labelled


# --------------------------------------------------------------------------- shapes
def resnet50_shapes() -> List[Tuple[int, ...]]:
    """161 parameter tensors, 25,557,032 elements: conv weights O x I x k x k, a
    (gamma, beta) pair after every conv, fc 1000 x 2048 + bias."""
    shapes: List[Tuple[int, ...]] = []

    def conv_bn(o, i, k):
        shapes.append((o, i, k, k))
        shapes.append((o,))
        shapes.append((o,))

    conv_bn(64, 3, 7)
    inplanes = 64
    for planes, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
        for b in range(blocks):
            conv_bn(planes, inplanes, 1)
            conv_bn(planes, planes, 3)
            conv_bn(planes * 4, planes, 1)
            if b == 0:
                conv_bn(planes * 4, inplanes, 1)  # downsample
            inplanes = planes * 4
    shapes.append((1000, 2048))
    shapes.append((1000,))
    return shapes


def bert_large_shapes() -> List[Tuple[int, ...]]:
    """391 tensors, 335,141,888 elements (24 layers, hidden 1024, FFN 4096, vocab 30522)."""
    h, ffn = 1024, 4096
    shapes: List[Tuple[int, ...]] = [(30522, h), (512, h), (2, h), (h,), (h,)]
    for _ in range(24):
        for _ in range(4):
            shapes += [(h, h), (h,)]
        shapes += [(h,), (h,)]
        shapes += [(ffn, h), (ffn,), (h, ffn), (h,)]
        shapes += [(h,), (h,)]
    shapes += [(h, h), (h,)]
    return shapes


def gpt2_medium_shapes() -> List[Tuple[int, ...]]:
    """292 tensors, 354,823,168 elements (24 layers, d_model 1024, vocab 50257, ctx 1024)."""
    d = 1024
    shapes: List[Tuple[int, ...]] = [(50257, d), (1024, d)]
    for _ in range(24):
        shapes += [(d,), (d,)]
        shapes += [(d, 3 * d), (3 * d,), (d, d), (d,)]
        shapes += [(d,), (d,)]
        shapes += [(d, 4 * d), (4 * d,), (4 * d, d), (d,)]
    shapes += [(d,), (d,)]
    return shapes


def numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


# --------------------------------------------------------------------------- workloads
def workload(name: str):
    """-> dict(shapes, optimizer, g_dtype, p_dtype, hyper kwargs, bucket_elems, bytes_per_elem, label)"""
    if name == "bert_lans":
        return dict(shapes=bert_large_shapes(), optimizer="lans", g_dtype="float16", p_dtype="float16",
                    hyper=dict(learning_rate=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.01,
                               bias_correction=1, grad_averaging=1, mode=1, normalize_grad=1,
                               grad_scale=2.0 ** -15),
                    # 80 Mi elements (160 MiB of fp16 gradients) per bucket: 5 buckets; measured
                    # 2.07 ms at 8 GPUs against 2.11 (9 buckets) and 2.37 (26 buckets of 25 MiB)
                    loss_scale=2.0 ** 15, bucket_elems=83886080, bytes_per_elem=28,
                    label="config 3: ZeRO-1 LANS, BERT-large shapes (391 tensors, 335,141,888 elements), "
                          "fp32 master/m/v, fp16 gradients (loss scale 2^15), fp16 parameter all-gather")
    if name == "rn50_sgd":
        return dict(shapes=resnet50_shapes(), optimizer="sgd", g_dtype="float32", p_dtype="float32",
                    hyper=dict(learning_rate=0.1, mu=0.9, weight_decay=1e-4), loss_scale=1.0,
                    bucket_elems=6553600, bytes_per_elem=20,
                    label="config 2: ZeRO-1 SGD-momentum, ResNet-50 shapes (161 fp32 tensors, 25,557,032 elements)")
    if name == "gpt2_adam":
        return dict(shapes=gpt2_medium_shapes(), optimizer="adam", g_dtype="bfloat16", p_dtype="bfloat16",
                    hyper=dict(learning_rate=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                               bias_correction=1, mode=1), loss_scale=1.0, bucket_elems=83886080,
                    bytes_per_elem=28,
                    label="config 4: ZeRO-2 Adam, GPT-2-medium shapes (292 tensors, 354,823,168 elements), bf16")
    if name.startswith("flat_adam"):
        mi = int(name.split(":")[1]) if ":" in name else 64
        return dict(shapes=[(mi << 20,)], optimizer="adam", g_dtype="float32", p_dtype="float32",
                    hyper=dict(learning_rate=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                               bias_correction=1, mode=1), loss_scale=1.0, bucket_elems=1 << 62,
                    bytes_per_elem=28, label=f"config 5: one flat fp32 tensor of {mi} Mi elements, Adam")
    if name == "flat_sgd":
        return dict(shapes=[(25557032,)], optimizer="sgd", g_dtype="float32", p_dtype="float32",
                    hyper=dict(learning_rate=0.1, mu=0.9, weight_decay=1e-4), loss_scale=1.0,
                    bucket_elems=1 << 62, bytes_per_elem=20,
                    label="config 1: one flat fp32 tensor of 25,557,032 elements, SGD-momentum")
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, an earlier copy measurement on B200)"


def profiled_traffic(workload_name: str, n_gpus: int, shard_of: int):
    """DRAM bytes (read + write) of one launch of the dominant kernel, from the table of ncu
    captures in profiles/dram_traffic_per_launch.md; None when that case was not captured."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.md")
    try:
        with open(path) as f:
            rows = f.read().splitlines()
    except OSError:
        return None
    for row in rows:
        cells = [c.strip() for c in row.strip().strip("|").split("|")]
        if len(cells) < 5 or cells[0] != workload_name:
            continue
        try:
            if int(cells[1]) == n_gpus and int(cells[2]) == shard_of:
                return int(re.sub(r"[^0-9]", "", cells[4]))
        except ValueError:
            continue
    return None


def rel_err(a, b) -> float:
    """max |a-b| / (|b| + rms(b)): a relative error scaled so that the few elements next to
    zero do not dominate; at most 2x looser than the plain relative error of an element of
    rms size, looser than it for smaller elements."""
    import numpy as np

    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    if a.size == 0:
        return 0.0
    rms = float(np.sqrt(np.mean(b * b)))
    return float(np.max(np.abs(a - b) / (np.abs(b) + (rms if rms > 0 else 1e-30))))


# --------------------------------------------------------------------------- CPU baseline
class CpuArm:
    """The oracle (C/OpenMP restatement of the reference math) on the host cores: one rank's
    full-size, unsharded update of the workload's tensors, no collectives, on every host
    thread this process may use.  Inputs are generated once (untimed); every `step()` is one
    optimizer step over them."""

    def __init__(self, wl):
        import numpy as np

        from oracle import oracle as O

        self.O, self.wl = O, wl
        self.cores = O.use_all_host_threads()
        code = {"float32": O.F32, "float16": O.F16, "bfloat16": O.BF16}
        self.out_code = code[wl["p_dtype"]]
        rng = np.random.default_rng(0)
        self.p, self.m, self.v, self.g = [], [], [], []
        self.elems = 0
        for s in wl["shapes"]:
            n = numel(s)
            if n == 0:
                continue
            self.p.append(rng.standard_normal(n, dtype=np.float32) * np.float32(0.02))
            self.m.append(np.zeros(n, np.float32))
            self.v.append(np.zeros(n, np.float32))
            g32 = rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3 * wl["loss_scale"])
            self.g.append(O.cast(g32, code[wl["g_dtype"]]) if wl["g_dtype"] != "float32" else g32)
            self.elems += n
        self.tensors = len(self.p)
        self.step_no = 0

    def step(self) -> float:
        """One optimizer step; returns its wall time in seconds."""
        O, wl, hy = self.O, self.wl, self.wl["hyper"]
        self.step_no += 1
        scale = 1.0 / wl["loss_scale"]
        t0 = time.perf_counter()
        if wl["optimizer"] == "sgd":
            for p, g, m in zip(self.p, self.g, self.m):
                O.sgd(p, g, m, hy["learning_rate"], hy["mu"], hy["weight_decay"], scale, out_code=self.out_code)
        elif wl["optimizer"] == "adam":
            for p, g, m, v in zip(self.p, self.g, self.m, self.v):
                O.adam(g, p, m, v, self.step_no, hy["learning_rate"], hy["beta1"], hy["beta2"], hy["eps"], 1,
                       hy["weight_decay"], hy["mode"], scale, out_code=self.out_code)
        else:
            O.lans(self.g, self.p, self.m, self.v, self.step_no, hy["learning_rate"], hy["beta1"], hy["beta2"],
                   hy["eps"], 1, hy["weight_decay"], 1, 1, 1, scale, norm_mode=0, out_code=self.out_code)
        return time.perf_counter() - t0

    def describe(self, steps, spent):
        return (f"all {self.tensors} tensors ({self.elems} elements), {steps} optimizer steps, "
                f"{spent:.2f} s of host time on {self.cores} threads; C/OpenMP restatement of the reference "
                f"math (RAF's TVM CPU path cannot be built without its TVM submodule; LANS and Adam have no "
                f"CPU path in RAF)")


def cpu_baseline(wl, budget_s=10.0):
    """Steps of the CPU arm until about `budget_s` seconds of CPU work have been spent."""
    arm = CpuArm(wl)
    arm.step()  # page in, warm the thread pool
    spent, steps = 0.0, 0
    while spent < budget_s and steps < 200:
        spent += arm.step()
        steps += 1
    return {"value": arm.elems * steps / spent, "unit": "param-elements/s", "cores": arm.cores,
            "kind": "port", "sample": arm.describe(steps, spent)}


def run_reference_arm(args, wl):
    """--impl reference: the CPU restatement of the reference's path on all host threads, over
    every tensor of the workload, `--warmup` + `--steps` optimizer steps.  Rank 0 alone runs."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm(wl)
    for _ in range(args.warmup):
        arm.step()
    times = [arm.step() for _ in range(args.steps)]
    spent = sum(times)
    val = arm.elems * len(times) / spent
    cpu = {"value": val, "unit": "param-elements/s", "cores": arm.cores, "kind": "port",
           "sample": arm.describe(len(times), spent)}
    line = {
        "impl": "reference", "metric": "ZeRO optimizer-step param-elements/s", "value": val,
        "unit": "param-elements/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * spent / len(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["label"]},
        "cpu_baseline": cpu,
        "e2e": {"value": val, "unit": "param-elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- verification
def _np(t):
    """torch tensor -> numpy (bf16 as uint16 bit patterns, which is what the oracle takes)."""
    import numpy as np
    import torch

    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def _as_f32(a):
    import numpy as np

    if a.dtype == np.uint16:
        return (a.astype(np.uint32) << 16).view(np.float32)
    return a.astype(np.float32)


def pick_tensors(sizes):
    """Indices to verify: the largest tensor, one of the next-largest distinct size, the
    smallest non-empty one and the last few of the list."""
    order = sorted((i for i, n in enumerate(sizes) if n > 0), key=lambda i: -sizes[i])
    if not order:
        return []
    chosen = [order[0]]
    for i in order:
        if sizes[i] < sizes[order[0]]:
            chosen.append(i)
            break
    chosen.append(order[-1])
    chosen += [i for i in range(max(0, len(sizes) - 4), len(sizes)) if sizes[i] > 0]
    out = []
    for i in chosen:
        if i not in out:
            out.append(i)
    return out


def verify_step(z, wl, plan, step_no, hyper, streams, grads, params, p, m, v, td, world, rank, dev):
    """One more step, checked against the CPU oracle.  Returns the `verified` object (on every
    rank; identical where it matters because the flags are reduced over ranks)."""
    import numpy as np
    import torch

    from oracle import oracle as O

    code = {"float32": O.F32, "float16": O.F16, "bfloat16": O.BF16}
    hy, opt = wl["hyper"], wl["optimizer"]
    k = len(wl["shapes"])
    shard = [int(plan.shard_elems[i]) for i in range(k)]
    idx = pick_tensors(shard)
    elementwise = opt != "lans"
    # elementwise optimizers are checked on windows of huge tensors; LANS needs whole tensors
    win = 8 << 20

    def windows(n):
        if not elementwise or n <= 4 * win:
            return [(0, n)]
        mid = (n // 2 + 12345) & ~1
        return [(0, win), (mid, mid + win), (n - win, n)]

    torch.cuda.synchronize()
    before = {i: [(lo, hi, _np(p[i][lo:hi]), _np(m[i][lo:hi]), _np(v[i][lo:hi]) if v is not None else None)
                  for lo, hi in windows(shard[i])] for i in idx}
    z.step(hyper, step_no, *streams)
    torch.cuda.synchronize()
    z.status()
    gscale = hy.get("grad_scale", 1.0) / (world if world > 1 else 1)
    worst, exact, rs_err, ag_ok = 0.0, True, 0.0, True
    for i in idx:
        g_red_t = z.shard_grad(i)
        # -- reduce-scatter: the reduced block against a float64 sum of every rank's gradient
        if world > 1:
            n_full, se = numel(wl["shapes"][i]), shard[i]
            mine = torch.zeros(se * world, dtype=grads[i].dtype, device=dev)
            mine[:n_full] = grads[i].reshape(-1)
            allg = [torch.empty_like(mine) for _ in range(world)]
            td.all_gather(allg, mine)
            ref = sum(_as_f32(_np(x[rank * se:(rank + 1) * se])).astype(np.float64) for x in allg)
            rs_err = max(rs_err, rel_err(_as_f32(_np(g_red_t)), ref))
            del allg, mine
        for lo, hi, p0, m0, v0 in before[i]:
            g = _np(g_red_t[lo:hi])
            if opt == "sgd":
                out = O.sgd(p0, g, m0, hy["learning_rate"], hy["mu"], hy["weight_decay"], gscale,
                            out_code=code[wl["p_dtype"]])
            elif opt == "adam":
                out = O.adam(g, p0, m0, v0, step_no, hy["learning_rate"], hy["beta1"], hy["beta2"], hy["eps"], 1,
                             hy["weight_decay"], hy["mode"], gscale, out_code=code[wl["p_dtype"]])
            else:
                outs, _ = O.lans([g], [p0], [m0], [v0], step_no, hy["learning_rate"], hy["beta1"], hy["beta2"],
                                 hy["eps"], 1, hy["weight_decay"], 1, 1, 1, gscale, norm_mode=0,
                                 out_code=code[wl["p_dtype"]])
                out = outs[0]
            for ours, want in ((p[i], p0), (m[i], m0)) + (((v[i], v0),) if v0 is not None else ()):
                got = _np(ours[lo:hi])
                exact = exact and got.tobytes() == want.tobytes()
                worst = max(worst, rel_err(got, want))
        # -- all-gather: the gathered parameter equals cast(master) of every rank's block
        master = p[i]
        if world > 1:
            blocks = [torch.empty_like(master) for _ in range(world)]
            td.all_gather(blocks, master)
            master = torch.cat(blocks)
        n_full = numel(wl["shapes"][i])
        want = master[:n_full].to(params[i].dtype)
        ag_ok = ag_ok and bool(torch.equal(want.view(torch.uint8), params[i].reshape(-1).view(torch.uint8)))
    tol = 1e-5 if opt == "lans" else 1e-6
    rs_tol = 0.0 if world == 1 else (1e-6 * world if wl["g_dtype"] == "float32" else 2e-2)
    flags = torch.tensor([worst, rs_err, 0.0 if exact else 1.0, 0.0 if ag_ok else 1.0], device=dev,
                         dtype=torch.float64)
    if td is not None:
        td.all_reduce(flags, op=td.ReduceOp.MAX)
    worst, rs_err, inexact, ag_bad = (float(x) for x in flags.tolist())
    return {"ok": bool(worst <= tol and rs_err <= rs_tol and ag_bad == 0.0),
            "tensors": [{"index": i, "shard_elements": shard[i]} for i in idx],
            "step": step_no, "max_rel_err": worst, "tolerance": tol, "bit_exact": inexact == 0.0,
            "reduce_scatter_max_rel_err": rs_err if world > 1 else None,
            "reduce_scatter_tolerance": rs_tol if world > 1 else None,
            "gathered_params_equal_cast_of_master": ag_bad == 0.0,
            "how": "state of the chosen tensors saved, one more step, CPU oracle replayed on every rank's own "
                   "row blocks from the reduced gradients the update read; error = max |a-b| / (|b| + rms(b)) "
                   "over p, m, v; max over ranks"}


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="bert_lans")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--update-blocks", type=int, default=0)
    ap.add_argument("--bucket-elems", type=int, default=None,
                    help="bucket size in elements (default: the workload's)")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="N = 1 only: run on the shard list that rank 0 of an N-way partition owns "
                         "(a small case of the same kernel, e.g. for profiler captures)")
    ap.add_argument("--collectives", default="auto", choices=["auto", "multimem", "peer", "nccl"],
                    help="N > 1: own kernels over symmetric memory (NVSwitch multicast / peer "
                         "pointers) or NCCL; auto = peer at N = 2, multicast from N = 4, NCCL if symmetric "
                         "memory cannot be set up")
    ap.add_argument("--comm-blocks", type=int, default=0, help="thread blocks per collective kernel")
    ap.add_argument("--fused", type=int, default=-1, choices=[-1, 0, 1, 2, 3],
                    help="LANS at N > 1: collectives inside the update kernel (1 reduce-scatter, 2 all-gather "
                         "too, 0 the bucketed pipeline of separate kernels; -1 = the default for N)")
    ap.add_argument("--no-views", action="store_true",
                    help="symmetric modes: keep gradients and parameters in separate tensors "
                         "(pack / unpack copies) instead of inside the symmetric buffer")
    ap.add_argument("--stages", action="store_true",
                    help="N > 1: also time each stage of the step alone (pack, reduce-scatter, ...)")
    ap.add_argument("--no-existing-kernel", action="store_true",
                    help="do not time the reference's own LANS kernel (oracle/_ref) on the same shards")
    args = ap.parse_args()
    wl = workload(args.workload)
    if args.bucket_elems:
        wl["bucket_elems"] = args.bucket_elems
    if args.impl == "reference":
        run_reference_arm(args, wl)
        return

    import torch

    from raf_b200 import distributed as dist
    from raf_b200.op import torch_dtype
    from raf_b200.zero import Plan, ZeroStep, make_hyper

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as td

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        td.init_process_group("nccl", device_id=dev)
        ids = [dist.unique_id() if rank == 0 else None]
        td.broadcast_object_list(ids, src=0)
        comm = dist.Communicator(world, rank, local_rank, unique_id=ids[0], timeout_ms=120000)
    else:
        td = None
        comm = dist.Communicator(1, 0, local_rank)
    dist.set_communicator(comm)

    shapes = wl["shapes"]
    if args.shard_of > 1:
        if world != 1:
            raise SystemExit("--shard-of needs --gpus 1")
        part = Plan(shapes, args.shard_of, 0, wl["bucket_elems"])
        shapes = [part.shard_shape(i) for i in range(len(shapes))]
        wl["shapes"] = shapes
        wl["label"] += f" -- rank 0's shards of a {args.shard_of}-way partition, no collectives"
        part.close()
    k = len(shapes)
    total = sum(numel(s) for s in shapes)
    plan = Plan(shapes, world, rank, wl["bucket_elems"])
    gdt, pdt = torch_dtype(wl["g_dtype"]), torch_dtype(wl["p_dtype"])
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000 * rank + 1)

    def randn_into(dst, std):
        dst.copy_((torch.randn(dst.numel(), generator=gen, device=dev, dtype=torch.float32) * std).to(dst.dtype))

    def randn(n, std, dtype):
        out = torch.empty(n, dtype=dtype, device=dev)
        randn_into(out, std)
        return out

    def arena(sizes, dtype, pinned=False):
        """One allocation; tensor i is the 16-byte aligned view at the running offset."""
        es = torch.empty((), dtype=dtype).element_size()
        per16 = 16 // es
        offs, at = [], 0
        for n in sizes:
            at = (at + per16 - 1) // per16 * per16
            offs.append(at)
            at += n
        buf = torch.empty(max(at, 1), dtype=dtype, device="cpu" if pinned else dev)
        if pinned:
            buf = buf.pin_memory()
        return buf, [buf[o:o + n] for o, n in zip(offs, sizes)]

    sizes = [numel(s) for s in shapes]
    # fp32 master shards and optimizer state (rank-local), model-dtype full parameters
    p = [randn(int(plan.shard_elems[i]), 0.02, torch.float32) for i in range(k)]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    params_buf, params = arena(sizes, pdt)
    params_buf.zero_()
    if world == 1 and pdt == torch.float32:
        params = p  # one rank, fp32 model: the parameters are the master copy (no second write)
    # Gradient sets: the step leaves the caller's gradients untouched, so a set can be reused;
    # two sets alternate when ranks exchange data.
    nsets = 1 if world == 1 else 2
    if args.fused < 0:
        # LANS: the collectives inside the update kernel (measured 2.12 / 1.69 ms at 2 / 4 GPUs
        # against 2.25 / 2.17 ms for the bucketed pipeline of separate kernels)
        args.fused = 2 if (world > 1 and args.stages is False) else 0
        if args.fused and world == 2 and wl["optimizer"] == "lans":
            # two ranks: the gradients through the switch, the copies as peer stores (1.97 ms
            # against 2.10 ms with both through the switch, which there also carries the rank's
            # own half of every multicast)
            args.fused = 3
    if args.collectives == "auto":
        # separate kernels on two ranks: plain peer loads / stores beat the switch-side
        # reduction (2.25 ms against 2.47 ms); inside the update kernel, and from four ranks on,
        # the multicast forms win
        # (two ranks, SGD / Adam inside the kernel: peer accesses again, 0.20 / 1.82 ms against
        # 0.31 / 1.99 ms through the switch, which at two ranks also carries the rank's own half)
        args.collectives = "peer" if (world == 2 and (args.fused == 0 or wl["optimizer"] != "lans")) else "multimem"
    if world > 1 and not args.update_blocks and wl["optimizer"] == "lans":
        # leave SMs to the collective kernels that run beside the update
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        args.update_blocks = sms - 16
    collectives_used = args.collectives if world > 1 else "none"
    views_used = 0
    gsets, gbufs = [], []
    for _ in range(nsets):
        gb, gs = arena(sizes, gdt)
        for x in gs:
            randn_into(x, 1e-3 * wl["loss_scale"])
        gsets.append(gs)
        gbufs.append(gb)
    zs, zgrads, zparams = [], [], []
    for gs in gsets:
        z = ZeroStep(plan, comm, gdt, pdt, wl["optimizer"])
        if world > 1 and args.collectives != "nccl":
            try:
                z.attach_symmetric(comm_blocks=args.comm_blocks, multicast=(args.collectives == "multimem"))
                if args.collectives == "multimem" and not z.multicast:
                    collectives_used = "peer (no multicast address available)"
                if args.fused > 0:
                    z.set_fused(args.fused)
            except Exception as exc:  # symmetric memory is plumbing: without it NCCL still works
                collectives_used = f"nccl (symmetric memory unavailable: {type(exc).__name__})"
                args.collectives = "nccl"
        zg, zp = gs, params
        if world > 1 and args.collectives != "nccl" and not args.no_views:
            # gradients and model parameters live inside the symmetric buffer where their
            # shard size allows (all tensors of the benchmark shapes): no pack / unpack
            gv, pv = z.arena_views()
            zg = [x.reshape(-1) if x is not None else own for x, own in zip(gv, gs)]
            zp = [x.reshape(-1) if x is not None else own for x, own in zip(pv, params)]
            for dst, src in zip(zg, gs):
                if dst is not src:
                    dst.copy_(src)
            views_used = sum(x is not None for x in gv)
        z.bind(zg, zp, p, m, v if wl["optimizer"] != "sgd" else None)
        if args.update_blocks:
            z.set_update_blocks(args.update_blocks)
        zs.append(z)
        zgrads.append(zg)
        zparams.append(zp)
    hyper = make_hyper(wl["optimizer"], average=1, **wl["hyper"])
    compute = torch.cuda.current_stream()
    comm_stream = dist.comm_stream()

    def barrier():
        torch.cuda.synchronize()
        if td is not None:
            td.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if td is None:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        td.all_reduce(t, op=td.ReduceOp.MAX)
        return float(t.item())

    step_no = 0
    barrier()  # ranks finish their set-up at different times; the step's own waits are bounded
    for w in range(args.warmup):
        step_no += 1
        zs[step_no % nsets].step(hyper, step_no, compute, comm_stream)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(compute)
    for _ in range(args.steps):
        step_no += 1
        zs[step_no % nsets].step(hyper, step_no, compute, comm_stream)
    e1.record(compute)
    barrier()
    for z in zs:
        z.status()  # raises if a bounded cross-GPU wait ran out
    clocks = sampler.stop() if rank == 0 else None
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    kernels, collectives = zs[0].launch_counts()

    # ---- values: one more step against the CPU oracle ----
    verified = None
    if not args.no_verify:
        step_no += 1
        sel = step_no % nsets
        verified = verify_step(zs[sel], wl, plan, step_no, hyper, (compute, comm_stream), zgrads[sel],
                               zparams[sel], p, m, v if wl["optimizer"] != "sgd" else None, td, world, rank, dev)

    # ---- the update kernel alone (this rank's shards, no collectives): roofline ----
    shard_elems = int(plan.total_shard)
    kz = None
    if world == 1:
        kern_ms = ms_step
    else:
        kcomm = dist.Communicator(1, 0, local_rank)
        kplan = Plan([(int(plan.shard_elems[i]),) for i in range(k)], 1, 0, 1 << 62)
        kz = ZeroStep(kplan, kcomm, gdt, pdt, wl["optimizer"])
        gsh = [randn(int(plan.shard_elems[i]), 1e-3 * wl["loss_scale"], gdt) for i in range(k)]
        psh = [torch.zeros(int(plan.shard_elems[i]), dtype=pdt, device=dev) for i in range(k)]
        kz.bind(gsh, psh, p, m, v if wl["optimizer"] != "sgd" else None)
        for _ in range(3):
            step_no += 1
            kz.step(hyper, step_no, compute, comm_stream)
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(compute)
        for _ in range(10):
            step_no += 1
            kz.step(hyper, step_no, compute, comm_stream)
        k1.record(compute)
        torch.cuda.synchronize()
        kern_ms = k0.elapsed_time(k1) / 10
    peak, peak_src = measured_hbm_peak()
    achieved = wl["bytes_per_elem"] * shard_elems / (kern_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": profiled_traffic(args.workload, world, args.shard_of if args.shard_of > 1 else 1),
                "traffic_source": "profiles/dram_traffic_per_launch.md (ncu dram__bytes_read.sum + dram__bytes_write.sum)",
                "peak_source": peak_src,
                "kernel": {"sgd": "update_list_kernel<SgdOp>", "adam": "update_list_kernel<AdamOp>",
                           "lans": "lans_kernel"}[wl["optimizer"]],
                "kernel_ms": kern_ms, "algorithmic_bytes_per_launch": wl["bytes_per_elem"] * shard_elems}

    # ---- step roofline: slower of update bytes at HBM peak and collective bytes at 900 GB/s ----
    gsz, psz = gsets[0][0].element_size(), params[0].element_size()
    coll_bytes = (world - 1) / world * int(plan.total_padded) * (gsz + psz)
    hbm_ms = wl["bytes_per_elem"] * shard_elems / (peak * 1e9) * 1e3
    bound_ms = max(hbm_ms, coll_bytes / (NVLINK_NOMINAL_GBS * 1e9) * 1e3)
    bound_peer_ms = max(hbm_ms, coll_bytes / (NVLINK_PEER_COPY_GBS * 1e9) * 1e3)

    # ---- end to end: host gradients in, host parameters out ----
    e2e = None
    if not args.no_e2e:
        ghost_buf, grads_host = arena(sizes, gdt, pinned=True)
        phost_buf, params_host = arena(sizes, pdt, pinned=True)
        for gh, gd in zip(grads_host, gsets[0]):
            gh.copy_(gd)
        for one in (ghost_buf, phost_buf, gbufs[0], params_buf):
            zs[0].declare_arena(one)
        # n ranks share one host: every rank still needs all of its own local gradients, but
        # each parameter has to reach the host only once - every rank returns the rows it owns
        zs[0].set_host_output(1 if world > 1 else 0)
        zs[0].step_host(hyper, step_no + 1, grads_host, params_host, compute, comm_stream)
        step_no += 1
        barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record(compute)
        for _ in range(args.e2e_steps):
            step_no += 1
            zs[0].step_host(hyper, step_no, grads_host, params_host, compute, comm_stream)
        h1.record(compute)
        barrier()
        e2e_ms = max_over_ranks(h0.elapsed_time(h1)) / args.e2e_steps
        d2h = sum(min(numel(s), (rank + 1) * int(plan.shard_elems[i])) - min(numel(s), rank * int(plan.shard_elems[i]))
                  for i, s in enumerate(shapes)) * psz if world > 1 else total * psz
        # yardstick: the same bytes as two plain pinned copies, one per direction, at the same time
        side = torch.cuda.Stream()
        gdev = gsets[0][0].new_empty(ghost_buf.numel())
        pdev = params[0].new_empty(max(1, d2h // psz))
        y0, y1, y2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        best = None
        for _ in range(3):
            barrier()
            y0.record(compute)
            side.wait_event(y0)
            gdev.copy_(ghost_buf, non_blocking=True)
            with torch.cuda.stream(side):
                phost_buf[:pdev.numel()].copy_(pdev, non_blocking=True)
                y1.record(side)
            compute.wait_event(y1)
            y2.record(compute)
            torch.cuda.synchronize()
            t = max_over_ranks(y0.elapsed_time(y2))
            best = t if best is None else min(best, t)
        e2e = {"value": total / (e2e_ms * 1e-3), "unit": "param-elements/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": total * gsz * world,
               "d2h_bytes_per_step": total * psz,
               "steps": args.e2e_steps, "pcie_copy_ms": best, "frac_of_pcie": best / e2e_ms,
               "host_output": "every rank copies back the rows it owns" if world > 1 else "all parameters",
               "how": "rafb200_zero_step_host: pinned host gradients in, updated parameters back to pinned host "
                      "memory, both inside the timed region; pcie_copy_ms = the same bytes as one plain "
                      "cudaMemcpyAsync per direction, concurrently, best of 3"}
        del gdev, pdev

    stage_ms = None
    if args.stages and world > 1:
        stage_ms = {}
        for name, mask in (("pack", 1), ("reduce_scatter", 2), ("update", 4), ("all_gather", 8),
                           ("unpack", 16), ("collectives", 10), ("kernels", 21)):
            zs[0].set_stage_mask(mask)
            for _ in range(2):
                step_no += 1
                zs[0].step(hyper, step_no, compute, comm_stream)
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(compute)
            for _ in range(5):
                step_no += 1
                zs[0].step(hyper, step_no, compute, comm_stream)
            s1.record(compute)
            barrier()
            stage_ms[name] = max_over_ranks(s0.elapsed_time(s1)) / 5
        zs[0].set_stage_mask(31)

    existing = None
    if not args.no_existing_kernel and wl["optimizer"] == "lans":
        from oracle import ref_lans

        if ref_lans.available():
            numels = [int(plan.shard_elems[i]) for i in range(k)]
            g32 = [randn(n, 1e-3, torch.float32) for n in numels]
            ref = ref_lans.RefLans(numels)
            for _ in range(2):
                ref(g32, p, m, v, 5)
            torch.cuda.synchronize()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record(compute)
            for _ in range(5):
                ref(g32, p, m, v, 5)
            r1.record(compute)
            torch.cuda.synchronize()
            ref_ms = max_over_ranks(r0.elapsed_time(r1) / 5)
            existing = {"kernel": "reference multi_tensor_lans_cuda<float> (src/op/dialect/cuda/kernels/"
                                  "multi_tensor_lans.cu) compiled unchanged for sm_100a",
                        "ms": ref_ms, "ours_ms": max_over_ranks(kern_ms),
                        "note": "same shards; the reference kernel takes fp32 gradients and does no "
                                "cast / unscale / fp16 copy, which this library fuses into its kernel"}
            del g32, ref

    if rank == 0:
        cpu = None if (args.no_cpu_baseline or world > 1) else cpu_baseline(wl)
        line = {
            "metric": "ZeRO optimizer-step param-elements/s", "value": total / (ms_step * 1e-3),
            "unit": "param-elements/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["label"], "optimizer": wl["optimizer"], "n_tensors": k,
                       "elements": total, "shard_elements_per_rank": shard_elems,
                       "bucket_elems": wl["bucket_elems"], "buckets": plan.num_buckets if world > 1 else 1,
                       "gradient_sets": nsets, "collectives": collectives_used,
                       "collectives_inside_update_kernel": (["no", "reduce-scatter", "reduce-scatter and all-gather", "reduce-scatter and all-gather (peer stores)"][args.fused]
                                                            if world > 1 and args.collectives != "nccl" else "no"),
                       "tensors_inside_symmetric_buffer": views_used,
                       "l2": (f"inputs larger than L2 ({wl['bytes_per_elem'] * shard_elems >> 20} MiB touched per step per rank)"
                              if wl['bytes_per_elem'] * shard_elems > L2_BYTES else
                              f"working set of {wl['bytes_per_elem'] * shard_elems >> 20} MiB fits the 126 MB L2 and is not "
                              "flushed between steps: not a DRAM-bound measurement")},
            "roofline": roofline,
            "step_roofline": {"bound_ms": bound_ms, "frac": bound_ms / ms_step,
                              "collective_bytes_per_direction": coll_bytes,
                              "nvlink_gbs": NVLINK_NOMINAL_GBS,
                              "nvlink_source": "nominal NVLink 5 bandwidth per direction per GPU",
                              "update_bound_ms": hbm_ms,
                              "bound_ms_at_measured_peer_copy_770": bound_peer_ms,
                              "frac_at_measured_peer_copy_770": bound_peer_ms / ms_step},
            "verified": verified,
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": kernels * args.steps,
            "nccl_calls": collectives * args.steps, "clocks": clocks,
        }
        if existing:
            line["existing_kernel"] = existing
        if stage_ms:
            line["stage_ms"] = stage_ms
        print(json.dumps(line), flush=True)
    barrier()
    for z in zs:
        z.close()
    if kz is not None:
        kz.close()
    comm.close()
    if td is not None:
        td.destroy_process_group()


if __name__ == "__main__":
    main()
