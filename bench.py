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
         inside the timed region;
  roofline  algorithmic bytes of the update kernel / its duration, against the
         measured HBM copy bandwidth;
  cpu_baseline  the CPU oracle (a restatement of the reference's math, OpenMP)
         timed on a bounded sample of the same workload.
Workloads (BASELINE.json configs): bert_lans (default, config 3), rn50_sgd (2),
gpt2_adam (4), flat_adam:<Mi elements> (5), flat_sgd (1).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 << 20


NVLINK_MEASURED_GBS = 770.0  # peer copy, per direction per GPU, measured on this pool
# DRAM bytes (read + write) of one launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (workload, n_gpus, shard_of) -> bytes
MEASURED_TRAFFIC = {
    ("bert_lans", 1, 1): 14644761344,
    ("bert_lans", 1, 8): 1695229304,
    ("rn50_sgd", 1, 1): 454225920,
    ("gpt2_adam", 1, 8): 1184124416,
}


# --------------------------------------------------------------------------- workloads
def workload(name: str):
    """-> dict(shapes, optimizer, g_dtype, p_dtype, hyper kwargs, bucket_elems, bytes_per_elem, label)"""
    from raf_b200.zero import bert_large_shapes, gpt2_medium_shapes, resnet50_shapes

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
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# --------------------------------------------------------------------------- CPU baseline
class CpuArm:
    """The oracle (C/OpenMP restatement of the reference math) on the host cores: one rank's
    full-size, unsharded update of a prefix of the workload's tensors, no collectives.
    Inputs are generated once (untimed); every `step()` is one optimizer step over them."""

    def __init__(self, wl, max_elems=None):
        import numpy as np

        from oracle import oracle as O
        from raf_b200.zero import numel

        self.O, self.wl = O, wl
        code = {"float32": O.F32, "float16": O.F16, "bfloat16": O.BF16}
        self.out_code = code[wl["p_dtype"]]
        rng = np.random.default_rng(0)
        self.p, self.m, self.v, self.g = [], [], [], []
        self.elems = 0
        for s in wl["shapes"]:
            n = numel(s)
            if n == 0:
                continue
            if max_elems is not None and self.elems + n > max_elems and self.elems > 0:
                break
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
        return (f"first {self.tensors} of {len(self.wl['shapes'])} tensors ({self.elems} elements), "
                f"{steps} optimizer steps, {spent:.2f} s of host time; C/OpenMP restatement of the "
                f"reference math (RAF's TVM CPU path cannot be built here; LANS and Adam have no CPU path in RAF)")


def cpu_baseline(wl, budget_s=10.0):
    """Steps of the CPU arm until about `budget_s` seconds of CPU work have been spent."""
    arm = CpuArm(wl)
    arm.step()  # page in, warm the thread pool
    spent, steps = 0.0, 0
    while spent < budget_s and steps < 200:
        spent += arm.step()
        steps += 1
    return {"value": arm.elems * steps / spent, "unit": "param-elements/s", "cores": arm.O.num_threads(),
            "kind": "port", "sample": arm.describe(steps, spent)}


def run_reference_arm(args, wl):
    """--impl reference: the CPU restatement of the reference's path on all host threads.
    A step is one optimizer step over a bounded prefix of the workload, sized from a probe so
    that warm-up plus timed steps stay within a few minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from raf_b200.zero import numel

    total = sum(numel(s) for s in wl["shapes"])
    probe = CpuArm(wl, max_elems=32 << 20)
    probe.step()
    rate = probe.elems / probe.step()  # elements/s on this box
    nsteps = max(1, args.steps + args.warmup)
    max_elems = int(min(total, max(8 << 20, rate * 120.0 / nsteps)))
    arm = CpuArm(wl, max_elems=max_elems) if max_elems < total else CpuArm(wl)
    for _ in range(args.warmup):
        arm.step()
    times = [arm.step() for _ in range(args.steps)]
    spent = sum(times)
    val = arm.elems * len(times) / spent
    cpu = {"value": val, "unit": "param-elements/s", "cores": arm.O.num_threads(), "kind": "port",
           "sample": arm.describe(len(times), spent)}
    line = {
        "impl": "reference", "metric": "ZeRO optimizer-step param-elements/s", "value": val,
        "unit": "param-elements/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / val, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["label"], "note": "CPU host cores; ms_per_step extrapolated from the sample to the full parameter count"},
        "cpu_baseline": cpu,
        "e2e": {"value": val, "unit": "param-elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="bert_lans")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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
    ap.add_argument("--no-views", action="store_true",
                    help="symmetric modes: keep gradients and parameters in separate tensors "
                         "(pack / unpack copies) instead of inside the symmetric buffer")
    ap.add_argument("--stages", action="store_true",
                    help="N > 1: also time each stage of the step alone (pack, reduce-scatter, ...)")
    ap.add_argument("--existing-kernel", action="store_true",
                    help="also time the reference's own LANS kernel (oracle/_ref) on the same shards")
    args = ap.parse_args()
    wl = workload(args.workload)
    if args.bucket_elems:
        wl["bucket_elems"] = args.bucket_elems
    if args.impl == "reference":
        run_reference_arm(args, wl)
        return

    import numpy as np
    import torch

    from raf_b200 import distributed as dist
    from raf_b200.op import torch_dtype
    from raf_b200.zero import Plan, ZeroStep, make_hyper, numel

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
        wl["label"] += f" -- rank 0's shards of a {args.shard_of}-way partition, no collectives"
        part.close()
    k = len(shapes)
    total = sum(numel(s) for s in shapes)
    plan = Plan(shapes, world, rank, wl["bucket_elems"])
    gdt, pdt = torch_dtype(wl["g_dtype"]), torch_dtype(wl["p_dtype"])
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000 * rank + 1)

    def randn(n, std, dtype):
        return (torch.randn(n, generator=gen, device=dev, dtype=torch.float32) * std).to(dtype)

    # fp32 master shards and optimizer state (rank-local), model-dtype full parameters
    p = [randn(int(plan.shard_elems[i]), 0.02, torch.float32) for i in range(k)]
    m = [torch.zeros_like(x) for x in p]
    v = [torch.zeros_like(x) for x in p]
    params = [torch.zeros(numel(s), dtype=pdt, device=dev) for s in shapes]
    if world == 1 and pdt == torch.float32:
        params = p  # one rank, fp32 model: the parameters are the master copy (no second write)
    # Gradient sets: the step leaves the caller's gradients untouched (they are packed into
    # the bucket buffers first), so a set can be reused; two sets alternate.
    nsets = 1 if world == 1 else 2
    if args.collectives == "auto":
        # two ranks: plain peer loads / stores beat the switch-side reduction (measured 2.25 ms
        # against 2.47 ms); from four ranks on the multicast kernels win
        args.collectives = "peer" if world == 2 else "multimem"
    if world > 1 and not args.update_blocks and wl["optimizer"] == "lans":
        # leave block slots to the collective kernels running beside the update: 16 SMs' worth
        # with the multicast kernels, one block per SM with peer loads (measured 2.13 against
        # 2.25 ms at two ranks)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        args.update_blocks = 2 * sms if args.collectives == "peer" else 3 * (sms - 16)
    collectives_used = args.collectives if world > 1 else "none"
    views_used = 0
    gsets = [[randn(numel(s), 1e-3 * wl["loss_scale"], gdt) for s in shapes] for _ in range(nsets)]
    zs = []
    for gs in gsets:
        z = ZeroStep(plan, comm, gdt, pdt, wl["optimizer"])
        if world > 1 and args.collectives != "nccl":
            try:
                z.attach_symmetric(comm_blocks=args.comm_blocks, multicast=(args.collectives == "multimem"))
                if args.collectives == "multimem" and not z.multicast:
                    collectives_used = "peer (no multicast address available)"
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

    # ---- the update kernel alone (this rank's shards, no collectives): roofline ----
    shard_elems = int(plan.total_shard)
    if world == 1:
        kern_ms = ms_step
        kz = None
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
                "traffic": MEASURED_TRAFFIC.get((args.workload, world, args.shard_of if args.shard_of > 1 else 1)),
                "peak_source": peak_src,
                "kernel": {"sgd": "update_list_kernel<SgdOp>", "adam": "update_list_kernel<AdamOp>",
                           "lans": "lans_kernel"}[wl["optimizer"]],
                "kernel_ms": kern_ms, "algorithmic_bytes_per_launch": wl["bytes_per_elem"] * shard_elems}

    # ---- step roofline: slower of update bytes at HBM peak and collective bytes at 900 GB/s ----
    gsz, psz = gsets[0][0].element_size(), params[0].element_size()
    coll_bytes = (world - 1) / world * int(plan.total_padded) * (gsz + psz)
    # measured peer-copy bandwidth of this pool (770 GB/s per direction per GPU); 900 nominal
    bound_ms = max(wl["bytes_per_elem"] * shard_elems / (peak * 1e9), coll_bytes / NVLINK_MEASURED_GBS / 1e9) * 1e3
    bound_nominal_ms = max(wl["bytes_per_elem"] * shard_elems / (peak * 1e9), coll_bytes / 900e9) * 1e3

    # ---- end to end: host gradients in, host parameters out ----
    e2e = None
    if not args.no_e2e:
        grads_host = [torch.empty(numel(s), dtype=gdt).pin_memory() for s in shapes]
        params_host = [torch.empty(numel(s), dtype=pdt).pin_memory() for s in shapes]
        for gh, gd in zip(grads_host, gsets[0]):
            gh.copy_(gd)
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
        e2e = {"value": total / (e2e_ms * 1e-3), "unit": "param-elements/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": total * gsz * world, "d2h_bytes_per_step": total * psz * world,
               "steps": args.e2e_steps}

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
    if args.existing_kernel and wl["optimizer"] == "lans":
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
            existing = {"kernel": "reference multi_tensor_lans_cuda<float> compiled for sm_100a",
                        "ms": r0.elapsed_time(r1) / 5, "note": "fp32 gradients, no cast/unscale, no fp16 copy"}

    if rank == 0:
        cpu = None if args.no_cpu_baseline else cpu_baseline(wl)
        line = {
            "metric": "ZeRO optimizer-step param-elements/s", "value": total / (ms_step * 1e-3),
            "unit": "param-elements/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["label"], "optimizer": wl["optimizer"], "n_tensors": k,
                       "elements": total, "shard_elements_per_rank": shard_elems,
                       "bucket_elems": wl["bucket_elems"], "buckets": plan.num_buckets if world > 1 else 1,
                       "gradient_sets": nsets, "collectives": collectives_used,
                       "tensors_inside_symmetric_buffer": views_used,
                       "l2": (f"inputs larger than L2 ({wl['bytes_per_elem'] * shard_elems >> 20} MiB touched per step per rank)"
                              if wl['bytes_per_elem'] * shard_elems > (126 << 20) else
                              f"working set of {wl['bytes_per_elem'] * shard_elems >> 20} MiB fits the 126 MB L2 and is not "
                              "flushed between steps: not a DRAM-bound measurement")},
            "roofline": roofline,
            "step_roofline": {"bound_ms": bound_ms, "frac": bound_ms / ms_step,
                              "collective_bytes_per_direction": coll_bytes,
                              "nvlink_gbs": NVLINK_MEASURED_GBS, "nvlink_source": "measured peer copy on this pool",
                              "bound_ms_at_nominal_900": bound_nominal_ms,
                              "frac_at_nominal_900": bound_nominal_ms / ms_step},
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
