"""Builds libraf_b200.so in-tree with nvcc for sm_100a.

``python -m raf_b200.build`` (or ``raf_b200.build.build()``) compiles every
source under ``raf_b200/csrc`` to an object file and links them, together with
NCCL, into ``raf_b200/libraf_b200.so``.  Cross-compilation needs no GPU.

It then compiles the RAF-side glue (``csrc/raf_dialect/b200_ops.cc``) against
``csrc/raf_compat`` - a small stand-in for the RAF headers a dialect touches -
into ``raf_b200/libraf_b200_glue.so``, so that the glue is type-checked and can
be driven on fake tensors by the tests.  Inside a RAF tree the same file is
compiled against RAF's own headers instead.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libraf_b200.so")
GLUE_LIB = os.path.join(HERE, "libraf_b200_glue.so")
COMPAT = os.path.join(CSRC, "raf_compat")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "-Xcompiler", "-Wall", "--expt-relaxed-constexpr"] + ARCH


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libraf_b200.so cannot be built")
    return nvcc


def _sources():
    out = []
    for root, _dirs, files in os.walk(CSRC):
        if "raf_dialect" in root or "raf_compat" in root:
            continue  # the glue is a library of its own, see build_glue()
        for f in sorted(files):
            if f.endswith((".cu", ".cc")):
                out.append(os.path.join(root, f))
    return out


def _headers_mtime() -> float:
    m = os.path.getmtime(os.path.join(HERE, "..", "include", "raf_b200.h"))
    for root, _dirs, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".h", ".cuh")):
                m = max(m, os.path.getmtime(os.path.join(root, f)))
    return m


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    srcs = _sources()
    hdr_m = _headers_mtime()
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s).rsplit(".", 1)[0] + ".o")
        objs.append(o)
        stale = force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_m)
        if stale:
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-x", "cu", "-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or ptxas_info or r.returncode != 0:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or not os.path.exists(LIB):
        link = [nvcc, "-shared"] + ARCH + ["-Xcompiler", "-fPIC", "-o", LIB] + objs + ["-lnccl"]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(link) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("link failed")
    build_glue(nvcc, force or bool(jobs))
    return LIB


def build_glue(nvcc: str, force: bool = False) -> str:
    """b200_ops.cc + the raf_compat runtime and test harness -> libraf_b200_glue.so."""
    srcs = [os.path.join(CSRC, "raf_dialect", "b200_ops.cc"), os.path.join(COMPAT, "registry.cc"),
            os.path.join(COMPAT, "harness.cc")]
    deps = list(srcs) + [os.path.join(HERE, "..", "include", "raf_b200.h")]
    for root, _dirs, files in os.walk(COMPAT):
        deps += [os.path.join(root, f) for f in files if f.endswith(".h")]
    newest = max(os.path.getmtime(d) for d in deps)
    if not force and os.path.exists(GLUE_LIB) and os.path.getmtime(GLUE_LIB) >= newest:
        return GLUE_LIB
    cmd = [nvcc, "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
           "-Xcompiler", "-Wall", "-x", "cu"] + ARCH + [
        "-I", os.path.join(COMPAT, "include"), "-I", os.path.join(COMPAT, "src", "op", "dialect", "b200"),
        "-I", COMPAT, "-I", os.path.join(HERE, "..", "include"), "-o", GLUE_LIB] + srcs + [
        "-L", HERE, "-lraf_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("building the RAF dialect glue failed")
    return GLUE_LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
