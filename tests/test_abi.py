"""The C-ABI shared library: loads without a GPU, exports every symbol the header
declares, and its host-only parts (plan geometry, argument checks) agree with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from raf_b200 import _lib

    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "raf_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"RAFB200_API\s+[\w\s\*]+?\b(rafb200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from raf_b200 import _lib

    names = _declared_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/raf_b200.h but not exported"
    # the ctypes table binds exactly the declared set
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_string(lib):
    assert lib.rafb200_version() >= 100
    assert isinstance(lib.rafb200_last_error(), bytes)


@pytest.mark.parametrize("n_ranks", [1, 2, 4, 8])
def test_plan_geometry_matches_oracle(n_ranks):
    from bench import bert_large_shapes, gpt2_medium_shapes, numel, resnet50_shapes
    from raf_b200.zero import Plan

    for shapes, bucket in ((resnet50_shapes(), 6553600), (bert_large_shapes(), 13107200),
                           (gpt2_medium_shapes(), 13107200), ([(7, 3), (1,), (0, 4), (9,)], 10)):
        for rank in {0, n_ranks - 1}:
            plan = Plan(shapes, n_ranks, rank, bucket)
            sizes = [numel(s) for s in shapes]
            nb, bucket_of = O.plan_buckets(sizes, bucket, rule=1)
            assert plan.num_buckets == nb
            assert plan.bucket_of.tolist() == bucket_of.tolist()
            for i, s in enumerate(shapes):
                rows = O.shard_rows(s[0], n_ranks)
                assert plan.shard_rows[i] == rows
                assert plan.shard_elems[i] == rows * (sizes[i] // s[0] if s[0] else numel(s[1:]))
                assert plan.padded_elems[i] == plan.shard_elems[i] * n_ranks
            assert plan.total_elems == sum(sizes)
            assert plan.total_shard * n_ranks == plan.total_padded


def test_plan_sizes_of_the_benchmark_configs():
    from bench import bert_large_shapes, gpt2_medium_shapes, resnet50_shapes
    from raf_b200.zero import Plan

    rn = Plan(resnet50_shapes(), 8, 0, 6553600)
    assert (rn.k, rn.total_elems, rn.total_padded, rn.num_buckets) == (161, 25557032, 25557032, 5)
    bl8 = Plan(bert_large_shapes(), 8, 0, 13107200)
    assert (bl8.k, bl8.total_elems, bl8.total_padded) == (391, 335141888, 335154176)
    assert Plan(bert_large_shapes(), 4, 0, 13107200).total_padded == 335145984
    g8 = Plan(gpt2_medium_shapes(), 8, 0, 13107200)
    assert (g8.k, g8.total_elems, g8.total_padded) == (292, 354823168, 354830336)


def test_plan_rejects_bad_arguments(lib):
    h = C.c_void_p()
    one = (C.c_int64 * 1)(4)
    assert lib.rafb200_plan_create(1, one, one, 4, 4, 10, C.byref(h)) == 1  # rank outside world
    assert b"rank" in lib.rafb200_last_error()
    assert lib.rafb200_plan_create(1, one, one, 0, 0, 10, C.byref(h)) == 1
    assert lib.rafb200_plan_create(1, None, one, 1, 0, 10, C.byref(h)) == 1


def test_invalid_computation_and_null_handles(lib):
    assert lib.rafb200_comm_size(None) == 0
    assert lib.rafb200_comm_rank(None) == -1
    assert lib.rafb200_tensor_list_total_elems(None) == 0
    assert lib.rafb200_lans_workspace_bytes(None) == 0
    assert lib.rafb200_sgd_list(None, 0.1, 0.9, 0.0, 1.0, None) == 1
    assert lib.rafb200_comm_check(None) == 1
    assert lib.rafb200_cast(None, 7, None, 0, 0, None) == 1  # bad dtype code


def test_comm_create_argument_checks(lib):
    h = C.c_void_p()
    assert lib.rafb200_comm_create(2, 2, 0, None, 100, C.byref(h)) == 1
    assert lib.rafb200_comm_create(2, 0, 0, None, 0, C.byref(h)) == 1


def test_comm_adopt_world_of_one_and_bad_arguments(lib):
    """The wrapper around a caller-owned ncclComm_t: a world of one needs no NCCL handle."""
    h = C.c_void_p()
    assert lib.rafb200_comm_adopt(None, 1, 0, C.byref(h)) == 0
    assert lib.rafb200_comm_size(h) == 1 and lib.rafb200_comm_rank(h) == 0
    assert lib.rafb200_comm_destroy(h) == 0
    assert lib.rafb200_comm_adopt(None, 2, 0, C.byref(h)) == 1  # world of two without a handle
    assert b"NULL ncclComm_t" in lib.rafb200_last_error()
    assert lib.rafb200_comm_adopt(None, 1, 3, C.byref(h)) == 1  # rank outside the world


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 with nothing but libc headers."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    src = tmp_path / "use_header.c"
    src.write_text('#include "raf_b200.h"\n'
                   "int main(void) { rafb200_hyper h; h.optimizer = RAFB200_OPT_LANS; "
                   "return rafb200_version() > 0 && h.optimizer == 2 ? 0 : 1; }\n")
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only",
                        "-I", os.path.join(ROOT, "include"), str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_no_cpu_fallback(tmp_path):
    """The product has no host path: CPU tensors are refused, and a missing library is an error
    at load time, not a silent switch to something else."""
    import subprocess
    import sys

    import torch

    from raf_b200 import op

    x = torch.zeros(8)
    with pytest.raises(ValueError, match="no CPU path"):
        op.sgd_(x, x.clone(), x.clone(), 0.1, 0.9)
    with pytest.raises(ValueError, match="no CPU path"):
        op.cast(x, "float16")
    env = dict(os.environ, RAFB200_LIB=str(tmp_path / "absent" / "libraf_b200.so"), PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", "from raf_b200 import _lib; _lib.load()"], env=env,
                       capture_output=True, text=True)
    assert r.returncode != 0 and "libraf_b200.so" in r.stderr


def test_plan_geometry_random_shapes_vs_oracle():
    """Shard rows, padding and bucket membership for random tensor lists, world sizes and bucket
    sizes, against the oracle's restatement of the partition passes."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    from raf_b200.zero import Plan, numel

    shape = st.lists(st.integers(0, 40), min_size=1, max_size=3).map(tuple)

    @settings(max_examples=80, deadline=None)
    @given(st.lists(shape, min_size=1, max_size=10), st.sampled_from([1, 2, 3, 4, 8]),
           st.sampled_from([1, 10, 100, 1000, 1 << 40]))
    def run(shapes, n, bucket):
        sizes = [numel(s) for s in shapes]
        nb, bucket_of = O.plan_buckets(sizes, bucket, rule=1)
        for rank in {0, n - 1}:
            plan = Plan(shapes, n, rank, bucket)
            assert plan.num_buckets == nb and plan.bucket_of.tolist() == bucket_of.tolist()
            for i, s in enumerate(shapes):
                rows = O.shard_rows(s[0], n)
                row = numel(s[1:]) if len(s) > 1 else 1
                assert plan.shard_rows[i] == rows == -(-s[0] // n)
                assert plan.shard_elems[i] == rows * row and plan.padded_elems[i] == rows * row * n
            assert plan.total_shard * n == plan.total_padded >= plan.total_elems == sum(sizes)
            plan.close()

    run()


def test_dist_config_lives_in_the_library():
    """include/raf/dist_config.h:17-48: same fields and defaults; the Python object and the C
    entry points read and write one process-wide record."""
    import ctypes as C

    from raf_b200 import _lib
    from raf_b200 import distributed as dist

    cfg = dist.get_config()
    before = cfg.dumps()
    try:
        assert before["auto_dp_profiling_start_iter"] == 2 and before["auto_dp_profiling_end_iter"] == 4
        assert before["group_bucket_size"] == 5000000000 and before["zero_opt_level"] in (0, 1, 2, 3)
        cfg.zero_opt_level = 2
        cfg.enable_data_parallel = True
        raw = dist._CDistConfig()
        _lib.check(_lib.load().rafb200_dist_config_get(C.byref(raw)))
        assert raw.zero_opt_level == 2 and raw.enable_data_parallel == 1
        assert cfg.enable_data_parallel is True and cfg.zero_opt_level == 2
        with pytest.raises(_lib.RafB200Error):
            cfg.zero_opt_level = 7
        with pytest.raises(KeyError):
            cfg.loads({"no_such_field": 1})
        with pytest.raises(AttributeError):
            cfg.no_such_field = 1
    finally:
        cfg.loads(before)
    assert cfg.dumps() == before
