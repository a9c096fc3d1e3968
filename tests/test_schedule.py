"""Invariants of the LANS work-item order (host only): every (phase, tensor, chunk) exactly
once, and every item after all items it waits for - the property that makes the persistent
kernel's in-kernel waits deadlock-free whatever the number of resident blocks."""
import ctypes as C

import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

CHUNK = 4096


def schedule(numels, with_norm, window_elems, slack):
    from raf_b200 import _lib

    lib = _lib.load()
    arr = (C.c_int64 * len(numels))(*numels)
    count = C.c_size_t()
    _lib.check(lib.rafb200_lans_schedule(len(numels), arr, int(with_norm), window_elems, slack, None, 0,
                                         C.byref(count)))
    items = np.zeros((count.value, 2), np.uint32)
    _lib.check(lib.rafb200_lans_schedule(len(numels), arr, int(with_norm), window_elems, slack,
                                         items.ctypes.data, count.value, C.byref(count)))
    return items[:, 0] >> 30, items[:, 0] & ((1 << 30) - 1), items[:, 1]


def check(numels, with_norm, window_elems, slack):
    phase, tensor, chunk = schedule(numels, with_norm, window_elems, slack)
    nchunks = [(n + CHUNK - 1) // CHUNK for n in numels]
    phases = (0, 1, 2) if with_norm else (1, 2)
    assert len(phase) == sum(nchunks) * len(phases)
    seen = set(zip(phase.tolist(), tensor.tolist(), chunk.tolist()))
    assert len(seen) == len(phase)                       # no item twice
    for ph in phases:                                    # and every expected item present
        for t, nc in enumerate(nchunks):
            assert all((ph, t, c) in seen for c in range(nc))
    last = {}                                            # position of the last item of (phase, tensor)
    first = {}
    for pos, key in enumerate(zip(phase.tolist(), tensor.tolist())):
        last[key] = pos
        first.setdefault(key, pos)
    for t, nc in enumerate(nchunks):
        if nc == 0:
            continue
        if with_norm:
            assert last[(0, t)] < first[(1, t)]          # moments need the gradient norm
        assert last[(1, t)] < first[(2, t)]              # the update needs the update norms


@pytest.mark.parametrize("with_norm", [True, False])
def test_schedule_of_the_benchmark_shapes(with_norm):
    from raf_b200.zero import bert_large_shapes, gpt2_medium_shapes, numel

    for shapes in (bert_large_shapes(), gpt2_medium_shapes()):
        check([numel(s) for s in shapes], with_norm, 32 << 20, 8 * 148)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.one_of(st.integers(0, 5), st.integers(0, 70000), st.integers(0, 3_000_000)), min_size=0, max_size=12),
       st.booleans(), st.sampled_from([0, 1, CHUNK, 1 << 20, 32 << 20]), st.sampled_from([0, 1, 7, 300, 5000]))
def test_schedule_invariants_random_lists(numels, with_norm, window_elems, slack):
    check(numels, with_norm, window_elems, slack)


def test_schedule_rejects_bad_arguments():
    from raf_b200 import _lib

    lib = _lib.load()
    count = C.c_size_t()
    neg = (C.c_int64 * 1)(-1)
    assert lib.rafb200_lans_schedule(1, neg, 1, 0, 0, None, 0, C.byref(count)) == 1
    one = (C.c_int64 * 1)(10000)
    small = (C.c_uint32 * 2)()
    assert lib.rafb200_lans_schedule(1, one, 1, 0, 0, small, 1, C.byref(count)) == 1  # 9 items, room for 1
    assert count.value == 9
