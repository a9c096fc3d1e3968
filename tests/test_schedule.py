"""Invariants of the LANS work-item order (host only).

Every unit of work exactly once, every item after all items it waits for, the stage-1 items
in tensor order and no more parked items per tensor than the grid has room for - together the
properties that make the persistent kernel's in-kernel waits deadlock-free: an item only
waits for items with smaller tickets, and the earliest tensor with work outstanding can always
get a slot, because only parked items of that tensor (fewer than there are slots) and items of
earlier tensors (which complete without it) can occupy the others."""
import ctypes as C

import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

ELEMS = 1024
A_ELEMS = {0: 4096, 1: 7168, 2: 7168}  # per gradient dtype code (f32, f16, bf16)
KIND_A, KIND_BS, KIND_CS, KIND_BCP = 0, 1, 2, 3


def schedule(numels, g_dtype, with_norm, slots_total, lead_elems, gap_items):
    from raf_b200 import _lib

    lib = _lib.load()
    arr = (C.c_int64 * len(numels))(*numels)
    count = C.c_size_t()
    _lib.check(lib.rafb200_lans_schedule(len(numels), arr, g_dtype, int(with_norm), slots_total, lead_elems,
                                         gap_items, None, 0, C.byref(count)))
    items = np.zeros((count.value, 2), np.uint32)
    _lib.check(lib.rafb200_lans_schedule(len(numels), arr, g_dtype, int(with_norm), slots_total, lead_elems,
                                         gap_items, items.ctypes.data, count.value, C.byref(count)))
    return items[:, 0] >> 30, items[:, 0] & ((1 << 30) - 1), items[:, 1]


def park_cap(cells_total):
    return cells_total * 5 // 8


def check(numels, g_dtype, with_norm, slots_total, lead_elems, gap_items):
    kind, tensor, chunk = schedule(numels, g_dtype, with_norm, slots_total, lead_elems, gap_items)
    n_a = [(n + A_ELEMS[g_dtype] - 1) // A_ELEMS[g_dtype] for n in numels]
    n_b = [(n + ELEMS - 1) // ELEMS for n in numels]
    cap = park_cap(slots_total)
    seen = {}
    for pos, key in enumerate(zip(kind.tolist(), tensor.tolist(), chunk.tolist())):
        assert key not in seen, f"item {key} twice"
        seen[key] = pos
    stage1_tensors = []
    for t, n in enumerate(numels):
        a_pos = [seen[(KIND_A, t, c)] for c in range(n_a[t])] if with_norm else []
        if not with_norm:
            assert not any(k == KIND_A for k in kind.tolist())
        parked = [c for c in range(n_b[t]) if (KIND_BCP, t, c) in seen]
        streamed = [c for c in range(n_b[t]) if (KIND_BS, t, c) in seen]
        assert sorted(parked + streamed) == list(range(n_b[t]))      # stage 1 of every chunk, once
        assert len(parked) <= cap and (len(parked) == min(n_b[t], cap))
        assert all((KIND_CS, t, c) in seen for c in streamed)        # a streamed chunk is updated later
        assert not any((KIND_CS, t, c) in seen for c in parked)      # a parked one is not loaded again
        s1_pos = [seen[(KIND_BS, t, c)] for c in streamed] + [seen[(KIND_BCP, t, c)] for c in parked]
        if s1_pos:
            stage1_tensors.append((min(s1_pos), max(s1_pos), t))
            if a_pos:
                assert max(a_pos) < min(s1_pos)                      # stage 1 needs the gradient norm
            for c in streamed:
                assert seen[(KIND_CS, t, c)] > max(s1_pos)           # stage 2 needs the update norms
            if parked and streamed:                                  # the parked part is the tail
                assert max(seen[(KIND_BS, t, c)] for c in streamed) < min(seen[(KIND_BCP, t, c)] for c in parked)
    assert len(seen) == sum(n_a) * (1 if with_norm else 0) + sum(n_b) + sum(
        1 for k in kind.tolist() if k == KIND_CS)
    stage1_tensors.sort()
    for (lo1, hi1, t1), (lo2, hi2, t2) in zip(stage1_tensors, stage1_tensors[1:]):
        assert hi1 < lo2 and t1 < t2                                 # stage 1 runs tensor by tensor


@pytest.mark.parametrize("with_norm", [True, False])
def test_schedule_of_the_benchmark_shapes(with_norm):
    from bench import bert_large_shapes, gpt2_medium_shapes, numel

    for shapes, g_dtype in ((bert_large_shapes(), 1), (gpt2_medium_shapes(), 2)):
        check([numel(s) for s in shapes], g_dtype, with_norm, 148 * 29, 8 << 20, 0)


@settings(max_examples=30, deadline=None)
@given(st.lists(st.one_of(st.integers(0, 5), st.integers(0, 70000), st.integers(0, 1_000_000)), min_size=0, max_size=10),
       st.sampled_from([0, 1, 2]), st.booleans(), st.sampled_from([1, 3, 29, 147, 4292]),
       st.sampled_from([0, 1, ELEMS, 1 << 20, 8 << 20]), st.sampled_from([0, 1, 7, 300, 5000]))
def test_schedule_invariants_random_lists(numels, g_dtype, with_norm, slots_total, lead_elems, gap_items):
    check(numels, g_dtype, with_norm, slots_total, lead_elems, gap_items)


def test_schedule_rejects_bad_arguments():
    from raf_b200 import _lib

    lib = _lib.load()
    count = C.c_size_t()
    neg = (C.c_int64 * 1)(-1)
    assert lib.rafb200_lans_schedule(1, neg, 0, 1, 15, 0, 0, None, 0, C.byref(count)) == 1
    one = (C.c_int64 * 1)(10000)
    assert lib.rafb200_lans_schedule(1, one, 0, 1, 0, 0, 0, None, 0, C.byref(count)) == 1  # no slots
    small = (C.c_uint32 * 2)()
    # 3 gradient-norm items of 4096 + 10 chunks of 1024, 6 of them parked, 4 streamed twice
    assert lib.rafb200_lans_schedule(1, one, 0, 1, 10, 0, 0, small, 1, C.byref(count)) == 1
    assert count.value == 3 + 10 + 4


GAP = 1000  # the same distance between a tensor's stage-1 and update items in both calls


def partition(numels, g_dtype, with_norm, grid):
    from raf_b200 import _lib

    lib = _lib.load()
    arr = (C.c_int64 * len(numels))(*numels)
    count, ce, co = C.c_size_t(), C.c_int(), C.c_int()
    _lib.check(lib.rafb200_lans_partition(len(numels), arr, g_dtype, int(with_norm), grid, 8 << 20, GAP, None, None, 0,
                                          C.byref(count), C.byref(ce), C.byref(co)))
    off = np.zeros(2 * grid + 1, np.uint32)
    items = np.zeros((count.value, 2), np.uint32)
    _lib.check(lib.rafb200_lans_partition(len(numels), arr, g_dtype, int(with_norm), grid, 8 << 20, GAP,
                                          off.ctypes.data, items.ctypes.data, count.value, C.byref(count),
                                          C.byref(ce), C.byref(co)))
    return off, items, ce.value, co.value


def check_partition(numels, g_dtype, with_norm, grid):
    """What the kernel's waits for cells rely on: every item in exactly one list, every list in
    the global order, the parked items of a list numbered 0, 1, 2, ... and never more of one
    tensor in a list than the list has cells."""
    off, items, cells_even, cells_odd = partition(numels, g_dtype, with_norm, grid)
    kind, tensor, chunk = schedule(numels, g_dtype, with_norm, grid * (cells_even + cells_odd), 8 << 20, GAP)
    order = {key: pos for pos, key in enumerate(zip(kind.tolist(), tensor.tolist(), chunk.tolist()))}
    assert off[0] == 0 and off[-1] == len(order) and np.all(np.diff(off.astype(np.int64)) >= 0)
    seen = set()
    sizes = []
    for h in range(2 * grid):
        rows = items[off[h]:off[h + 1]]
        k = (rows[:, 0] >> 30).tolist()
        t = (rows[:, 0] & ((1 << 30) - 1)).tolist()
        c = (rows[:, 1] & ((1 << 21) - 1)).tolist()
        seq = (rows[:, 1] >> 21).tolist()
        pos = [order[key] for key in zip(k, t, c)]
        assert pos == sorted(pos), "a list does not keep the global order"
        seen.update(zip(k, t, c))
        parked = [i for i, kk in enumerate(k) if kk == KIND_BCP]
        assert [seq[i] for i in parked] == [j % 2048 for j in range(len(parked))]
        assert all(seq[i] == 0 for i, kk in enumerate(k) if kk != KIND_BCP)
        per_tensor = {}
        for i in parked:
            per_tensor[t[i]] = per_tensor.get(t[i], 0) + 1
        limit = cells_even if h % 2 == 0 else cells_odd
        assert not per_tensor or max(per_tensor.values()) <= limit, (h, max(per_tensor.values()), limit)
        sizes.append(len(k))
    assert len(seen) == len(order)
    return sizes


def test_partition_of_the_benchmark_shapes():
    from bench import bert_large_shapes, gpt2_medium_shapes, numel

    for shapes, g_dtype in ((bert_large_shapes(), 1), (gpt2_medium_shapes(), 2)):
        for world in (1, 8):
            numels = [-(-s[0] // world) * (numel(s) // s[0]) for s in shapes]
            sizes = check_partition(numels, g_dtype, True, 148)
            even, odd = sizes[0::2], sizes[1::2]
            assert max(even) - min(even) <= 2 + len(numels) // 50 and max(odd) - min(odd) <= 2 + len(numels) // 50


@settings(max_examples=25, deadline=None)
@given(st.lists(st.one_of(st.integers(0, 5), st.integers(0, 70000), st.integers(0, 600_000)), min_size=0, max_size=8),
       st.sampled_from([0, 1, 2]), st.booleans(), st.sampled_from([1, 2, 7, 148]))
def test_partition_invariants_random_lists(numels, g_dtype, with_norm, grid):
    check_partition(numels, g_dtype, with_norm, grid)
