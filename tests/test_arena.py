"""The activation arena planner (greedy by size for offset calculation) against the known answer of
nncv's own MemSolver test and against the properties any valid plan has.  Host only."""
import ctypes

import numpy as np
import pytest

from nncv_b200._lib import lib


def plan(first, last, size, align=1):
    n = len(size)
    F = (ctypes.c_int * n)(*first)
    L = (ctypes.c_int * n)(*last)
    S = (ctypes.c_size_t * n)(*size)
    O = (ctypes.c_size_t * n)()
    T = ctypes.c_size_t()
    rc = lib().nncv_b200_arena_plan(n, F, L, S, align, O, ctypes.byref(T))
    assert rc == 0, lib().nncv_b200_last_error()
    return list(O), T.value


def check_valid(first, last, size, off, total, align=1):
    up = lambda v: (v + align - 1) // align * align
    n = len(size)
    for i in range(n):
        assert off[i] % align == 0 and off[i] + up(size[i]) <= total
        for j in range(i):
            if max(first[i], first[j]) <= min(last[i], last[j]):   # alive together
                assert off[i] + up(size[i]) <= off[j] or off[j] + up(size[j]) <= off[i], (i, j)


def test_known_answer_of_the_reference_memsolver_test():
    """tests/MemSolver/test.cpp:17-37 of nncv (the example of the paper): total consumption 124."""
    first = [0, 1, 2, 3, 4, 5, 6, 7]
    last = [1, 4, 5, 5, 5, 7, 8, 8]
    size = [32, 28, 36, 16, 8, 64, 10, 40]
    off, total = plan(first, last, size)
    assert total == 124
    check_valid(first, last, size, off, total)


@pytest.mark.parametrize("seed", range(20))
def test_random_plans_are_valid_and_no_worse_than_private_buffers(seed):
    g = np.random.default_rng(seed)
    n = int(g.integers(1, 60))
    first = [int(v) for v in g.integers(0, 40, n)]
    last = [f + int(v) for f, v in zip(first, g.integers(0, 8, n))]
    size = [int(v) for v in g.integers(1, 5000, n)]
    align = int(g.choice([1, 16, 1024]))
    off, total = plan(first, last, size, align)
    check_valid(first, last, size, off, total, align)
    up = lambda v: (v + align - 1) // align * align
    assert total <= sum(up(s) for s in size)
    # lower bound: the most memory alive at any one op
    peak = max(sum(up(s) for f, l, s in zip(first, last, size) if f <= t <= l) for t in range(0, 50))
    assert total >= peak


def test_chain_of_equal_tensors_needs_two_buffers():
    """x0 -> x1 -> x2 ...: each tensor is read by the next op only, so two slots alternate."""
    n = 12
    first, last, size = list(range(n)), [i + 1 for i in range(n)], [100] * n
    off, total = plan(first, last, size)
    assert total == 200 and set(off) == {0, 100}


def test_bad_interval_and_null_arguments():
    L = lib()
    T = ctypes.c_size_t()
    assert L.nncv_b200_arena_plan(0, None, None, None, 1, None, ctypes.byref(T)) == 0 and T.value == 0
    F, La, S, O = (ctypes.c_int * 1)(3), (ctypes.c_int * 1)(2), (ctypes.c_size_t * 1)(8), (ctypes.c_size_t * 1)()
    assert L.nncv_b200_arena_plan(1, F, La, S, 1, O, ctypes.byref(T)) == 1
    assert L.nncv_b200_arena_plan(1, F, La, S, 1, O, None) == 1
