"""Host side of the multi-device fan-out behind `_mlir_ciface_forward`, without a device: the slice
rule, the worker threads, the join, and the hand-over of a failing part's status (the failure is
made on the host: a stand-in job that returns an error).  The GPU part runs where two devices are
visible."""
import ctypes

import numpy as np
import pytest

from nncv_b200._lib import lib
from nncv_b200.shard import shard_range


def c_shard(n, r, w):
    lo, hi = ctypes.c_int(), ctypes.c_int()
    assert lib().nncv_b200_shard_range(n, r, w, ctypes.byref(lo), ctypes.byref(hi)) == 0
    return lo.value, hi.value


@pytest.mark.parametrize("n,world", [(256, 8), (256, 3), (5, 8), (0, 2), (7, 7), (1000, 6)])
def test_slices_tile_the_batch_and_match_the_python_rule(n, world):
    cover = []
    for r in range(world):
        assert c_shard(n, r, world) == shard_range(n, r, world)
        cover += list(range(*c_shard(n, r, world)))
    assert cover == list(range(n))
    assert lib().nncv_b200_shard_range(4, 4, 4, None, None) == 1


def fanout(n, parts, fail_rank=-1):
    lo, hi = (ctypes.c_int * parts)(), (ctypes.c_int * parts)()
    other = ctypes.c_int()
    rc = lib().nncv_b200_selftest_fanout(n, parts, fail_rank, lo, hi, ctypes.byref(other))
    return rc, list(lo), list(hi), other.value


@pytest.mark.parametrize("n,parts", [(256, 8), (10, 4), (3, 8), (1, 1)])
def test_every_part_runs_once_on_its_own_thread(n, parts):
    for _ in range(3):                      # the workers are reused from call to call
        rc, lo, hi, other = fanout(n, parts)
        live = min(n, parts)
        assert rc == 0
        assert [(lo[r], hi[r]) for r in range(live)] == [shard_range(n, r, live) for r in range(live)]
        assert all(lo[r] == -1 for r in range(live, parts))
        assert other == live - 1            # part 0 on the caller's thread, the others on workers


@pytest.mark.parametrize("fail_rank", [0, 3, 7])
def test_a_failing_part_is_reported_after_all_parts_finished(fail_rank):
    rc, lo, hi, _ = fanout(64, 8, fail_rank)
    assert rc == 6                                            # the injected status
    msg = lib().nncv_b200_last_error().decode()
    assert f"part {fail_rank} of 8" in msg and "injected failure" in msg
    assert all(h > l >= 0 for l, h in zip(lo, hi))            # nobody was skipped or left running
    assert fanout(64, 8)[0] == 0                              # and the pool still works


@pytest.mark.gpu
def test_batch_split_over_two_devices_equals_one_device():
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    from oracle import binding as ob
    from nncv_b200 import runtime as rt
    from nncv_b200._lib import F16
    from nncv_b200.split_params import random_input, random_state_dict, to_flat_array
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    x = random_input(37, 96, 96, 4, "normal")                  # ragged split: 19 + 18
    torch.cuda.set_device(0)
    try:
        rt.load_blob("resnet18", blob, F16)
        one = np.zeros((37, 1000), np.float32)
        rt.forward(one, x)
        rt.load_blob("resnet18", blob, F16, device_mask=0b11)
        two = np.zeros((37, 1000), np.float32)
        rt.forward(two, x)
        rt.forward(two, x)
        # image i does not depend on its batch or device: the split changes nothing
        assert np.array_equal(one, two)
        ref = ob.resnet_forward(18, x[:8], blob)
        assert np.linalg.norm(two[:8] - ref) / np.linalg.norm(ref) <= 1e-2
        big = random_input(256, 64, 64, 5, "normal")
        out = np.zeros((256, 1000), np.float32)
        rt.forward(out, big)
        rt.unload()
        rt.load_blob("resnet18", blob, F16)
        out1 = np.zeros((256, 1000), np.float32)
        rt.forward(out1, big)
        assert np.array_equal(out, out1)
    finally:
        rt.unload()
    assert lib().nncv_b200_device_status() == 0
