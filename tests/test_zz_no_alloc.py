"""nncv_b200_matmul_noalloc: the matmul variant for callers that may not allocate device memory
(a server whose own pool owns all device memory, or a loop that cannot afford the device-wide
synchronisation of cudaMalloc).  Its repacked B lives in a fixed array inside the library image.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  The checks call the entry point through the C ABI and compare with the allocating
entry point nncv_b200_matmul on the same operands, twice in a row, with the second problem
smaller than the first so that stale bytes of the first call sit behind it in the shared array."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import binding as ob  # noqa: E402
from nncv_b200._lib import BF16, F16, F32, check, lib  # noqa: E402
import gpu_util as G  # noqa: E402


def _both(m, n, k, ab, c_dt, bias, relu, seed, ref=False):
    g = np.random.default_rng(seed)
    A = G.dev(g.uniform(-1, 1, (m, k)).astype(np.float32), ab)
    B = G.dev(g.uniform(-1, 1, (k, n)).astype(np.float32), ab)
    bias_t = G.dev(g.standard_normal(n).astype(np.float32), F32) if bias else None
    outs = []
    for fn in (lib().nncv_b200_matmul_noalloc, lib().nncv_b200_matmul):
        C = torch.full((m, n), float("nan"), device="cuda", dtype=G.TORCH_DT[c_dt])
        check(fn(G.p(A), G.p(B), G.p(C), m, n, k, ab, c_dt, G.p(bias_t), int(relu), G.stream_ptr()))
        torch.cuda.synchronize()
        assert lib().nncv_b200_device_status() == 0, lib().nncv_b200_last_error()   # no wait ran out in either path
        outs.append(G.host(C))
    if ref:
        r = ob.matmul(G.host(A), G.host(B), G.host(bias_t) if bias else None, relu, acc64=True)
        assert G.rel_l2(outs[0], r) <= (2e-3 if c_dt != F32 else 1e-5)   # and directly against the CPU oracle
    return outs


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    # first call: large enough to fill most of the fixed array; second: small, ragged, other dtype
    a1, b1 = _both(512, 2048, 1024, F16, F16, True, True, 1)
    assert np.isfinite(a1).all() and G.rel_l2(a1, b1) <= 1e-6
    a2, b2 = _both(100, 200, 72, BF16, F32, False, False, 2, ref=True)
    assert np.isfinite(a2).all() and G.rel_l2(a2, b2) <= 1e-6
    # and once more on the first shape: the array was overwritten in between
    a3, b3 = _both(512, 2048, 1024, F16, F16, True, True, 3)
    assert G.rel_l2(a3, b3) <= 1e-6


def test_narrow_output_and_a_problem_exactly_at_the_limit():
    # N < 64 takes the gather kernel; N = K = 2048 packs into exactly the 8 MiB the array holds
    a, b = _both(300, 40, 136, F16, F32, True, False, 4, ref=True)
    assert G.rel_l2(a, b) <= 1e-6
    a, b = _both(256, 2048, 2048, F16, F32, False, False, 5, ref=True)
    assert G.rel_l2(a, b) <= 1e-6


def test_problem_beyond_the_fixed_array_is_rejected_cleanly():
    A = torch.zeros((128, 4096), device="cuda", dtype=torch.float16)
    B = torch.zeros((4096, 4096), device="cuda", dtype=torch.float16)
    C = torch.full((128, 4096), 3.0, device="cuda", dtype=torch.float16)
    rc = lib().nncv_b200_matmul_noalloc(G.p(A), G.p(B), G.p(C), 128, 4096, 4096, F16, F16, None, 0, G.stream_ptr())
    torch.cuda.synchronize()
    assert rc == 1                                   # NNCV_B200_EINVAL
    assert b"fixed scratch" in lib().nncv_b200_last_error()
    assert (C == 3.0).all()                          # nothing ran
    rc = lib().nncv_b200_matmul_noalloc(G.p(A), G.p(B), G.p(C), 128, 4096, 4096, F32, F32, None, 0, G.stream_ptr())
    assert rc == 1
