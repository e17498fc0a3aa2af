"""The failure path of the device side, exercised without a fault: a kernel whose bounded wait is
left to run out reports into the device status word and returns; the host maps the word to
NNCV_B200_ETIMEOUT, clears it, and the library keeps working."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import binding as ob  # noqa: E402
from nncv_b200 import runtime as rt  # noqa: E402
from nncv_b200._lib import F16, F32, lib  # noqa: E402
from nncv_b200.split_params import random_input, random_state_dict, to_flat_array  # noqa: E402
import gpu_util as G  # noqa: E402


def test_a_wait_that_runs_out_becomes_a_status_not_a_hang():
    L = lib()
    assert L.nncv_b200_device_status() == 0
    # an mbarrier nobody arrives on, limit 2^20 clocks (about half a millisecond)
    assert L.nncv_b200_selftest_wait_timeout(20, G.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert L.nncv_b200_device_status() == 6                      # NNCV_B200_ETIMEOUT
    msg = L.nncv_b200_last_error()
    assert b"bounded wait" in msg and b"code 4" in msg
    assert L.nncv_b200_device_status() == 0                      # read once, cleared
    # out-of-range limits are refused on the host
    assert L.nncv_b200_selftest_wait_timeout(40, G.stream_ptr()) == 1
    # the context is intact: a matmul and a forward still agree with the oracle
    g = np.random.default_rng(0)
    a = g.uniform(-1, 1, (256, 128)).astype(np.float32)
    b = g.uniform(-1, 1, (128, 192)).astype(np.float32)
    c, ar, br = G.matmul(a, b, F16, F32)
    assert G.rel_l2(c, ob.matmul(ar, br, acc64=True)) <= 1e-5
    assert L.nncv_b200_device_status() == 0


def test_forward_reports_a_pending_timeout_and_recovers():
    """_mlir_ciface_forward reads the status word itself: a time-out left by an earlier kernel of the
    stream fails that call with ETIMEOUT (dst may be written), and the next call is clean."""
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    rt.load_blob("resnet18", blob, F16)
    try:
        x = random_input(2, 64, 64, 0, "normal")
        out = np.zeros((2, 1000), np.float32)
        rt.forward(out, x)
        good = out.copy()
        assert lib().nncv_b200_selftest_wait_timeout(18, None) == 0
        torch.cuda.synchronize()
        with pytest.raises(Exception) as e:
            rt.forward(out, x)
        assert getattr(e.value, "code", None) == 6
        rt.forward(out, x)
        assert np.array_equal(out, good)
    finally:
        rt.unload()


def test_log_and_nvtx_switches(tmp_path):
    """NNCV_B200_LOG=1 reports the load, the activation arena and the tuning decisions on stderr; NNCV_B200_NVTX=1 wraps
    every plan node in an NVTX range (nothing listens here: the ranges must simply cost nothing and change nothing)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import numpy as np, sys\n"
        f"sys.path.insert(0, {root!r})\n"
        "from nncv_b200 import runtime as rt\n"
        "from nncv_b200._lib import F16\n"
        "from nncv_b200.split_params import random_input, random_state_dict, to_flat_array\n"
        "blob = to_flat_array(18, random_state_dict(18, 0), np.float16).blob()\n"
        "rt.load_blob('resnet18', blob, F16)\n"
        "x = random_input(2, 64, 64, 0, 'normal').astype(np.float16)\n"
        "y = np.zeros((2, 1000), np.float16)\n"
        "rt.forward(y, x)\n"
        "print('finite', bool(np.isfinite(y.astype(np.float32)).all()))\n")
    env = dict(os.environ, NNCV_B200_LOG="1", NNCV_B200_NVTX="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "finite True" in r.stdout
    assert "[nncv_b200] loaded resnet18" in r.stderr and "activation arena:" in r.stderr and "tuned conv" in r.stderr
