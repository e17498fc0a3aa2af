"""The C-ABI library loads and exports exactly what include/nncv_b200.h declares; without a GPU every
compute entry point fails loudly (there is no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from nncv_b200 import _lib
from nncv_b200 import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "nncv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)   # preprocessor lines
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", text)
    return sorted(set(n for n in names if n.startswith(("nncv_", "_mlir_ciface_"))))


def test_header_and_library_agree():
    declared = declared_functions()
    assert "_mlir_ciface_forward" in declared and "nncv_b200_load" in declared
    L = _lib.lib()
    missing = [n for n in declared if not hasattr(L, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert sorted(_lib.EXPORTS) == declared, "nncv_b200/_lib.py EXPORTS is out of step with the header"


def test_library_does_not_link_the_oracle():
    out = os.popen(f"ldd {_lib.LIB_PATH}").read()
    assert "oracle" not in out and "nncv_rt_ref" not in out


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_gpu_means_loud_failure_not_cpu_fallback():
    L = _lib.lib()
    a = np.zeros((8, 8), np.float16)
    rc = L.nncv_b200_matmul(a.ctypes.data, a.ctypes.data, a.ctypes.data, 8, 8, 8, _lib.F16, _lib.F16, None, 0, None)
    assert rc == 3 and b"no CPU fallback" in L.nncv_b200_last_error()   # NNCV_B200_ENODEVICE
    with pytest.raises(_lib.NncvError) as e:
        rt.load_blob("resnet18", np.zeros(11699112, np.float32))
    assert e.value.code == 3
    out = np.full((1, 1000), 5.0, np.float32)
    with pytest.raises(_lib.NncvError):
        rt.forward(out, np.zeros((1, 3, 64, 64), np.float32), np.zeros(11699112, np.float32))
    assert (out == 5.0).all()
    # the newer entry points fail the same way: plans cannot even be created without a device
    w = np.zeros((128, 64, 3, 3), np.float32)
    assert not L.nncv_b200_conv_create(w.ctypes.data, _lib.F32, 128, 64, 3, 3, 2, 1, _lib.F16, 0)
    assert L.nncv_b200_last_status() == 3
    rc = L.nncv_b200_conv_run_fused(None, None, None, None, None, 1, 8, 8, None, None, None, None, 0, None)
    assert rc != 0
    rc = L.nncv_b200_stem_pool(a.ctypes.data, _lib.F16, a.ctypes.data, _lib.F32, None, None, a.ctypes.data, _lib.F16,
                               1, 8, 8, None)
    assert rc == 3
    assert L.nncv_b200_stem_variant(-1) == 0   # no stem launch has happened
    # the operators added for the mobile / detection fixtures, the status query and the wait self-test
    assert L.nncv_b200_depthwise_conv_nhwc(a.ctypes.data, a.ctypes.data, _lib.F32, None, None, a.ctypes.data, _lib.F16, 1, 8, 8, 8,
                                           3, 3, 1, 1, 0, None) == 3
    assert L.nncv_b200_activation(a.ctypes.data, a.ctypes.data, _lib.F16, 64, 1, None) == 3
    assert L.nncv_b200_upsample2x_nhwc(a.ctypes.data, a.ctypes.data, _lib.F16, 1, 2, 2, 8, None) == 3
    assert L.nncv_b200_device_status() == 3
    assert L.nncv_b200_selftest_wait_timeout(10, None) == 3
    # a plan loads nothing without a device either, but it is still parsed and checked on the host
    assert L.nncv_b200_plan_check(b"resnet18", None, None, None) == 0
    with pytest.raises(_lib.NncvError) as e2:
        rt.load_blob("plan:nncv_b200_plan 1\nparams 10 out 2\n", np.zeros(10, np.float32))
    assert e2.value.code == 1


def test_missing_library_raises(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libnncv_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()
