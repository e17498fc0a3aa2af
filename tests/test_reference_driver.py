"""The drop-in boundary exercised by the reference's own caller: nncv's examples/Res18/main.cpp,
compiled UNCHANGED (with nncv's src/libnncv/DataType.cpp and its vendored stb_image) and linked
against libnncv_b200.so instead of a compiled model object + libnncv_rt (oracle/Makefile builds it
into oracle/_ref/ where the nncv tree is present; the binary travels with the repository's other
built files).  The driver reads model.bin with nncv's MemRefFlatArray, decodes cat_256x256.jpg,
fills the two MemRefDescriptors, calls _mlir_ciface_forward(&dst, &src, params.get()) and prints
the arg-max class."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

from nncv_b200.split_params import write_model_bin

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFDIR = os.path.join(ROOT, "oracle", "_ref")
DRIVER = os.path.join(REFDIR, "res18_driver")
IMAGE = os.path.join(REFDIR, "cat_256x256.jpg")
STB = os.path.join(REFDIR, "libnncv_stb_ref.so")
have = all(os.path.exists(p) for p in (DRIVER, IMAGE, STB))


def run_driver(tmp_path):
    write_model_bin(str(tmp_path / "model.bin"), 18, 0, np.float32)   # what `nncv-c -split-params` would leave beside the object
    shutil.copy(IMAGE, tmp_path / "cat_256x256.jpg")
    r = subprocess.run([DRIVER], cwd=tmp_path, capture_output=True, text=True, timeout=600)
    return r


@pytest.mark.skipif(not have, reason="oracle/_ref/res18_driver has not been built (needs the nncv tree)")
def test_driver_links_and_runs_without_a_gpu_and_gets_no_logits(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("checks the no-GPU behaviour")
    r = run_driver(tmp_path)
    assert r.returncode == 0, r.stderr[-500:]
    lines = r.stdout.split()
    assert lines[:3] == ["256", "256", "3"]        # the driver decoded the image and got as far as the call


@pytest.mark.gpu
@pytest.mark.skipif(not have, reason="oracle/_ref/res18_driver has not been built (needs the nncv tree)")
def test_unchanged_reference_driver_gets_the_oracle_argmax(tmp_path):
    from oracle import binding as ob
    from nncv_b200.split_params import random_state_dict, to_flat_array
    r = run_driver(tmp_path)
    assert r.returncode == 0, r.stderr[-500:]
    out = r.stdout.split()
    assert out[:3] == ["256", "256", "3"] and out[3] == "Time:"
    idx = int(out[-1])
    # the same pixels through the oracle: decode with the driver's decoder, repeat its preprocessing
    L = ctypes.CDLL(STB)
    buf = np.zeros(256 * 256 * 3, np.uint8)
    w, h, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    assert L.ref_decode_image(IMAGE.encode(), buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(buf.size), ctypes.byref(w),
                              ctypes.byref(h), ctypes.byref(c)) == 0
    assert (w.value, h.value, c.value) == (256, 256, 3)
    px = buf.reshape(256, 256, 3).astype(np.float32) / np.float32(255.0)
    x = px.transpose(2, 0, 1)[None].copy()
    mean = np.array([0.485, 0.456, 0.406], np.float32)[None, :, None, None]
    std = np.array([0.229, 0.224, 0.225], np.float32)[None, :, None, None]
    x = (x - mean) / std
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    ref = ob.resnet_forward(18, x, blob, acc64=True)
    assert idx == int(ref[0].argmax())
    top2 = np.sort(ref[0])[-2:]
    assert top2[1] - top2[0] > 1e-3 * abs(top2[1])     # the winner is not a coin toss at fp32 accuracy
