"""Generates the committed fixtures under tests/golden/.  Run where the nncv source tree is
available (its location comes from the environment variable NNCV_REFERENCE; a GPU box has no such
tree, so the tests read only the files this script wrote):

    NNCV_REFERENCE=<nncv source tree> python tests/golden/make_golden.py

  res18_constants.json   shapes of the constants of tests/Nets/Res18.mlir:12-110, in order
  kat0_two_params.bin    the SplitParams known-answer weights (tests/SplitParams/getParams.py:15-29)
                         written by the REFERENCE's own MemRefFlatArray::write (oracle/_ref)
  res18_fp32_n1_256.npz  logits of ResNet-18 fp32, N=1, 3x256x256 U[0,1) seed 0, from the oracle
                         (fp32 and fp64 accumulation) and from PyTorch CPU
  res18_fp32_n4_64.npz   same at N=4, 64x64 (small case)
  res50_fp32_n2_64.npz   ResNet-50, N=2, 64x64
  res18_from_mlir.plan   the layer plan nncv_b200.mlir_import reads out of tests/Nets/Res18.mlir
                         (tests/Nets/Res18-half.mlir, the f16 module, gives the same plan: asserted)
"""
import ctypes
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import binding as ob  # noqa: E402
from nncv_b200.split_params import random_input, random_state_dict, to_flat_array  # noqa: E402
import torch_ref  # noqa: E402

REF = os.environ.get("NNCV_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set NNCV_REFERENCE to the nncv source tree")


def constants():
    shapes = []
    with open(os.path.join(REF, "tests/Nets/Res18.mlir")) as f:
        for i, line in enumerate(f, 1):
            if 12 <= i <= 110:
                m = re.search(r"(%cst(?:_\d+)?) = arith.constant dense_resource<__elided__> : tensor<([0-9x]+)xf32>", line)
                assert m, line
                shapes.append([m.group(1), [int(v) for v in m.group(2).split("x")]])
    with open(os.path.join(HERE, "res18_constants.json"), "w") as f:
        json.dump(shapes, f)


def kat0():
    L = ob.ref_lib()
    assert L is not None, "build oracle/_ref first (make -C oracle)"
    w2 = np.zeros((1, 1, 5, 5), np.float32)
    for i in range(5):
        w2[0, 0, i, i] = 1
    w1 = np.zeros((1, 3, 3, 3), np.float32)
    w1[0, 0, 0, 0] = w1[0, 1, 1, 1] = w1[0, 2, 2, 2] = 1
    names = (ctypes.c_char_p * 2)(b"__constant_1x1x5x5xf32", b"__constant_1x3x3x3xf32")
    dims = (ctypes.c_size_t * 2)(4, 4)
    shapes = (ctypes.c_size_t * 16)(1, 1, 5, 5, 0, 0, 0, 0, 1, 3, 3, 3, 0, 0, 0, 0)
    data = (ctypes.c_void_p * 2)(w2.ctypes.data, w1.ctypes.data)
    rc = L.ref_flat_array_write(os.path.join(HERE, "kat0_two_params.bin").encode(), 2, names, dims, shapes, 4, data)
    assert rc == 0


def logits(depth, n, hw, name):
    sd = random_state_dict(depth, 0)
    blob = to_flat_array(depth, sd).blob()
    x = random_input(n, hw, hw, 0, "uniform")
    o32 = ob.resnet_forward(depth, x, blob, acc64=False)
    o64 = ob.resnet_forward(depth, x, blob, acc64=True)
    tr = torch_ref.resnet_forward(depth, x, sd)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    print(name, "oracle32 vs oracle64", rel(o32, o64), "torch vs oracle64", rel(tr, o64))
    np.savez_compressed(os.path.join(HERE, name), oracle_f32=o32, oracle_f64acc=o64, torch_cpu=tr)


def plans():
    from nncv_b200 import mlir_import
    mlir_import.import_mlir_file(os.path.join(REF, "tests/Nets/Res18.mlir")).write(os.path.join(HERE, "res18_from_mlir.plan"))
    half = mlir_import.import_mlir_file(os.path.join(REF, "tests/Nets/Res18-half.mlir"))
    assert half.to_text() == open(os.path.join(HERE, "res18_from_mlir.plan")).read()
    mlir_import.import_mlir_file(os.path.join(REF, "tests/Nets/MobileNetV3.mlir")).write(os.path.join(HERE, "mobilenetv3_from_mlir.plan"))


if __name__ == "__main__":
    if sys.argv[1:] == ["plans"]:
        plans()
        raise SystemExit(0)
    constants()
    kat0()
    logits(18, 1, 256, "res18_fp32_n1_256.npz")
    logits(18, 4, 64, "res18_fp32_n4_64.npz")
    logits(50, 2, 64, "res50_fp32_n2_64.npz")
    plans()
