"""Forwards driven by imported layer plans, through `_mlir_ciface_forward`, against the CPU oracle:
the plan read from nncv's own ResNet-18 module (committed golden text) with a model.bin laid out in
that module's constant order, and a small non-ResNet module written in the same linalg style."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import binding as ob  # noqa: E402
from nncv_b200 import mlir_import as mi  # noqa: E402
from nncv_b200 import runtime as rt  # noqa: E402
from nncv_b200._lib import BF16, F16, F32, NncvError, lib  # noqa: E402
from nncv_b200.memref import MemRefFlatArray  # noqa: E402
from nncv_b200.split_params import random_input  # noqa: E402
import gpu_util as G  # noqa: E402
import plan_util as P  # noqa: E402


@pytest.fixture(autouse=True)
def _unload():
    yield
    rt.unload()
    assert lib().nncv_b200_device_status() == 0, lib().nncv_b200_last_error()


def write_model_bin(path, nodes, blob, dtype=np.float32):
    arr = MemRefFlatArray(np.dtype(dtype).itemsize)
    for (name, shape), (off, _, _) in zip(P.blob_indexers(nodes), P.plan_tensors(nodes)):
        arr.add(name, blob[off:off + int(np.prod(shape))].reshape(shape).astype(dtype))
    arr.write(path)


@pytest.mark.parametrize("compute", [F32, F16])
def test_resnet18_from_the_reference_module(tmp_path, golden_dir, compute):
    """Plan = what the importer read from tests/Nets/Res18.mlir (99 tensor constants: 102 minus three shared batch-norm
    vectors); weights = a container with exactly those 99 tensors in module order."""
    plan_path = os.path.join(golden_dir, "res18_from_mlir.plan")
    total, out, nodes = P.parse_plan_text(open(plan_path).read())
    blob = P.random_blob(total, nodes, seed=3)
    assert len(P.plan_tensors(nodes)) == 99
    bin_path = str(tmp_path / "model.bin")
    write_model_bin(bin_path, nodes, blob)
    rt.load(plan_path, bin_path, compute)
    n, hw = (2, 256) if compute == F32 else (8, 224)
    x = random_input(n, hw, hw, 7, "uniform" if compute == F32 else "normal")
    got = np.zeros((n, 1000), np.float32)
    rt.forward(got, x)
    ref = P.run_plan_cpu(nodes, blob, x, ob, acc64=compute == F32)
    assert G.rel_l2(got, ref) <= (1e-4 if compute == F32 else 1e-2)
    assert (got.argmax(1) == ref.argmax(1)).all()


@pytest.mark.parametrize("compute", [F32, F16])
def test_small_non_resnet_module(tmp_path, compute):
    text = mi.import_mlir(P.small_net_mlir()).to_text()
    total, out, nodes = P.parse_plan_text(text)
    blob = P.random_blob(total, nodes, seed=5)
    bin_path = str(tmp_path / "small.bin")
    write_model_bin(bin_path, nodes, blob)
    rt.load("plan:" + text, bin_path, compute)
    for n, h, w in ((3, 40, 56), (1, 33, 47), (1, 96, 112)):   # not tied to the static shape; the last pools a map of 672 pixels
        x = random_input(n, h, w, 9, "normal")
        got = np.zeros((n, out), np.float32)
        rt.forward(got, x)
        ref = P.run_plan_cpu(nodes, blob, x, ob, acc64=True)
        assert got.shape == (n, 10) and np.isfinite(got).all()
        assert G.rel_l2(got, ref) <= (1e-4 if compute == F32 else 1e-2)


@pytest.mark.parametrize("compute", [F32, F16])
def test_small_mobile_module(tmp_path, compute):
    """conv + hard-swish, depthwise conv + BN + ReLU / hard-swish, squeeze-and-excitation (scaling in place), a residual
    add without activation and an FC + hard-swish -> FC head, imported from linalg text in the MobileNetV3 fixture's spellings."""
    text = mi.import_mlir(P.small_mobile_mlir()).to_text()
    total, out, nodes = P.parse_plan_text(text)
    blob = P.random_blob(total, nodes, seed=11)
    bin_path = str(tmp_path / "mobile.bin")
    write_model_bin(bin_path, nodes, blob)
    rt.load("plan:" + text, bin_path, compute)
    for n, h, w in ((2, 64, 48), (3, 97, 131), (1, 160, 192)):   # the last one pools a map of 1920 pixels in its first SE block
        x = random_input(n, h, w, 13, "normal")
        got = np.zeros((n, out), np.float32)
        rt.forward(got, x)
        ref = P.run_plan_cpu(nodes, blob, x, ob, acc64=True)
        assert got.shape == (n, 10) and np.isfinite(got).all()
        assert G.rel_l2(got, ref) <= (1e-4 if compute == F32 else 1e-2)


@pytest.mark.parametrize("compute,n,hw", [(F32, 1, (128, 128)), (F16, 4, (224, 224)), (F16, 2, (256, 256)), (F16, 1, (225, 193)),
                                          (F32, 3, (64, 96)), (F16, 1, (33, 35)), (BF16, 2, (128, 128))])
def test_mobilenetv3_from_the_reference_module(tmp_path, golden_dir, compute, n, hw):
    """Plan = what the importer read from tests/Nets/MobileNetV3.mlir (210 tensor constants, 46 nodes); weights = a
    container with exactly those tensors in module order, seeded random values."""
    plan_path = os.path.join(golden_dir, "mobilenetv3_from_mlir.plan")
    total, out, nodes = P.parse_plan_text(open(plan_path).read())
    blob = P.random_blob(total, nodes, seed=4)
    bin_path = str(tmp_path / "model.bin")
    write_model_bin(bin_path, nodes, blob)
    rt.load(plan_path, bin_path, compute)
    x = random_input(n, hw[0], hw[1], 5, "normal")
    got = np.zeros((n, 1000), np.float32)
    rt.forward(got, x)
    ref = P.run_plan_cpu(nodes, blob, x, ob, acc64=compute == F32)
    assert np.isfinite(got).all()
    # bf16 (8 mantissa bits) through 46 layers measures 1e-2 .. 3e-2 depending on the seed; fp16 1e-3 .. 2e-3; fp32 1e-6
    assert G.rel_l2(got, ref) <= {F32: 1e-4, F16: 1e-2, BF16: 5e-2}[compute]
    assert (got.argmax(1) == ref.argmax(1)).all()


def test_weights_that_do_not_match_the_plan_are_refused(tmp_path):
    text = mi.import_mlir(P.small_net_mlir()).to_text()
    total, out, nodes = P.parse_plan_text(text)
    blob = P.random_blob(total, nodes, seed=5)
    # a container with one tensor of the right total size: offsets do not fall on tensor boundaries
    arr = MemRefFlatArray(4)
    arr.add("everything", blob)
    path = str(tmp_path / "one.bin")
    arr.write(path)
    with pytest.raises(NncvError, match="is not a tensor of"):
        rt.load("plan:" + text, path, F32)
    with pytest.raises(NncvError):
        rt.load_blob("plan:" + text, blob[:-1], F32)


def test_activation_arena_is_smaller_than_private_buffers_and_survives_shape_changes():
    import ctypes
    from nncv_b200.split_params import random_state_dict, to_flat_array
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    rt.load_blob("resnet18", blob, F16)
    outs = {}
    for n, hw in ((4, 96), (2, 160), (4, 96)):
        x = random_input(n, hw, hw, 21, "normal")
        o = np.zeros((n, 1000), np.float32)
        rt.forward(o, x)
        a, u = ctypes.c_size_t(), ctypes.c_size_t()
        assert lib().nncv_b200_activation_bytes(ctypes.byref(a), ctypes.byref(u)) == 0
        assert 0 < a.value <= 0.8 * u.value        # three or four live tensors per stage instead of five
        if (n, hw) in outs:
            assert np.array_equal(outs[(n, hw)], o)   # re-planned arena, same logits bit for bit
        outs[(n, hw)] = o
        assert G.rel_l2(o, ob.resnet_forward(18, x, blob)) <= 1e-2
