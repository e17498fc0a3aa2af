"""GPU parity of the whole forward through `_mlir_ciface_forward` against the CPU oracle and
the committed golden logits."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import binding as ob  # noqa: E402
from nncv_b200 import runtime as rt  # noqa: E402
from nncv_b200._lib import BF16, F16, F32, NncvError  # noqa: E402
from nncv_b200.split_params import random_input, random_state_dict, to_flat_array, write_model_bin  # noqa: E402
import gpu_util as G  # noqa: E402


@pytest.fixture(autouse=True)
def _unload():
    yield
    rt.unload()


def test_resnet18_fp32_config0_matches_golden(tmp_path, golden_dir):
    """ResNet-18 fp32, 1x3x256x256 U[0,1) seed 0 (the reference's own CPU-runnable case):
    logits rel-L2 <= 1e-4 vs the oracle; weights arrive through a model.bin file."""
    path = str(tmp_path / "model.bin")
    write_model_bin(path, 18, 0, np.float32)
    rt.load("resnet18", path)
    x = random_input(1, 256, 256, 0, "uniform")
    out = np.full((1, 1000), np.nan, np.float32)
    rt.forward(out, x)
    gold = np.load(os.path.join(golden_dir, "res18_fp32_n1_256.npz"))
    assert G.rel_l2(out, gold["oracle_f64acc"]) <= 1e-4
    assert G.rel_l2(out, gold["torch_cpu"]) <= 1e-4
    assert out.argmax() == gold["oracle_f64acc"].argmax()


def test_resnet18_fp32_lazy_plan_from_params_descriptor():
    """No load call: the plan is built from the rank-1 params descriptor, like the reference's
    driver passes `params.get()` (examples/Res18/main.cpp:96)."""
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    x = random_input(4, 64, 64, 0, "uniform")
    out = np.zeros((4, 1000), np.float32)
    rt.forward(out, x, blob)
    ref = ob.resnet_forward(18, x, blob, acc64=True)
    assert G.rel_l2(out, ref) <= 1e-4


@pytest.mark.parametrize("compute", [F16, BF16])
def test_resnet18_half_vs_fp32_oracle(compute):
    """fp16/bf16 tensor-core path vs the fp32 oracle: rel-L2 <= 1e-2 and top-1 agreement >= 99.5 %."""
    n = 16
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    x = random_input(n, 224, 224, 1, "normal")
    rt.load_blob("resnet18", blob, compute)
    out = np.zeros((n, 1000), np.float32)
    rt.forward(out, x)
    ref = ob.resnet_forward(18, x, blob, acc64=False)
    assert G.rel_l2(out, ref) <= 1e-2
    assert (out.argmax(1) == ref.argmax(1)).mean() >= 0.995


def test_resnet18_fp16_params_and_io(tmp_path):
    """fp16 model.bin (the format nncv's -split-params cannot write itself): fp16 in, fp16 out."""
    path = str(tmp_path / "model_h.bin")
    write_model_bin(path, 18, 0, np.float16)
    rt.load("resnet18", path)
    n = 8
    x = random_input(n, 224, 224, 2, "normal").astype(np.float16)
    out = np.zeros((n, 1000), np.float16)
    rt.forward(out, x)
    sd = {k: v.astype(np.float16).astype(np.float32) for k, v in random_state_dict(18, 0).items()}
    ref = ob.resnet_forward(18, x.astype(np.float32), to_flat_array(18, sd).blob())
    assert G.rel_l2(out.astype(np.float32), ref) <= 1e-2
    assert (out.argmax(1) == ref.argmax(1)).mean() >= 0.995


def test_resnet50_fp32_and_fp16(golden_dir):
    sd = random_state_dict(50, 0)
    blob = to_flat_array(50, sd).blob()
    x = random_input(2, 64, 64, 0, "uniform")
    gold = np.load(os.path.join(golden_dir, "res50_fp32_n2_64.npz"))["oracle_f64acc"]
    rt.load_blob("resnet50", blob, F32)
    out = np.zeros((2, 1000), np.float32)
    rt.forward(out, x)
    assert G.rel_l2(out, gold) <= 1e-4
    rt.load_blob("resnet50", blob, F16)
    out16 = np.zeros((2, 1000), np.float32)
    rt.forward(out16, x)
    assert G.rel_l2(out16, gold) <= 1e-2


def test_device_resident_forward_and_batch_independence():
    """Device pointers in the descriptors; image i of a batch equals the same image run alone
    (the property batch sharding across GPUs relies on)."""
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    rt.load_blob("resnet18", blob, F16)
    x = random_input(6, 96, 96, 3, "normal")
    X = torch.from_numpy(x).cuda()
    out = torch.zeros((6, 1000), device="cuda")
    rt.forward(out, X)
    full = out.cpu().numpy()
    out2 = torch.zeros((2, 1000), device="cuda")
    rt.forward(out2, X[2:4].contiguous())
    assert np.array_equal(out2.cpu().numpy(), full[2:4])


def test_bad_descriptors_are_rejected_without_touching_dst():
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    rt.load_blob("resnet18", blob, F16)
    out = np.full((1, 1000), 7.0, np.float32)
    with pytest.raises(NncvError):
        rt.forward(out, np.zeros((1, 4, 64, 64), np.float32))          # 4 channels
    with pytest.raises(NncvError):
        rt.forward(np.zeros((2, 1000), np.float32), np.zeros((1, 3, 64, 64), np.float32))  # batch mismatch
    assert (out == 7.0).all()


@pytest.mark.parametrize("n", [128, 256])
def test_large_host_batch_is_split_and_matches_device_path(n):
    """Host batches of 128 or more run as two halves so that the second half's host->device copy
    overlaps the first half's forward; the logits must equal the unsplit device-resident forward."""
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    rt.load_blob("resnet18", blob, F16)
    x = random_input(n, 64, 64, 5, "normal")
    out_host = np.zeros((n, 1000), np.float32)
    rt.forward(out_host, x)
    X = torch.from_numpy(x).cuda()
    out_dev = torch.zeros((n, 1000), device="cuda")
    rt.forward(out_dev, X)
    assert G.rel_l2(out_host, out_dev.cpu().numpy()) <= 1e-6
    ref = ob.resnet_forward(18, x[:8], blob)
    assert G.rel_l2(out_host[:8], ref) <= 1e-2


@pytest.mark.parametrize("n,h,w", [(1, 256, 256), (3, 97, 131), (5, 224, 224), (2, 64, 600)])
def test_resnet18_fp16_odd_shapes(n, h, w):
    """Ragged maps, batch 1, a map wider than one stem tile, and one too wide for the fused stem (falls
    back to the unfused stem + pool kernels): fp16 path vs the fp32 oracle."""
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    rt.load_blob("resnet18", blob, F16)
    x = random_input(n, h, w, 11, "normal")
    out = np.zeros((n, 1000), np.float32)
    rt.forward(out, x)
    ref = ob.resnet_forward(18, x, blob)
    assert np.isfinite(out).all()
    assert G.rel_l2(out, ref) <= 1e-2
    assert (out.argmax(1) == ref.argmax(1)).all()


def test_logits_do_not_depend_on_the_tile_choice():
    """Which kernel or tile the first-call timing picks must not change the result: both tcgen05 conv
    kernels accumulate in the same order.  Compare two shapes of batch against each other instead of
    toggling the library-wide switch (it is read once at load)."""
    blob = to_flat_array(18, random_state_dict(18, 0)).blob()
    rt.load_blob("resnet18", blob, F16)
    x = random_input(40, 96, 96, 13, "normal")
    X = torch.from_numpy(x).cuda()
    full = torch.zeros((40, 1000), device="cuda")
    rt.forward(full, X)
    part = torch.zeros((7, 1000), device="cuda")
    rt.forward(part, X[30:37].contiguous())
    assert torch.equal(part, full[30:37])


@pytest.mark.gpu
def test_tuning_decisions_persist_across_processes(tmp_path):
    """NNCV_B200_TUNE_CACHE: the first process times its candidates and writes its decisions, the
    second one reads them back, launches far fewer kernels and returns the same logits."""
    import json
    import subprocess
    import sys
    cache = tmp_path / "tune.txt"
    prog = (
        "import sys, json, torch, numpy as np\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})\n"
        "from nncv_b200 import runtime as rt\n"
        "from nncv_b200._lib import F16\n"
        "from nncv_b200.split_params import random_input, random_state_dict, to_flat_array\n"
        "rt.load_blob('resnet18', to_flat_array(18, random_state_dict(18, 0)).blob(), F16)\n"
        "X = torch.from_numpy(random_input(8, 64, 64, 5, 'normal')).cuda()\n"
        "Y = torch.zeros((8, 1000), device='cuda')\n"
        "rt.forward(Y, X)\n"
        "print(json.dumps({'launches': rt.launch_count(), 'sum': float(Y.double().sum()), 'max': float(Y.max())}))\n"
    )
    env = dict(os.environ, NNCV_B200_TUNE_CACHE=str(cache))
    outs = []
    for _ in range(2):
        r = subprocess.run([sys.executable, "-c", prog], env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(json.loads(r.stdout.strip().splitlines()[-1]))
    lines = cache.read_text().splitlines()
    assert any(l.startswith("conv ") for l in lines)
    assert outs[1]["launches"] < outs[0]["launches"]
    assert outs[0]["sum"] == outs[1]["sum"] and outs[0]["max"] == outs[1]["max"]
