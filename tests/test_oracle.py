"""The CPU oracle against the reference's own known-answer fixtures and against PyTorch CPU."""
import json
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import binding as ob
from nncv_b200.netspec import conv_groups, conv_macs, tensor_order
from nncv_b200.split_params import random_input, random_state_dict, to_flat_array
import torch_ref


def rel(a, b):
    return float(np.linalg.norm(np.asarray(a, np.float64) - b) / np.linalg.norm(b))


def test_kat0_split_params_all_fifteen(golden_dir):
    """tests/SplitParams/data.mlir of the reference: all-ones 1x3x224x224 through the 3x3 tap-selecting
    conv and the 5x5 diagonal conv gives 1x1x218x218 of exactly 15 (weights read from the container
    the reference's own writer produced)."""
    from nncv_b200.memref import MemRefFlatArray
    arr = MemRefFlatArray.read(os.path.join(golden_dir, "kat0_two_params.bin"))
    assert [t.shape for t in arr.tensors] == [(1, 1, 5, 5), (1, 3, 3, 3)]
    y = ob.conv2d(ob.conv2d(np.ones((1, 3, 224, 224), np.float32), arr.tensors[1].data), arr.tensors[0].data)
    assert y.shape == (1, 1, 218, 218) and (y == 15.0).all()


def test_winograd_fixture_closed_form():
    """tests/ConvOptimization/conv2dNchwWinograd.mlir: NHWC 1x16x16x4, HWCF 3x3x4x16 splat 0.1, no padding:
    every output = 0.1 * sum of the 3x3x4 window (3.6 for an all-ones input)."""
    g = np.random.default_rng(0)
    x = g.standard_normal((1, 4, 16, 16)).astype(np.float32)
    w = np.full((16, 4, 3, 3), 0.1, np.float32)
    y = ob.conv2d(x, w)
    win = np.lib.stride_tricks.sliding_window_view(x[0], (3, 3), axis=(1, 2)).sum(axis=(0, 3, 4))
    np.testing.assert_allclose(y[0, 5], np.float32(0.1) * win, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ob.conv2d(np.ones_like(x), w), 3.6, rtol=1e-6)


def test_batchnorm_fixture_identity_stats():
    """tests/Nets/BatchNorm2d.mlir:7-8: gamma=1, beta=0, mean=0, var=1 -> y = x * rsqrt(1 + 1e-5f)."""
    x = np.random.default_rng(1).standard_normal((1, 3, 8, 8)).astype(np.float32)
    one, zero = np.ones(3, np.float32), np.zeros(3, np.float32)
    y = ob.batchnorm(x, one, zero, zero, one)
    rs = np.float32(1.0) / np.sqrt(np.float32(1.0) + np.float32(1e-5))
    np.testing.assert_array_equal(y, (x * rs) * np.float32(1.0) + np.float32(0.0))


def test_relu_passes_nan_like_unordered_gt():
    x = np.array([-1.0, 0.0, 2.0, np.nan, -0.0], np.float32)
    y = ob.relu(x)
    assert y[0] == 0 and y[1] == 0 and y[2] == 2 and np.isnan(y[3]) and y[4] == 0


def test_maxpool_fixture_shape_and_minus_inf_padding():
    """tests/Nets/Pool2DMax.mlir: 3x3 stride 3 no padding on 224 -> 74; ResNet's pool pads with -inf."""
    x = np.random.default_rng(2).standard_normal((1, 3, 224, 224)).astype(np.float32)
    y = ob.maxpool(x, 3, 3, 0)
    assert y.shape == (1, 3, 74, 74)
    np.testing.assert_array_equal(y, F.max_pool2d(torch.from_numpy(x), 3, 3).numpy())
    neg = -np.abs(x) - 1
    np.testing.assert_array_equal(ob.maxpool(neg, 3, 2, 1), F.max_pool2d(torch.from_numpy(neg), 3, 2, 1).numpy())


@pytest.mark.parametrize("stride,pad,k", [(1, 1, 3), (2, 1, 3), (2, 0, 1), (2, 3, 7)])
def test_conv_matches_torch(stride, pad, k):
    g = np.random.default_rng(k + stride)
    x = g.standard_normal((2, 5, 19, 23)).astype(np.float32)
    w = g.standard_normal((7, 5, k, k)).astype(np.float32)
    ref = F.conv2d(torch.from_numpy(x), torch.from_numpy(w), stride=stride, padding=pad).numpy()
    assert rel(ob.conv2d(x, w, stride, pad), ref) < 2e-6
    assert rel(ob.conv2d(x, w, stride, pad, acc64=True), ref) < 2e-6


def test_matmul_bias_relu_and_avgpool():
    g = np.random.default_rng(3)
    a, b, bias = g.standard_normal((33, 47)), g.standard_normal((47, 29)), g.standard_normal(29)
    ref = np.maximum(a @ b + bias, 0)
    assert rel(ob.matmul(a, b, bias, True, acc64=True), ref) < 1e-6
    x = g.standard_normal((2, 6, 7, 7)).astype(np.float32)
    assert rel(ob.avgpool_global(x), x.mean(axis=(2, 3))) < 1e-6


@pytest.mark.parametrize("name,depth,n,hw", [("res18_fp32_n1_256.npz", 18, 1, 256), ("res18_fp32_n4_64.npz", 18, 4, 64),
                                             ("res50_fp32_n2_64.npz", 50, 2, 64)])
def test_network_matches_committed_golden_logits(golden_dir, name, depth, n, hw):
    """The fixtures hold the oracle's logits and PyTorch CPU's for the same seeded tensors; the live
    oracle must reproduce its own file bit for bit and stay within 1e-5 of the PyTorch logits."""
    gold = np.load(os.path.join(golden_dir, name))
    blob = to_flat_array(depth, random_state_dict(depth, 0)).blob()
    x = random_input(n, hw, hw, 0, "uniform")
    out = ob.resnet_forward(depth, x, blob)
    assert rel(out, gold["oracle_f32"]) < 1e-6
    assert rel(out, gold["torch_cpu"]) < 1e-5
    assert rel(ob.resnet_forward(depth, x, blob, acc64=True), gold["oracle_f64acc"]) < 1e-6


def test_network_matches_pytorch_live():
    sd = random_state_dict(18, 7)
    x = random_input(2, 96, 96, 7, "normal")
    out = ob.resnet_forward(18, x, to_flat_array(18, sd).blob())
    assert rel(out, torch_ref.resnet_forward(18, x, sd)) < 1e-5


def test_tensor_order_mirrors_reference_constants(golden_dir):
    """Shapes of the constants of tests/Nets/Res18.mlir:12-110 (extracted by tests/golden/make_golden.py).
    torch-mlir dedups equal constants, so the reference file has 99; ours keeps every tensor (102).
    Removing our extra batch-norm vectors must give the reference's sequence of shapes."""
    with open(os.path.join(golden_dir, "res18_constants.json")) as f:
        ref = [tuple(s) for _, s in json.load(f)]
    ours = [s for _, s in tensor_order(18)]
    assert len(ours) == 102 and len(ref) == 99
    it = iter(ours)
    for s in ref:           # ref must be a subsequence of ours
        for o in it:
            if o == s:
                break
        else:
            pytest.fail(f"reference constant of shape {s} has no counterpart in order")
    assert [s for s in ours if len(s) == 4] == [s for s in ref if len(s) == 4]
    assert ours[0] == (1000,) and ours[1] == (1000, 512)


def test_mac_counts():
    assert conv_macs(18, 224, 224) == 1_814_073_344
    assert conv_macs(18, 256, 256) == 2_369_245_184
    assert conv_macs(50, 224, 224) == 4_089_184_256
    assert len(conv_groups(18)) == 20 and len(conv_groups(50)) == 53
    assert ob.oracle().nncv_oracle_resnet_param_count(18) == sum(int(np.prod(s)) for _, s in tensor_order(18))
    assert ob.oracle().nncv_oracle_resnet_param_count(50) == sum(int(np.prod(s)) for _, s in tensor_order(50))


# ---- operators of the mobile / detection fixtures (MobileNetV3.mlir, Yolov5s.mlir) ------------
@pytest.mark.parametrize("stride,pad,k", [(1, 1, 3), (2, 1, 3), (2, 2, 5), (1, 0, 1)])
def test_depthwise_conv_matches_torch(stride, pad, k):
    g = np.random.default_rng(k * 10 + stride)
    x = g.standard_normal((2, 24, 13, 17)).astype(np.float32)
    w = g.standard_normal((24, k, k)).astype(np.float32)
    ref = F.conv2d(torch.from_numpy(x), torch.from_numpy(w)[:, None], stride=stride, padding=pad, groups=24).numpy()
    assert rel(ob.depthwise_conv2d(x, w, stride, pad), ref) < 2e-6
    assert rel(ob.depthwise_conv2d(x, w, stride, pad, acc64=True), ref) < 2e-6


def test_activations_match_torch_and_pass_nan():
    x = np.random.default_rng(3).standard_normal(4096).astype(np.float32) * 4
    t = torch.from_numpy(x)
    for kind, fn in (("hard_sigmoid", F.hardsigmoid), ("hard_swish", F.hardswish), ("sigmoid", torch.sigmoid), ("silu", F.silu),
                     ("relu", F.relu)):
        assert np.abs(ob.activation(x, kind) - fn(t).numpy()).max() < 2e-6, kind
    edge = np.array([-3.0, 3.0, -7.0, 9.0, np.nan], np.float32)
    hs = ob.activation(edge, "hard_sigmoid")
    assert hs[0] == 0 and hs[1] == 1 and hs[2] == 0 and hs[3] == 1 and np.isnan(hs[4])   # olt/ogt selects keep a NaN
    assert np.isnan(ob.activation(edge, "silu")[4])


def test_se_gate_concat_upsample_match_torch():
    g = np.random.default_rng(4)
    p = g.standard_normal((3, 16)).astype(np.float32)
    w1, b1 = g.standard_normal((8, 16)).astype(np.float32), g.standard_normal(8).astype(np.float32)
    w2, b2 = g.standard_normal((16, 8)).astype(np.float32), g.standard_normal(16).astype(np.float32)
    tp = torch.from_numpy(p)
    ref = F.hardsigmoid(F.linear(F.relu(F.linear(tp, torch.from_numpy(w1), torch.from_numpy(b1))), torch.from_numpy(w2),
                                 torch.from_numpy(b2))).numpy()
    assert np.abs(ob.se_gate(p, w1, b1, w2, b2) - ref).max() < 1e-5
    x = g.standard_normal((2, 8, 5, 7)).astype(np.float32)
    y = g.standard_normal((2, 16, 5, 7)).astype(np.float32)
    assert np.array_equal(ob.concat_channels([x, y, x]), np.concatenate([x, y, x], 1))
    assert np.array_equal(ob.upsample2x(x), F.interpolate(torch.from_numpy(x), scale_factor=2, mode="nearest").numpy())
