"""GPU parity of the single kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import binding as ob  # noqa: E402
from nncv_b200._lib import BF16, F16, F32, check, lib  # noqa: E402
import gpu_util as G  # noqa: E402

TOL_16 = 2e-3   # fp16/bf16 operands, fp32 accumulate, vs the fp64-accumulated oracle on the same rounded inputs
TOL_32 = 1e-5


def _rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (256, 128, 256), (512, 512, 512), (100, 1000, 72),
                                   (1, 8, 8), (300, 200, 1024), (1024, 1024, 1024)])
@pytest.mark.parametrize("ab", [F16, BF16])
def test_matmul_tcgen05(m, n, k, ab):
    r = _rng(m * 7 + n * 3 + k)
    a = r.uniform(-1, 1, (m, k)).astype(np.float32)
    b = r.uniform(-1, 1, (k, n)).astype(np.float32)
    c, ar, br = G.matmul(a, b, ab, F32)
    ref = ob.matmul(ar, br, acc64=True)
    assert np.isfinite(c).all()
    assert G.rel_l2(c, ref) <= 1e-5  # same rounded inputs, fp32 accumulate: only summation order differs


@pytest.mark.parametrize("c_dt", ["same", "f32"])
def test_matmul_bias_relu(c_dt):
    r = _rng(5)
    m, n, k = 384, 320, 192
    a = r.uniform(-1, 1, (m, k)).astype(np.float32)
    b = r.uniform(-1, 1, (k, n)).astype(np.float32)
    bias = r.standard_normal(n).astype(np.float32)
    c, ar, br = G.matmul(a, b, F16, F16 if c_dt == "same" else F32, bias, True)
    ref = ob.matmul(ar, br, bias, True, acc64=True)
    assert (c >= 0).all()
    assert G.rel_l2(c, ref) <= (TOL_16 if c_dt == "same" else 1e-5)


def test_matmul_f32_simt():
    r = _rng(6)
    m, n, k = 200, 136, 260
    a = r.uniform(-1, 1, (m, k)).astype(np.float32)
    b = r.uniform(-1, 1, (k, n)).astype(np.float32)
    bias = r.standard_normal(n).astype(np.float32)
    c, _, _ = G.matmul(a, b, F32, F32, bias, True)
    assert G.rel_l2(c, ob.matmul(a, b, bias, True, acc64=True)) <= TOL_32


CONV_CASES = [
    # n, c, h, w, k, r, stride, pad
    (2, 64, 16, 16, 64, 3, 1, 1),
    (2, 64, 16, 16, 128, 3, 2, 1),
    (2, 64, 16, 16, 128, 1, 2, 0),
    (2, 3, 32, 32, 64, 7, 2, 3),
    (1, 128, 7, 7, 256, 3, 1, 1),
    (3, 16, 9, 11, 24, 3, 1, 1),     # ragged everything
    (1, 256, 14, 14, 512, 1, 1, 0),
    (1, 512, 7, 7, 512, 3, 1, 1),
    (3, 64, 56, 56, 128, 3, 2, 1),   # ResNet-18 layer2.0.conv1 shape
    (3, 64, 56, 56, 128, 1, 2, 0),   # and its downsample conv
    (5, 256, 14, 14, 512, 3, 2, 1),  # layer4.0.conv1: two images per M tile
    (2, 128, 30, 50, 64, 1, 1, 0),   # ragged 1x1
]


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("dtype,algo", [(F16, 0), (F16, 3), (BF16, 0), (F32, 0)])
def test_conv_epilogue(case, dtype, algo):
    """algo 0: TMA-fed kernel where C % 64 == 0, gather kernel otherwise; algo 3: always the gather kernel."""
    n, c, h, w, k, r, stride, pad = case
    g = _rng(sum(case))
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((k, c, r, r)) * np.sqrt(2.0 / (c * r * r))).astype(np.float32)
    scale = g.uniform(0.5, 1.5, k).astype(np.float32)
    shift = (g.standard_normal(k) * 0.1).astype(np.float32)
    oh, ow = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    res = g.standard_normal((n, k, oh, ow)).astype(np.float32)
    conv = G.Conv(wt, stride, pad, dtype, algo)
    try:
        y, xr = conv.run(x, scale, shift, res, True)
    finally:
        conv.close()
    if dtype == F32:
        wr, rr = wt, res
    else:
        tdt = G.TORCH_DT[dtype]
        wr = torch.from_numpy(wt).to(tdt).float().numpy()
        rr = torch.from_numpy(res).to(tdt).float().numpy()
    ref = ob.conv2d(xr, wr, stride, pad, acc64=True) * scale[None, :, None, None] + shift[None, :, None, None] + rr
    ref = np.where(ref > 0, ref, 0)
    assert y.shape == ref.shape and np.isfinite(y).all()
    tol = TOL_32 if dtype == F32 else (TOL_16 if dtype == F16 else 8e-3)
    assert G.rel_l2(y, ref) <= tol


SV_CASES = [
    # n, c, h, w, k, (bn, mt, resident) or None for the built-in choice
    (1, 64, 8, 8, 64, (64, 1, 1)),
    (2, 64, 56, 56, 64, (64, 2, 1)),
    (2, 64, 56, 56, 64, None),
    (2, 128, 28, 28, 128, (64, 1, 1)),
    (2, 128, 28, 28, 128, (128, 2, 0)),
    (3, 256, 14, 14, 256, (128, 4, 0)),
    (3, 256, 14, 14, 256, (256, 2, 0)),
    (3, 256, 14, 14, 256, (64, 1, 0)),
    (5, 512, 7, 7, 512, None),
    (3, 256, 14, 14, 256, (256, 1, 2)),   # CTA-pair kernel (tcgen05.mma.cta_group::2)
    (5, 512, 7, 7, 512, (256, 1, 2)),
    (9, 128, 28, 28, 256, (256, 1, 2)),
    (1, 64, 8, 8, 256, (256, 1, 2)),
    (3, 64, 56, 56, 64, (64, 1, 2)),      # pair kernel, N = 64, weights resident
    (4, 128, 28, 28, 128, (128, 1, 2)),   # N = 128, weights resident
    (2, 64, 17, 23, 128, (64, 1, 2)),     # two Kout tiles of 64, streamed weights
    (5, 256, 14, 14, 256, (128, 1, 2)),
    (7, 256, 14, 14, 256, (128, 2, 2)),     # two sub-tiles of 256 slots per item, halo tile in two TMA boxes
    (9, 256, 14, 14, 256, (256, 2, 2)),     # 512 accumulator columns: one buffer, MMAs wait for the epilogue
    (11, 512, 7, 7, 512, (128, 4, 2)),      # four sub-tiles, single buffer, two Kout tiles
    (60, 256, 14, 14, 256, (256, 2, 3)),
    (3, 64, 56, 56, 64, (64, 4, 2)),
    (40, 128, 28, 28, 256, (128, 2, 3)),
    (100, 256, 14, 14, 256, (256, 1, 3)),   # 88 items on 74 pairs: the 14 of the last round run as 4 column slices each
    (84, 128, 14, 14, 256, (128, 1, 3)),    # 148 items: two full rounds, nothing to slice
    (90, 128, 14, 14, 256, (128, 1, 3)),    # 160 items: the last 12 run as two 64-column halves each
    (2, 64, 17, 23, 128, None),      # ragged map, Kout != C
    (1, 192, 5, 3, 64, None),
]


@pytest.mark.parametrize("case", SV_CASES)
@pytest.mark.parametrize("dtype,res", [(F16, True), (F16, False), (BF16, True)])
def test_conv3x3_shifted_view(case, dtype, res):
    """3x3 stride-1 pad-1 kernel whose taps are shifted views of one halo tile (algo 2), every
    tile configuration, against the fp64-accumulated oracle on the same rounded operands."""
    n, c, h, w, k, cfg = case
    g = _rng(n + c + h + w + k)
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((k, c, 3, 3)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    scale = g.uniform(0.5, 1.5, k).astype(np.float32)
    shift = (g.standard_normal(k) * 0.1).astype(np.float32)
    rs = g.standard_normal((n, k, h, w)).astype(np.float32) if res else None
    conv = G.Conv(wt, 1, 1, dtype, algo=2)
    try:
        if cfg:
            check(lib().nncv_b200_conv_set_tile(conv.h, *cfg))
        y, xr = conv.run(x, scale, shift, rs, True)
    finally:
        conv.close()
    tdt = G.TORCH_DT[dtype]
    wr = torch.from_numpy(wt).to(tdt).float().numpy()
    ref = ob.conv2d(xr, wr, 1, 1, acc64=True) * scale[None, :, None, None] + shift[None, :, None, None]
    if res:
        ref = ref + torch.from_numpy(rs).to(tdt).float().numpy()
    ref = np.where(ref > 0, ref, 0)
    assert np.isfinite(y).all()
    assert G.rel_l2(y, ref) <= (TOL_16 if dtype == F16 else 8e-3)


@pytest.mark.parametrize("case", [(2, 64, 16, 16, 64), (1, 64, 17, 23, 128), (3, 128, 7, 7, 64), (2, 256, 14, 14, 256)])
@pytest.mark.parametrize("dtype,res", [(F16, True), (F16, False), (BF16, False)])
def test_conv3x3_winograd_f2x2(case, dtype, res):
    """Winograd F(2x2,3x3) in three stages (algo 1), odd map sizes included; V is rounded to 16 bits
    between the stages, hence the wider tolerance than for the direct kernels."""
    n, c, h, w, k = case
    g = _rng(3 * n + c + h + w + k)
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((k, c, 3, 3)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    scale = g.uniform(0.5, 1.5, k).astype(np.float32)
    shift = (g.standard_normal(k) * 0.1).astype(np.float32)
    rs = g.standard_normal((n, k, h, w)).astype(np.float32) if res else None
    conv = G.Conv(wt, 1, 1, dtype, algo=1)
    try:
        y, xr = conv.run(x, scale, shift, rs, True)
    finally:
        conv.close()
    tdt = G.TORCH_DT[dtype]
    ref = ob.conv2d(xr, wt, 1, 1, acc64=True) * scale[None, :, None, None] + shift[None, :, None, None]
    if res:
        ref = ref + torch.from_numpy(rs).to(tdt).float().numpy()
    ref = np.where(ref > 0, ref, 0)
    assert np.isfinite(y).all()
    assert G.rel_l2(y, ref) <= (5e-3 if dtype == F16 else 3e-2)


def test_winograd_fixture_through_winograd_kernel():
    """The reference's Winograd fixture (conv2dNchwWinograd.mlir: filter splat 0.1) padded to 64 channels:
    all-ones input, interior outputs = 0.1 * 9 * 64."""
    x = np.ones((1, 64, 16, 16), np.float32)
    w = np.full((64, 64, 3, 3), 0.1, np.float32)
    conv = G.Conv(w, 1, 1, F16, algo=1)
    try:
        y, _ = conv.run(x)
    finally:
        conv.close()
    np.testing.assert_allclose(y[:, :, 1:-1, 1:-1], 0.1 * 9 * 64, rtol=2e-3)


def test_conv3x3_shifted_view_matches_gather_kernel():
    """The two tcgen05 kernels agree on the same layer up to the order of the fp32 sums."""
    g = _rng(77)
    x = g.standard_normal((4, 128, 28, 28)).astype(np.float32)
    wt = (g.standard_normal((128, 128, 3, 3)) * np.sqrt(2.0 / (9 * 128))).astype(np.float32)
    a, b = G.Conv(wt, 1, 1, F16, algo=0), G.Conv(wt, 1, 1, F16, algo=2)
    try:
        ya, _ = a.run(x)
        yb, _ = b.run(x)
    finally:
        a.close()
        b.close()
    assert G.rel_l2(ya, yb) <= 5e-4


@pytest.mark.parametrize("dtype", [F16, F32])
def test_conv_kat0_split_params(dtype, golden_dir):
    """tests/SplitParams/data.mlir of the reference: all-ones input -> every output is 15."""
    from nncv_b200.memref import MemRefFlatArray
    arr = MemRefFlatArray.read(f"{golden_dir}/kat0_two_params.bin")
    w2, w1 = arr.tensors[0].data, arr.tensors[1].data
    x = np.ones((1, 3, 224, 224), np.float32)
    c1, c2 = G.Conv(w1, 1, 0, dtype), G.Conv(w2, 1, 0, dtype)
    try:
        y1, _ = c1.run(x)
        y2, _ = c2.run(y1)
    finally:
        c1.close()
        c2.close()
    assert y2.shape == (1, 1, 218, 218)
    assert (y2 == 15.0).all()


def test_conv_winograd_fixture_closed_form():
    """tests/ConvOptimization/conv2dNchwWinograd.mlir: 1x16x16x4 input, 3x3x4x16 filter splat 0.1:
    all-ones input and zero init give 0.1 * 36 = 3.6 everywhere."""
    x = np.ones((1, 4, 16, 16), np.float32)
    w = np.full((16, 4, 3, 3), 0.1, np.float32)
    conv = G.Conv(w, 1, 0, F32)
    try:
        y, _ = conv.run(x)
    finally:
        conv.close()
    assert y.shape == (1, 16, 14, 14)
    np.testing.assert_allclose(y, 3.6, rtol=1e-6)


@pytest.mark.parametrize("case", [
    # n, c, h, w, k, r, stride, pad, bn
    (3, 64, 56, 56, 128, 3, 2, 1, 128),
    (5, 128, 28, 28, 256, 3, 2, 1, 256),
    (2, 256, 14, 14, 512, 3, 2, 1, 256),
    (7, 128, 28, 28, 256, 1, 2, 0, 128),
    (1, 64, 9, 13, 128, 3, 2, 1, 128),       # odd number of pixel tiles: the peer CTA's last tile is empty
    (4, 64, 16, 16, 256, 3, 1, 1, 256),
])
@pytest.mark.parametrize("dtype,res", [(F16, False), (F16, True), (BF16, False)])
def test_conv_per_tap_on_cta_pairs(case, dtype, res):
    """The per-tap TMA kernel with tcgen05.mma.cta_group::2 (each CTA loads its own pixel tile and half
    of every weight tile) against the oracle, and bit for bit against the single-CTA kernel."""
    n, c, h, w, k, r, stride, pad, bn = case
    g = _rng(n * 7 + c + h + k + r)
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((k, c, r, r)) * np.sqrt(2.0 / (r * r * c))).astype(np.float32)
    scale = g.uniform(0.5, 1.5, k).astype(np.float32)
    shift = (g.standard_normal(k) * 0.1).astype(np.float32)
    oh, ow = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    rs = g.standard_normal((n, k, oh, ow)).astype(np.float32) if res else None
    conv = G.Conv(wt, stride, pad, dtype)
    try:
        check(lib().nncv_b200_conv_set_tile(conv.h, bn, 1, 0))
        y1, xq = conv.run(x, scale, shift, rs, True)
        check(lib().nncv_b200_conv_set_tile(conv.h, bn, 1, 2))
        y2, _ = conv.run(x, scale, shift, rs, True)
    finally:
        conv.close()
    assert np.array_equal(y1, y2)
    tdt = G.TORCH_DT[dtype]
    ref = ob.conv2d(xq, torch.from_numpy(wt).to(tdt).float().numpy(), stride, pad, acc64=True)
    ref = ref * scale[None, :, None, None] + shift[None, :, None, None]
    if res:
        ref = ref + torch.from_numpy(rs).to(tdt).float().numpy()
    ref = np.where(ref > 0, ref, 0)
    assert G.rel_l2(y2, ref) <= (TOL_16 if dtype == F16 else 8e-3)


@pytest.mark.parametrize("case", [
    # n, c, h, w, k, r, stride, pad, bn     channel counts of MobileNetV3 / ResNet-50 that are not multiples of 64
    (3, 16, 56, 56, 72, 1, 1, 0, 128), (2, 72, 28, 28, 24, 1, 1, 0, 64), (2, 88, 28, 28, 24, 1, 1, 0, 64), (4, 40, 14, 14, 240, 1, 1, 0, 128),
    (1, 96, 14, 14, 40, 1, 1, 0, 64), (2, 24, 17, 19, 88, 3, 2, 1, 64), (2, 64, 28, 28, 256, 1, 1, 0, 256), (3, 256, 14, 14, 64, 1, 1, 0, 64),
    (2, 128, 28, 28, 512, 1, 1, 0, 128), (3, 64, 56, 56, 128, 3, 2, 1, 128),
])
@pytest.mark.parametrize("dtype,res", [(F16, False), (F16, True), (BF16, True)])
def test_conv_ragged_channels(case, dtype, res):
    """The TMA-fed kernel on channel counts that are not multiples of 64 (last channel block zero-filled by the copy engine,
    weights packed per tap; output widths below 64 and not a multiple of 32, residual read with guarded loads), with streamed
    and with resident weights.  Against the oracle, and the two against each other bit for bit."""
    n, c, h, w, k, r, stride, pad, bn = case
    g = _rng(n * 3 + c + h + k + r)
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((k, c, r, r)) * np.sqrt(2.0 / (r * r * c))).astype(np.float32)
    scale = g.uniform(0.5, 1.5, k).astype(np.float32)
    shift = (g.standard_normal(k) * 0.1).astype(np.float32)
    oh, ow = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    rs = g.standard_normal((n, k, oh, ow)).astype(np.float32) if res else None
    conv = G.Conv(wt, stride, pad, dtype)
    try:
        check(lib().nncv_b200_conv_set_tile(conv.h, bn, 1, 0))
        y1, xq = conv.run(x, scale, shift, rs, True)
        check(lib().nncv_b200_conv_set_tile(conv.h, 64, 1, 1))      # resident weights
        y2, _ = conv.run(x, scale, shift, rs, True)
    finally:
        conv.close()
    assert np.array_equal(y1, y2)
    tdt = G.TORCH_DT[dtype]
    ref = ob.conv2d(xq, torch.from_numpy(wt).to(tdt).float().numpy(), stride, pad, acc64=True)
    ref = ref * scale[None, :, None, None] + shift[None, :, None, None]
    if res:
        ref = ref + torch.from_numpy(rs).to(tdt).float().numpy()
    ref = np.where(ref > 0, ref, 0)
    assert G.rel_l2(y1, ref) <= (TOL_16 if dtype == F16 else 8e-3)
    assert lib().nncv_b200_device_status() == 0


@pytest.mark.parametrize("case", [(3, 16, 56, 56, 16), (2, 32, 28, 28, 24), (2, 24, 29, 31, 32), (5, 16, 17, 112, 16), (2, 8, 14, 14, 32),
                                  (1, 8, 9, 7, 8)])
@pytest.mark.parametrize("dtype,res,relu", [(F16, False, True), (F16, True, False), (BF16, True, True)])
def test_conv_pointwise_few_channels(case, dtype, res, relu):
    """1x1 stride-1 convolutions with at most 32 channels on both sides take the CUDA-core pointwise kernel (a rule on the
    layer alone): against the oracle, and within 16-bit rounding of the tensor-core kernel forced on the same inputs."""
    n, c, h, w, k = case
    g = _rng(n + c + h + k)
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((k, c, 1, 1)) * np.sqrt(2.0 / c)).astype(np.float32)
    scale = g.uniform(0.5, 1.5, k).astype(np.float32)
    shift = (g.standard_normal(k) * 0.1).astype(np.float32)
    rs = g.standard_normal((n, k, h, w)).astype(np.float32) if res else None
    conv = G.Conv(wt, 1, 0, dtype)
    try:
        launches0 = lib().nncv_b200_launch_count()
        y1, xq = conv.run(x, scale, shift, rs, relu)
        check(lib().nncv_b200_conv_set_tile(conv.h, 64, 1, 0))       # the TMA-fed tensor-core kernel
        y2, _ = conv.run(x, scale, shift, rs, relu)
    finally:
        conv.close()
    assert lib().nncv_b200_launch_count() > launches0
    tdt = G.TORCH_DT[dtype]
    ref = ob.conv2d(xq, torch.from_numpy(wt).to(tdt).float().numpy(), 1, 0, acc64=True)
    ref = ref * scale[None, :, None, None] + shift[None, :, None, None]
    if res:
        ref = ref + torch.from_numpy(rs).to(tdt).float().numpy()
    if relu:
        ref = np.where(ref > 0, ref, 0)
    tol = TOL_16 if dtype == F16 else 8e-3
    assert G.rel_l2(y1, ref) <= tol and G.rel_l2(y2, ref) <= tol and G.rel_l2(y1, y2) <= tol
    assert lib().nncv_b200_device_status() == 0


@pytest.mark.parametrize("shape", [(3, 64, 56, 56, 128), (2, 128, 28, 28, 256), (5, 256, 14, 14, 512), (1, 64, 9, 13, 128)])
@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("pair", [False, True])
def test_conv_fused_downsample(shape, dtype, pair):
    """The 3x3 stride-2 conv and the 1x1 stride-2 downsample conv of a BasicBlock in one launch
    (Res18.mlir: convs on %padded_107 and %cst_62): equal to two separate launches bit for bit and
    to the oracle within the 16-bit tolerance."""
    n, c, h, w, k = shape
    g = _rng(n + c + h + k)
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    w3 = (g.standard_normal((k, c, 3, 3)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    w1 = (g.standard_normal((k, c, 1, 1)) * np.sqrt(2.0 / c)).astype(np.float32)
    sc3, sh3 = g.uniform(0.5, 1.5, k).astype(np.float32), (g.standard_normal(k) * 0.1).astype(np.float32)
    sc1, sh1 = g.uniform(0.5, 1.5, k).astype(np.float32), (g.standard_normal(k) * 0.1).astype(np.float32)
    main, branch = G.Conv(w3, 2, 1, dtype), G.Conv(w1, 2, 0, dtype)
    try:
        y3, xq = main.run(x, sc3, sh3, relu=True)
        y1, _ = branch.run(x, sc1, sh1, relu=False)
        check(lib().nncv_b200_conv_set_tile(main.h, 128, 1, 2 if pair else 0))   # one CTA per tile, or CTA pairs
        X = G.dev(np.ascontiguousarray(x.transpose(0, 2, 3, 1)), dtype)
        oh, ow = (h + 2 - 3) // 2 + 1, (w + 2 - 3) // 2 + 1
        Y3 = torch.full((n, oh, ow, k), float("nan"), device="cuda", dtype=G.TORCH_DT[dtype])
        Y1 = torch.full((n, oh, ow, k), float("nan"), device="cuda", dtype=G.TORCH_DT[dtype])
        S3, H3, S1, H1 = (G.dev(a, F32) for a in (sc3, sh3, sc1, sh1))
        check(lib().nncv_b200_conv_run_fused(main.h, branch.h, G.p(X), G.p(Y3), G.p(Y1), n, h, w, G.p(S3), G.p(H3),
                                             G.p(S1), G.p(H1), 1, G.stream_ptr()))
        G.sync_check()
    finally:
        main.close()
        branch.close()
    f3, f1 = G.host(Y3).transpose(0, 3, 1, 2), G.host(Y1).transpose(0, 3, 1, 2)
    assert np.array_equal(f3, y3) and np.array_equal(f1, y1)
    tdt = G.TORCH_DT[dtype]
    q = lambda a: torch.from_numpy(a).to(tdt).float().numpy()
    r3 = ob.relu(ob.conv2d(xq, q(w3), 2, 1, acc64=True) * sc3[None, :, None, None] + sh3[None, :, None, None])
    r1 = ob.conv2d(xq, q(w1), 2, 0, acc64=True) * sc1[None, :, None, None] + sh1[None, :, None, None]
    tol = TOL_16 if dtype == F16 else 8e-3
    assert G.rel_l2(f3, r3) <= tol and G.rel_l2(f1, r1) <= tol


@pytest.mark.parametrize("shape", [(2, 32, 32), (2, 224, 224), (1, 37, 53), (1, 64, 300), (3, 256, 256), (1, 7, 7)])
@pytest.mark.parametrize("dtype,in_dt", [(F16, F32), (F16, F16), (BF16, F32)])
@pytest.mark.parametrize("policy", [0, 1])
def test_stem_pool_fused(shape, dtype, in_dt, policy):
    """7x7 s2 conv + scale/shift + ReLU + 3x3 s2 max-pool in one kernel vs the oracle's
    conv -> batch-norm-style affine -> ReLU -> max-pool chain (Res18.mlir:118-151), on both
    operand paths (policy 0: swizzled operand through an overlapping-stride tensor map where the
    shape allows it; policy 1: plain rows and the un-swizzled operand)."""
    n, h, w = shape
    g = _rng(n * 1000 + h + w)
    x = g.standard_normal((n, 3, h, w)).astype(np.float32)
    wt = (g.standard_normal((64, 3, 7, 7)) * np.sqrt(2.0 / 147)).astype(np.float32)
    scale = g.uniform(0.5, 1.5, 64).astype(np.float32)
    shift = (g.standard_normal(64) * 0.1).astype(np.float32)
    X = G.dev(x, in_dt)
    Wd = G.dev(wt, F32)
    sc, sh = G.dev(scale, F32), G.dev(shift, F32)
    oh, ow = (h + 6 - 7) // 2 + 1, (w + 6 - 7) // 2 + 1
    ph, pw = (oh + 2 - 3) // 2 + 1, (ow + 2 - 3) // 2 + 1
    Y = torch.full((n, ph, pw, 64), float("nan"), device="cuda", dtype=G.TORCH_DT[dtype])
    lib().nncv_b200_stem_variant(policy)
    try:
        check(lib().nncv_b200_stem_pool(G.p(X), in_dt, G.p(Wd), F32, G.p(sc), G.p(sh), G.p(Y), dtype, n, h, w,
                                        G.stream_ptr()))
        torch.cuda.synchronize()
        took = lib().nncv_b200_stem_variant(-1)
    finally:
        lib().nncv_b200_stem_variant(0)
    assert took == (2 if policy == 0 and ow <= 128 and h % 2 == 0 else 1)
    tdt = G.TORCH_DT[dtype]
    xr = torch.from_numpy(x).to(G.TORCH_DT[in_dt]).to(tdt).float().numpy()
    wr = torch.from_numpy(wt).to(tdt).float().numpy()
    conv = ob.conv2d(xr, wr, 2, 3, acc64=True) * scale[None, :, None, None] + shift[None, :, None, None]
    ref = ob.maxpool(ob.relu(conv), 3, 2, 1)
    y = G.host(Y).transpose(0, 3, 1, 2)
    assert y.shape == ref.shape and np.isfinite(y).all()
    assert G.rel_l2(y, ref) <= (TOL_16 if dtype == F16 else 8e-3)


@pytest.mark.parametrize("dtype", [F16, F32])
def test_maxpool(dtype):
    g = _rng(11)
    x = g.standard_normal((2, 64, 17, 19)).astype(np.float32)
    X = G.dev(x.transpose(0, 2, 3, 1), dtype)
    oh, ow = (17 + 2 - 3) // 2 + 1, (19 + 2 - 3) // 2 + 1
    Y = torch.empty((2, oh, ow, 64), device="cuda", dtype=G.TORCH_DT[dtype])
    check(lib().nncv_b200_maxpool_nhwc(G.p(X), G.p(Y), dtype, 2, 17, 19, 64, 3, 2, 1, G.stream_ptr()))
    torch.cuda.synchronize()
    ref = ob.maxpool(G.host(X).transpose(0, 3, 1, 2), 3, 2, 1)
    assert np.array_equal(G.host(Y).transpose(0, 3, 1, 2), ref)   # max is exact


@pytest.mark.parametrize("dtype", [F16, F32])
def test_avgpool(dtype):
    g = _rng(12)
    x = g.standard_normal((3, 512, 7, 7)).astype(np.float32)
    X = G.dev(x.transpose(0, 2, 3, 1), dtype)
    Y = torch.empty((3, 512), device="cuda", dtype=G.TORCH_DT[dtype])
    check(lib().nncv_b200_avgpool_nhwc(G.p(X), G.p(Y), dtype, 3, 49, 512, G.stream_ptr()))
    torch.cuda.synchronize()
    ref = ob.avgpool_global(G.host(X).transpose(0, 3, 1, 2))
    assert G.rel_l2(G.host(Y), ref) <= (1e-3 if dtype == F16 else 1e-6)


@pytest.mark.parametrize("n,c,h,w", [(2, 72, 56, 56), (1, 4096, 23, 23), (3, 2088, 19, 27), (5, 8, 64, 65), (2, 120, 28, 28)])
@pytest.mark.parametrize("dtype", [F16, F32, BF16])
def test_avgpool_large_map(n, c, h, w, dtype):
    """Maps of 512 pixels and more take the cluster kernel (eight CTAs per image, totals added through
    distributed shared memory): channel-vector counts that are not powers of two, more than 256
    vectors (several channel groups), pixel counts that do not divide by eight."""
    g = _rng(n * c + h)
    x = (g.standard_normal((n, c, h, w)) + 0.5).astype(np.float32)
    X = G.dev(x.transpose(0, 2, 3, 1), dtype)
    Y = torch.full((n, c), float("nan"), device="cuda", dtype=G.TORCH_DT[dtype])
    check(lib().nncv_b200_avgpool_nhwc(G.p(X), G.p(Y), dtype, n, h * w, c, G.stream_ptr()))
    torch.cuda.synchronize()
    ref = ob.avgpool_global(G.host(X).transpose(0, 3, 1, 2))
    assert np.abs(G.host(Y) - ref).max() <= {F16: 1e-3, F32: 2e-6, BF16: 8e-3}[dtype]
    assert lib().nncv_b200_device_status() == 0


def test_nchw_to_nhwc_and_bn_fold():
    g = _rng(13)
    x = g.standard_normal((2, 3, 10, 12)).astype(np.float32)
    X = G.dev(x, F32)
    Y = torch.empty((2, 10, 12, 8), device="cuda", dtype=torch.float16)
    check(lib().nncv_b200_nchw_to_nhwc(G.p(X), F32, G.p(Y), F16, 2, 3, 10, 12, 8, G.stream_ptr()))
    torch.cuda.synchronize()
    y = G.host(Y)
    assert (y[..., 3:] == 0).all()
    assert np.array_equal(y[..., :3], x.astype(np.float16).astype(np.float32).transpose(0, 2, 3, 1))
    c = 70
    gamma, beta = g.uniform(0.5, 1.5, c).astype(np.float32), g.standard_normal(c).astype(np.float32)
    mean, var = g.standard_normal(c).astype(np.float32), g.uniform(0.5, 1.5, c).astype(np.float32)
    sc = torch.empty(c, device="cuda")
    sh = torch.empty(c, device="cuda")
    t = [G.dev(v, F32) for v in (gamma, beta, mean, var)]
    check(lib().nncv_b200_bn_fold(G.p(t[0]), G.p(t[1]), G.p(t[2]), G.p(t[3]), F32, c, G.p(sc), G.p(sh), G.stream_ptr()))
    torch.cuda.synchronize()
    xs = g.standard_normal((1, c, 4, 4)).astype(np.float32)
    ref = ob.batchnorm(xs, gamma, beta, mean, var)
    got = xs * G.host(sc)[None, :, None, None] + G.host(sh)[None, :, None, None]
    assert G.rel_l2(got, ref) <= 1e-6
