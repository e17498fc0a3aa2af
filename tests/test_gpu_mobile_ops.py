"""GPU parity of the memory-bound operators of nncv's mobile / detection fixtures (depthwise conv +
batch-norm + activation, hard-swish / SiLU, squeeze-and-excitation, channel concat, nearest 2x
upsampling) against the CPU oracle, through the C ABI; shapes from MobileNetV3.mlir / Yolov5s.mlir."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import binding as ob  # noqa: E402
from nncv_b200._lib import BF16, F16, F32, check, lib  # noqa: E402
import gpu_util as G  # noqa: E402

ACT = {"none": 0, "relu": 1, "hard_sigmoid": 2, "hard_swish": 3, "sigmoid": 4, "silu": 5}
TOL = {F32: 2e-6, F16: 2e-3, BF16: 1.2e-2}


def nhwc(a):
    return np.ascontiguousarray(a.transpose(0, 2, 3, 1))


@pytest.mark.parametrize("case", [
    # n, c, h, w, k, stride, pad   (MobileNetV3-small: 16@128 s2, 72@64 s2, 88@32 s1, 96@32 5x5 s2, 576@8 5x5)
    (2, 16, 128, 128, 3, 2, 1), (2, 72, 64, 64, 3, 2, 1), (3, 88, 32, 32, 3, 1, 1), (2, 96, 32, 32, 5, 2, 2),
    (4, 576, 8, 8, 5, 1, 2), (1, 8, 5, 7, 3, 1, 1), (1, 24, 37, 153, 3, 1, 1), (2, 40, 30, 29, 5, 1, 2), (3, 200, 15, 14, 3, 2, 1)])
@pytest.mark.parametrize("dtype,act", [(F16, "hard_swish"), (F16, "relu"), (F32, "hard_swish"), (BF16, "none")])
def test_depthwise_conv_bn_activation(case, dtype, act):
    n, c, h, w, k, stride, pad = case
    g = np.random.default_rng(sum(case))
    x = g.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (g.standard_normal((c, k, k)) * np.sqrt(2.0 / (k * k))).astype(np.float32)
    scale = g.uniform(0.5, 1.5, c).astype(np.float32)
    shift = (g.standard_normal(c) * 0.1).astype(np.float32)
    X = G.dev(nhwc(x), dtype)
    Wd, sc, sh = G.dev(wt, F32), G.dev(scale, F32), G.dev(shift, F32)
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    Y = torch.full((n, oh, ow, c), float("nan"), device="cuda", dtype=G.TORCH_DT[dtype])
    check(lib().nncv_b200_depthwise_conv_nhwc(G.p(X), G.p(Wd), F32, G.p(sc), G.p(sh), G.p(Y), dtype, n, h, w, c, k, k, stride, pad,
                                              ACT[act], G.stream_ptr()))
    torch.cuda.synchronize()
    xq = G.host(X).transpose(0, 3, 1, 2)
    ref = ob.depthwise_conv2d(xq, wt, stride, pad, acc64=True) * scale[None, :, None, None] + shift[None, :, None, None]
    ref = ob.activation(ref, act)
    y = G.host(Y).transpose(0, 3, 1, 2)
    assert y.shape == ref.shape and np.isfinite(y).all()
    assert G.rel_l2(y, ref) <= TOL[dtype]
    assert lib().nncv_b200_device_status() == 0      # no bounded wait of the TMA-staged kernel gave up


@pytest.mark.parametrize("dtype", [F16, F32, BF16])
@pytest.mark.parametrize("act", ["relu", "hard_sigmoid", "hard_swish", "sigmoid", "silu"])
def test_activation(dtype, act):
    g = np.random.default_rng(len(act))
    x = (g.standard_normal(8 * 4099) * 4).astype(np.float32)
    x[5] = np.nan
    X = G.dev(x, dtype)
    Y = torch.empty_like(X)
    check(lib().nncv_b200_activation(G.p(X), G.p(Y), dtype, x.size, ACT[act], G.stream_ptr()))
    torch.cuda.synchronize()
    ref = ob.activation(G.host(X), act)
    y = G.host(Y)
    assert np.isnan(y[5]) and np.isnan(ref[5])                   # a NaN passes through every one of them
    m = ~np.isnan(ref)
    assert G.rel_l2(y[m], ref[m]) <= TOL[dtype]
    assert lib().nncv_b200_activation(G.p(X), G.p(Y), dtype, 13, ACT[act], G.stream_ptr()) == 1


@pytest.mark.parametrize("n,c,cr,hw", [(2, 16, 8, 64 * 64), (3, 96, 24, 16 * 16), (2, 576, 144, 8 * 8)])
@pytest.mark.parametrize("dtype", [F16, F32])
def test_squeeze_and_excitation(n, c, cr, hw, dtype):
    """avg-pool -> two 1x1 convs (ReLU, hard-sigmoid) -> broadcast multiply (MobileNetV3.mlir:319-383)."""
    g = np.random.default_rng(c + cr)
    side = int(round(hw ** 0.5))
    x = g.standard_normal((n, c, side, side)).astype(np.float32)
    w1, b1 = (g.standard_normal((cr, c)) / np.sqrt(c)).astype(np.float32), (g.standard_normal(cr) * 0.1).astype(np.float32)
    w2, b2 = (g.standard_normal((c, cr)) / np.sqrt(cr)).astype(np.float32), (g.standard_normal(c) * 0.1).astype(np.float32)
    X = G.dev(nhwc(x), dtype)
    P = torch.empty((n, c), device="cuda", dtype=G.TORCH_DT[dtype])
    Gt = torch.empty((n, c), device="cuda", dtype=G.TORCH_DT[dtype])
    Y = torch.empty_like(X)
    t = [G.dev(v, F32) for v in (w1, b1, w2, b2)]
    st = G.stream_ptr()
    check(lib().nncv_b200_avgpool_nhwc(G.p(X), G.p(P), dtype, n, hw, c, st))
    check(lib().nncv_b200_se_gate(G.p(P), G.p(t[0]), G.p(t[1]), G.p(t[2]), G.p(t[3]), G.p(Gt), dtype, n, c, cr, st))
    check(lib().nncv_b200_scale_channels_nhwc(G.p(X), G.p(Gt), G.p(Y), dtype, n, hw, c, st))
    torch.cuda.synchronize()
    xq = G.host(X).transpose(0, 3, 1, 2)
    gate = ob.se_gate(ob.avgpool_global(xq), w1, b1, w2, b2)
    assert np.abs(G.host(Gt) - gate).max() <= (2e-3 if dtype == F16 else 1e-5)
    ref = xq * gate[:, :, None, None]
    assert G.rel_l2(G.host(Y).transpose(0, 3, 1, 2), ref) <= (3e-3 if dtype == F16 else 1e-5)


@pytest.mark.parametrize("dtype", [F16, F32])
def test_concat_and_upsample(dtype):
    g = np.random.default_rng(9)
    n, h, w = 2, 20, 20
    parts = [g.standard_normal((n, c, h, w)).astype(np.float32) for c in (256, 256, 256, 256)]   # the SPPF concat of Yolov5s.mlir:837
    parts2 = [g.standard_normal((n, c, 7, 9)).astype(np.float32) for c in (8, 40, 16)]
    for ps in (parts, parts2):
        T = [G.dev(nhwc(a), dtype) for a in ps]
        ptrs = (ctypes.c_void_p * len(T))(*[t.data_ptr() for t in T])
        ch = (ctypes.c_int * len(T))(*[a.shape[1] for a in ps])
        nn, _, hh, ww = ps[0].shape
        Y = torch.empty((nn, hh, ww, sum(a.shape[1] for a in ps)), device="cuda", dtype=G.TORCH_DT[dtype])
        check(lib().nncv_b200_concat_channels_nhwc(ptrs, ch, len(T), G.p(Y), dtype, nn * hh * ww, G.stream_ptr()))
        torch.cuda.synchronize()
        ref = ob.concat_channels([G.host(t).transpose(0, 3, 1, 2) for t in T])
        assert np.array_equal(G.host(Y).transpose(0, 3, 1, 2), ref)           # a copy: exact
    X = G.dev(nhwc(parts[0]), dtype)
    U = torch.empty((n, 2 * h, 2 * w, 256), device="cuda", dtype=G.TORCH_DT[dtype])
    check(lib().nncv_b200_upsample2x_nhwc(G.p(X), G.p(U), dtype, n, h, w, 256, G.stream_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(G.host(U).transpose(0, 3, 1, 2), ob.upsample2x(G.host(X).transpose(0, 3, 1, 2)))
    bad = (ctypes.c_int * 2)(8, 3)
    assert lib().nncv_b200_concat_channels_nhwc(ptrs, bad, 2, G.p(U), dtype, 4, G.stream_ptr()) == 1


def test_yolo_spp_block_chain():
    """conv 1x1 + SiLU -> three chained 5x5 stride-1 max-pools -> concat -> conv 1x1 + SiLU (Yolov5s.mlir:790-860),
    16-bit, every op through the library."""
    g = np.random.default_rng(11)
    n, c, hw = 2, 64, 20
    x = g.standard_normal((n, c, hw, hw)).astype(np.float32)
    w1 = (g.standard_normal((32, c, 1, 1)) * np.sqrt(2.0 / c)).astype(np.float32)
    w2 = (g.standard_normal((64, 128, 1, 1)) * np.sqrt(2.0 / 128)).astype(np.float32)
    c1, c2 = G.Conv(w1, 1, 0, F16), G.Conv(w2, 1, 0, F16)
    st = G.stream_ptr()
    try:
        X = G.dev(nhwc(x), F16)
        A = torch.empty((n, hw, hw, 32), device="cuda", dtype=torch.float16)
        check(lib().nncv_b200_conv_run(c1.h, G.p(X), G.p(A), n, hw, hw, None, None, None, 0, st))
        check(lib().nncv_b200_activation(G.p(A), G.p(A), F16, A.numel(), ACT["silu"], st))
        pools = [A]
        for _ in range(3):
            Pn = torch.empty_like(A)
            check(lib().nncv_b200_maxpool_nhwc(G.p(pools[-1]), G.p(Pn), F16, n, hw, hw, 32, 5, 1, 2, st))
            pools.append(Pn)
        ptrs = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in pools])
        ch = (ctypes.c_int * 4)(32, 32, 32, 32)
        Cc = torch.empty((n, hw, hw, 128), device="cuda", dtype=torch.float16)
        check(lib().nncv_b200_concat_channels_nhwc(ptrs, ch, 4, G.p(Cc), F16, n * hw * hw, st))
        Y = torch.empty((n, hw, hw, 64), device="cuda", dtype=torch.float16)
        check(lib().nncv_b200_conv_run(c2.h, G.p(Cc), G.p(Y), n, hw, hw, None, None, None, 0, st))
        check(lib().nncv_b200_activation(G.p(Y), G.p(Y), F16, Y.numel(), ACT["silu"], st))
        torch.cuda.synchronize()
    finally:
        c1.close()
        c2.close()
    q = lambda a: torch.from_numpy(a).to(torch.float16).float().numpy()
    a = ob.activation(ob.conv2d(q(x), q(w1), 1, 0, acc64=True), "silu")
    ps = [a]
    for _ in range(3):
        ps.append(ob.maxpool(ps[-1], 5, 1, 2))
    ref = ob.activation(ob.conv2d(ob.concat_channels(ps), q(w2), 1, 0, acc64=True), "silu")
    assert G.rel_l2(G.host(Y).transpose(0, 3, 1, 2), ref) <= 5e-3
    assert lib().nncv_b200_device_status() == 0
