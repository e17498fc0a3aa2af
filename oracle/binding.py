"""ctypes binding of the CPU oracle (oracle/libnncv_oracle.so) and of the compiled reference
container code (oracle/_ref/libnncv_rt_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU
baseline legs.  The product library never touches it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_char_p, c_int, c_long, c_size_t, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libnncv_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libnncv_rt_ref.so")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_o = None


def build() -> None:
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


def oracle() -> ctypes.CDLL:
    global _o
    if _o is None:
        if not os.path.exists(ORACLE_SO):
            build()
        L = ctypes.CDLL(ORACLE_SO)
        L.nncv_oracle_num_threads.restype = c_int
        L.nncv_oracle_set_threads.argtypes = [c_int]
        L.nncv_oracle_set_threads.restype = None
        L.nncv_oracle_conv2d_nchw_fchw.argtypes = [_f32p, _f32p, _f32p] + [c_int] * 10
        L.nncv_oracle_conv2d_nchw_fchw.restype = None
        L.nncv_oracle_batchnorm.argtypes = [_f32p] * 6 + [c_int, c_int, c_long]
        L.nncv_oracle_batchnorm.restype = None
        L.nncv_oracle_relu.argtypes = [_f32p, c_size_t]
        L.nncv_oracle_relu.restype = None
        L.nncv_oracle_add.argtypes = [_f32p, _f32p, c_size_t]
        L.nncv_oracle_add.restype = None
        L.nncv_oracle_maxpool_nchw.argtypes = [_f32p, _f32p] + [c_int] * 7
        L.nncv_oracle_maxpool_nchw.restype = None
        L.nncv_oracle_avgpool_global.argtypes = [_f32p, _f32p, c_int, c_int, c_long]
        L.nncv_oracle_avgpool_global.restype = None
        L.nncv_oracle_matmul.argtypes = [_f32p, _f32p, _f32p, c_int, c_int, c_int, c_void_p, c_int, c_int]
        L.nncv_oracle_matmul.restype = None
        L.nncv_oracle_depthwise_conv_nchw_chw.argtypes = [_f32p, _f32p, _f32p] + [c_int] * 9
        L.nncv_oracle_depthwise_conv_nchw_chw.restype = None
        L.nncv_oracle_activation.argtypes = [_f32p, c_size_t, c_int]
        L.nncv_oracle_activation.restype = None
        L.nncv_oracle_concat_channels.argtypes = [ctypes.POINTER(c_void_p), ctypes.POINTER(c_int), c_int, _f32p, c_int, c_long]
        L.nncv_oracle_concat_channels.restype = None
        L.nncv_oracle_upsample2x.argtypes = [_f32p, _f32p, c_int, c_int, c_int, c_int]
        L.nncv_oracle_upsample2x.restype = None
        L.nncv_oracle_resnet_param_count.argtypes = [c_int]
        L.nncv_oracle_resnet_param_count.restype = c_size_t
        L.nncv_oracle_resnet_forward.argtypes = [c_int, _f32p, c_int, c_int, c_int, _f32p, c_size_t, _f32p, c_int]
        L.nncv_oracle_resnet_forward.restype = c_int
        _o = L
    return _o


def _c(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def conv2d(x, w, stride=1, pad=0, acc64=False) -> np.ndarray:
    x, w = _c(x), _c(w)
    n, c, h, wd = x.shape
    k, c2, r, s = w.shape
    assert c == c2
    oh, ow = (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - s) // stride + 1
    y = np.empty((n, k, oh, ow), np.float32)
    oracle().nncv_oracle_conv2d_nchw_fchw(x, w, y, n, c, h, wd, k, r, s, stride, pad, int(acc64))
    return y


def batchnorm(x, gamma, beta, mean, var) -> np.ndarray:
    x = _c(x)
    n, c = x.shape[:2]
    y = np.empty_like(x)
    oracle().nncv_oracle_batchnorm(x, _c(gamma), _c(beta), _c(mean), _c(var), y, n, c, x[0, 0].size)
    return y


def relu(x) -> np.ndarray:
    y = _c(x).copy()
    oracle().nncv_oracle_relu(y, y.size)
    return y


def maxpool(x, k=3, stride=2, pad=1) -> np.ndarray:
    x = _c(x)
    n, c, h, w = x.shape
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    y = np.empty((n, c, oh, ow), np.float32)
    oracle().nncv_oracle_maxpool_nchw(x, y, n, c, h, w, k, stride, pad)
    return y


def avgpool_global(x) -> np.ndarray:
    x = _c(x)
    n, c = x.shape[:2]
    y = np.empty((n, c), np.float32)
    oracle().nncv_oracle_avgpool_global(x, y, n, c, x[0, 0].size)
    return y


def matmul(a, b, bias=None, relu=False, acc64=False) -> np.ndarray:
    a, b = _c(a), _c(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    bp = None
    if bias is not None:
        bias = _c(bias)
        bp = bias.ctypes.data
    oracle().nncv_oracle_matmul(a, b, c, m, n, k, bp, int(relu), int(acc64))
    return c


ACT = {"none": 0, "relu": 1, "hard_sigmoid": 2, "hard_swish": 3, "sigmoid": 4, "silu": 5}


def depthwise_conv2d(x, w, stride=1, pad=0, acc64=False) -> np.ndarray:
    """x [N,C,H,W], w [C,R,S] (linalg.depthwise_conv_2d_nchw_chw)."""
    x, w = _c(x), _c(w)
    n, c, h, wd = x.shape
    c2, r, s = w.shape
    assert c == c2
    oh, ow = (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - s) // stride + 1
    y = np.empty((n, c, oh, ow), np.float32)
    oracle().nncv_oracle_depthwise_conv_nchw_chw(x, w, y, n, c, h, wd, r, s, stride, pad, int(acc64))
    return y


def activation(x, kind: str) -> np.ndarray:
    y = _c(x).copy()
    oracle().nncv_oracle_activation(y, y.size, ACT[kind])
    return y


def se_gate(pooled, w1, b1, w2, b2) -> np.ndarray:
    """Squeeze-and-excitation gate from the pooled map: the two 1x1 convs on [N,C,1,1] of the fixture are matmuls."""
    hid = matmul(pooled, np.ascontiguousarray(_c(w1).T), b1, relu=True)
    return activation(matmul(hid, np.ascontiguousarray(_c(w2).T), b2), "hard_sigmoid")


def concat_channels(xs) -> np.ndarray:
    xs = [_c(x) for x in xs]
    n, _, h, w = xs[0].shape
    chans = (c_int * len(xs))(*[x.shape[1] for x in xs])
    ptrs = (c_void_p * len(xs))(*[x.ctypes.data for x in xs])
    y = np.empty((n, sum(x.shape[1] for x in xs), h, w), np.float32)
    oracle().nncv_oracle_concat_channels(ptrs, chans, len(xs), y, n, h * w)
    return y


def upsample2x(x) -> np.ndarray:
    x = _c(x)
    n, c, h, w = x.shape
    y = np.empty((n, c, 2 * h, 2 * w), np.float32)
    oracle().nncv_oracle_upsample2x(x, y, n, c, h, w)
    return y


def resnet_forward(depth: int, x, blob, acc64=False) -> np.ndarray:
    x, blob = _c(x), _c(blob)
    n, c, h, w = x.shape
    assert c == 3
    out = np.empty((n, 1000), np.float32)
    rc = oracle().nncv_oracle_resnet_forward(depth, x, n, h, w, blob, blob.size, out, int(acc64))
    if rc != 0:
        raise ValueError(f"oracle resnet forward failed with {rc}")
    return out


def num_threads() -> int:
    return oracle().nncv_oracle_num_threads()


def use_all_cores() -> int:
    """Use every host core the process may run on (overrides an exported OMP_NUM_THREADS)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    oracle().nncv_oracle_set_threads(n)
    return num_threads()


def ref_lib():
    """The reference's own container code, or None when it has not been built."""
    if not os.path.exists(REF_SO):
        return None
    L = ctypes.CDLL(REF_SO)
    L.ref_flat_array_write.argtypes = [c_char_p, c_int, ctypes.POINTER(c_char_p), ctypes.POINTER(c_size_t),
                                       ctypes.POINTER(c_size_t), c_size_t, ctypes.POINTER(c_void_p)]
    L.ref_flat_array_read.argtypes = [c_char_p, c_size_t, ctypes.POINTER(c_long), c_void_p, c_size_t]
    for f in ("ref_sizeof_head", "ref_sizeof_indexer", "ref_sizeof_desc1", "ref_sizeof_desc2", "ref_sizeof_desc4"):
        getattr(L, f).restype = c_size_t
    return L
