"""Helpers for the GPU parity tests: torch is used only to own device memory; every compute
call goes through the C ABI of libnncv_b200.so via ctypes."""
import ctypes

import numpy as np
import torch

from nncv_b200 import _lib
from nncv_b200._lib import BF16, F16, F32, check, lib

TORCH_DT = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}


def dev(a: np.ndarray, dt=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(TORCH_DT[dt]) if dt is not None else t


def host(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def sync_check():
    torch.cuda.synchronize()


def matmul(a, b, ab, c_dt, bias=None, relu=False):
    """a [M,K], b [K,N] numpy fp32 -> numpy fp32 result computed by nncv_b200_matmul."""
    m, k = a.shape
    n = b.shape[1]
    A, B = dev(a, ab), dev(b, ab)
    C = torch.full((m, n), float("nan"), device="cuda", dtype=TORCH_DT[c_dt])
    bias_t = dev(bias, F32) if bias is not None else None
    check(lib().nncv_b200_matmul(p(A), p(B), p(C), m, n, k, ab, c_dt, p(bias_t), int(relu), stream_ptr()))
    sync_check()
    return host(C), host(A), host(B)


class Conv:
    """nncv_b200_conv_create / _run / _destroy."""

    def __init__(self, w: np.ndarray, stride, pad, dtype, algo=0):
        k, c, r, s = w.shape
        self.shape = (k, c, r, s, stride, pad)
        self.dtype = dtype
        w = np.ascontiguousarray(w, np.float32)
        self.h = lib().nncv_b200_conv_create(w.ctypes.data, F32, k, c, r, s, stride, pad, dtype, algo)
        if not self.h:
            raise _lib.NncvError(lib().nncv_b200_last_status(), lib().nncv_b200_last_error().decode())

    def run(self, x_nchw: np.ndarray, scale=None, shift=None, residual_nchw=None, relu=False):
        """x NCHW fp32 numpy -> y NCHW fp32 numpy (layout conversion on the host side of the test)."""
        k, c, r, s, stride, pad = self.shape
        n, _, h, w = x_nchw.shape
        cpad = (c + 3) // 4 * 4 if self.dtype == F32 else (c + 7) // 8 * 8
        xh = np.zeros((n, h, w, cpad), np.float32)
        xh[..., :c] = x_nchw.transpose(0, 2, 3, 1)
        X = dev(xh, self.dtype)
        oh, ow = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - s) // stride + 1
        Y = torch.full((n, oh, ow, k), float("nan"), device="cuda", dtype=TORCH_DT[self.dtype])
        sc = dev(scale, F32) if scale is not None else None
        sh = dev(shift, F32) if shift is not None else None
        res = dev(residual_nchw.transpose(0, 2, 3, 1), self.dtype) if residual_nchw is not None else None
        check(lib().nncv_b200_conv_run(self.h, p(X), p(Y), n, h, w, p(sc), p(sh), p(res), int(relu), stream_ptr()))
        sync_check()
        return host(Y).transpose(0, 3, 1, 2), host(X)[..., :c].transpose(0, 3, 1, 2)

    def close(self):
        if self.h:
            lib().nncv_b200_conv_destroy(self.h)
            self.h = None
