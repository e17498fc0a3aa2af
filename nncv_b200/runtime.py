"""Python face of the drop-in boundary: what nncv's example driver does in C++
(examples/Res18/main.cpp:25-118: read model.bin, fill two MemRefDescriptors, call
``_mlir_ciface_forward``), over the C ABI of libnncv_b200.so.  Tensors are numpy arrays (host)
or torch CUDA tensors (device); all arithmetic happens in the library's CUDA kernels.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from . import _lib
from ._lib import BF16, F16, F32, Opts, check, check_last, lib
from .memref import MemRefDescriptor1, make_descriptor


def _ptr(t) -> int:
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()  # torch tensor


def load(net: str, model_bin: str, compute_dtype: int = -1, device_mask: int = 0) -> None:
    """`-split-params` weight loading: parse, upload, fold BN, pack (include/nncv_b200.h).
    device_mask: replicas on several devices of this process (bit d = device d), batches in host
    memory are then split over them."""
    o = Opts()
    o.compute_dtype = compute_dtype
    o.device_mask = device_mask
    check(lib().nncv_b200_load(net.encode(), model_bin.encode(), ctypes.byref(o)))


def load_blob(net: str, blob: np.ndarray, compute_dtype: int = -1, device_mask: int = 0) -> None:
    o = Opts()
    o.compute_dtype = compute_dtype
    o.device_mask = device_mask
    blob = np.ascontiguousarray(blob)
    check(lib().nncv_b200_load_blob(net.encode(), blob.ctypes.data, blob.size, blob.itemsize, ctypes.byref(o)))


def unload() -> None:
    check(lib().nncv_b200_unload())


def forward(dst, src, params: Optional[np.ndarray] = None) -> None:
    """``_mlir_ciface_forward(&dst, &src, params)``: dst [N,1000], src [N,3,H,W] dense NCHW.

    dst/src are numpy arrays or torch tensors (host or CUDA); params, if given, is the rank-1
    blob (as MemRefFlatArray::get() hands out) and is needed only when no model was loaded.
    """
    d = make_descriptor(_ptr(dst), dst.shape)
    s = make_descriptor(_ptr(src), src.shape)
    p = None
    if params is not None:
        pd = make_descriptor(_ptr(params), (params.size,))
        p = ctypes.cast(ctypes.pointer(pd), ctypes.c_void_p)
    lib()._mlir_ciface_forward(ctypes.byref(d), ctypes.byref(s), p)
    check_last()


def forward_device(dst, src, stream: int = 0) -> None:
    """Device-resident forward on a caller's CUDA stream; does not synchronise."""
    d = make_descriptor(_ptr(dst), dst.shape)
    s = make_descriptor(_ptr(src), src.shape)
    check(lib().nncv_b200_forward_device(ctypes.byref(d), ctypes.byref(s), ctypes.c_void_p(stream)))


def launch_count() -> int:
    return int(lib().nncv_b200_launch_count())


def set_stream(stream: int, enable: bool = True) -> None:
    """Run `_mlir_ciface_forward` on the caller's CUDA stream."""
    check(lib().nncv_b200_set_stream(ctypes.c_void_p(stream), int(enable)))


def profile(enable: bool) -> None:
    check(lib().nncv_b200_profile(int(enable)))


def profile_records():
    """Per-launch records (kind, M, N, K, bn, flops, bytes, ms) since profile(True)."""
    out = []
    n = int(lib().nncv_b200_profile_count())
    for i in range(n):
        r = _lib.ProfRec()
        check(lib().nncv_b200_profile_get(i, ctypes.byref(r)))
        out.append(dict(kind=r.kind, M=r.M, N=r.N, K=r.K, bn=r.bn, flops=r.flops, bytes=r.bytes, ms=r.ms))
    return out
