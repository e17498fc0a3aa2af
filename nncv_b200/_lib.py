"""ctypes binding of libnncv_b200.so (the C ABI declared in include/nncv_b200.h).

There is no CPU fallback: if the shared library is missing this module raises, and every
compute entry point of the library itself fails when no sm_100 device is present.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_size_t, c_void_p

from .memref import MemRefDescriptor1, MemRefDescriptor2, MemRefDescriptor4, MemRefIndexer

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnncv_b200.so")

# every symbol include/nncv_b200.h declares
EXPORTS = [
    "_mlir_ciface_forward", "nncv_b200_load", "nncv_b200_load_blob", "nncv_b200_unload",
    "nncv_b200_forward_device", "nncv_b200_last_status", "nncv_b200_last_error",
    "nncv_b200_launch_count", "nncv_b200_set_stream", "nncv_b200_profile", "nncv_b200_profile_count",
    "nncv_b200_profile_get", "nncv_b200_device_status", "nncv_b200_selftest_wait_timeout",
    "nncv_b200_arena_plan", "nncv_b200_activation_bytes", "nncv_b200_plan_check", "nncv_b200_plan_text",
    "nncv_b200_shard_range", "nncv_b200_selftest_fanout",
    "nncv_b200_depthwise_conv_nhwc", "nncv_b200_activation", "nncv_b200_se_gate", "nncv_b200_scale_channels_nhwc",
    "nncv_b200_concat_channels_nhwc", "nncv_b200_upsample2x_nhwc",
    "nncv_flat_array_read", "nncv_flat_array_free", "nncv_flat_array_count",
    "nncv_flat_array_indexer", "nncv_flat_array_data", "nncv_flat_array_wrapped",
    "nncv_flat_array_write",
    "nncv_b200_matmul", "nncv_b200_matmul_noalloc", "nncv_b200_conv_create", "nncv_b200_conv_destroy", "nncv_b200_conv_run",
    "nncv_b200_conv_run_fused", "nncv_b200_conv_set_tile", "nncv_b200_stem_pool", "nncv_b200_stem_variant",
    "nncv_b200_maxpool_nhwc", "nncv_b200_avgpool_nhwc", "nncv_b200_nchw_to_nhwc", "nncv_b200_bn_fold",
]

F32, F16, BF16 = 0, 1, 2


class ProfRec(ctypes.Structure):
    _fields_ = [("kind", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("bn", c_int),
                ("flops", ctypes.c_double), ("bytes", ctypes.c_double), ("ms", ctypes.c_float)]


class Opts(ctypes.Structure):
    _fields_ = [("compute_dtype", c_int), ("device_mask", ctypes.c_uint), ("reserved", c_int * 6)]


_lib = None


def lib() -> ctypes.CDLL:
    """Load the library once; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `make -C nncv_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no CPU fallback.")
    L = ctypes.CDLL(LIB_PATH)
    L._mlir_ciface_forward.argtypes = [POINTER(MemRefDescriptor2), POINTER(MemRefDescriptor4), c_void_p]
    L._mlir_ciface_forward.restype = None
    L.nncv_b200_load.argtypes = [c_char_p, c_char_p, POINTER(Opts)]
    L.nncv_b200_load_blob.argtypes = [c_char_p, c_void_p, c_size_t, c_size_t, POINTER(Opts)]
    L.nncv_b200_unload.argtypes = []
    L.nncv_b200_forward_device.argtypes = [POINTER(MemRefDescriptor2), POINTER(MemRefDescriptor4), c_void_p]
    L.nncv_b200_last_status.restype = c_int
    L.nncv_b200_last_error.restype = c_char_p
    L.nncv_b200_launch_count.restype = c_longlong
    L.nncv_b200_set_stream.argtypes = [c_void_p, c_int]
    L.nncv_b200_device_status.restype = c_int
    L.nncv_b200_arena_plan.argtypes = [c_size_t, POINTER(c_int), POINTER(c_int), POINTER(c_size_t), c_size_t,
                                       POINTER(c_size_t), POINTER(c_size_t)]
    L.nncv_b200_depthwise_conv_nhwc.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 10 + [c_void_p]
    L.nncv_b200_activation.argtypes = [c_void_p, c_void_p, c_int, c_size_t, c_int, c_void_p]
    L.nncv_b200_se_gate.argtypes = [c_void_p] * 6 + [c_int] * 4 + [c_void_p]
    L.nncv_b200_scale_channels_nhwc.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    L.nncv_b200_concat_channels_nhwc.argtypes = [POINTER(c_void_p), POINTER(c_int), c_int, c_void_p, c_int, c_longlong, c_void_p]
    L.nncv_b200_upsample2x_nhwc.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
    L.nncv_b200_shard_range.argtypes = [c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)]
    L.nncv_b200_selftest_fanout.argtypes = [c_int, c_int, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)]
    L.nncv_b200_plan_text.argtypes = [c_char_p, ctypes.c_char_p, c_size_t]
    L.nncv_b200_plan_text.restype = c_longlong
    L.nncv_b200_plan_check.argtypes = [c_char_p, POINTER(c_size_t), POINTER(c_int), POINTER(c_int)]
    L.nncv_b200_activation_bytes.argtypes = [POINTER(c_size_t), POINTER(c_size_t)]
    L.nncv_b200_selftest_wait_timeout.argtypes = [c_int, c_void_p]
    L.nncv_b200_profile.argtypes = [c_int]
    L.nncv_b200_profile_count.restype = c_longlong
    L.nncv_b200_profile_get.argtypes = [c_longlong, POINTER(ProfRec)]
    L.nncv_flat_array_read.argtypes = [c_char_p]
    L.nncv_flat_array_read.restype = c_void_p
    L.nncv_flat_array_free.argtypes = [c_void_p]
    L.nncv_flat_array_free.restype = None
    L.nncv_flat_array_count.argtypes = [c_void_p]
    L.nncv_flat_array_count.restype = c_size_t
    L.nncv_flat_array_indexer.argtypes = [c_void_p, c_size_t]
    L.nncv_flat_array_indexer.restype = POINTER(MemRefIndexer)
    L.nncv_flat_array_data.argtypes = [c_void_p, c_size_t]
    L.nncv_flat_array_data.restype = c_void_p
    L.nncv_flat_array_wrapped.argtypes = [c_void_p]
    L.nncv_flat_array_wrapped.restype = POINTER(MemRefDescriptor1)
    L.nncv_flat_array_write.argtypes = [c_char_p, c_size_t, POINTER(MemRefIndexer), POINTER(c_void_p)]
    L.nncv_b200_matmul.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_int, c_void_p]
    L.nncv_b200_matmul_noalloc.argtypes = L.nncv_b200_matmul.argtypes
    L.nncv_b200_conv_create.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int]
    L.nncv_b200_conv_create.restype = c_void_p
    L.nncv_b200_conv_destroy.argtypes = [c_void_p]
    L.nncv_b200_conv_destroy.restype = None
    L.nncv_b200_conv_run.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_void_p]
    L.nncv_b200_conv_run_fused.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    L.nncv_b200_conv_set_tile.argtypes = [c_void_p, c_int, c_int, c_int]
    L.nncv_b200_stem_pool.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_int, c_void_p]
    L.nncv_b200_stem_variant.argtypes = [c_int]
    L.nncv_b200_maxpool_nhwc.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_int, c_void_p]
    L.nncv_b200_avgpool_nhwc.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    L.nncv_b200_nchw_to_nhwc.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p]
    L.nncv_b200_bn_fold.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                    c_void_p]
    _lib = L
    return L


class NncvError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"nncv_b200 status {code}: {msg}")
        self.code = code


def check(code: int) -> None:
    if code != 0:
        raise NncvError(code, lib().nncv_b200_last_error().decode())


def check_last() -> None:
    check(lib().nncv_b200_last_status())
