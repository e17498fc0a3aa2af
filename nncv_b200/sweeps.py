"""Kernel and network sweeps over the benchmark configs other than the headline one.

    python -m nncv_b200.sweeps [gemm [SIZE]] [conv] [nets] [hbm] [mobilenet [BATCH]]

  gemm : M=N=K in {512,1024,2048,4096}, fp16 in / fp32 accumulate (fp16 and fp32 C), optional fused
         bias + ReLU, and the fp32 CUDA-core path (config 1).
  conv : 3x3 stride-1 pad-1, batch 32 (and 256 with "conv256"), (C=K, H=W) in {(64,64),(128,32),(256,16),(512,8)}, fp16, fused
         scale/shift + ReLU (config 2), for the shifted-view kernel and the TMA-fed per-tap kernel.
  nets : ResNet-18 fp32 N=1 @256 (config 0), ResNet-50 fp16 N=512 @224 (config 4), device-resident.
  hbm  : the memory-bound operators (depthwise conv + BN + hard-swish, activations, SE scaling, concat,
         2x upsampling, max-pool, global average pool) on MobileNetV3 / YOLOv5-sized maps: GB/s of
         algorithmic bytes (elements read + written) against the measured HBM copy bandwidth.
  mobilenet : MobileNetV3-small fp16 @224 from a layer plan file (default: the plan the importer wrote from nncv's
         tests/Nets/MobileNetV3.mlir, kept under tests/golden/), seeded weights, batch 256 unless given.
One JSON line per measurement; times are CUDA-event medians on the launching stream with an L2 flush
(256 MiB fill) before every timed call.  Torch only owns the device memory.
"""
from __future__ import annotations

import ctypes
import json
import sys

import numpy as np
import torch

from . import runtime as rt
from ._lib import BF16, F16, F32, check, lib

PEAK_TF = 1644.0
_flush = None


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _time(fn, reps=7):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def gemm(sizes=(512, 1024, 2048, 4096)):
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for n in sizes:
        for ab, cdt, epi in ((F16, F32, False), (F16, F16, False), (F16, F16, True), (F32, F32, False)):
            tdt = torch.float16 if ab == F16 else torch.float32
            A = (torch.rand((n, n), device="cuda") * 2 - 1).to(tdt)
            B = (torch.rand((n, n), device="cuda") * 2 - 1).to(tdt)
            C = torch.empty((n, n), device="cuda", dtype=torch.float16 if cdt == F16 else torch.float32)
            bias = torch.randn(n, device="cuda") if epi else None
            ms = _time(lambda: check(lib().nncv_b200_matmul(_p(A), _p(B), _p(C), n, n, n, ab, cdt, _p(bias), int(epi), st)))
            tf = 2.0 * n ** 3 / ms / 1e9
            print(json.dumps({"sweep": "gemm", "M=N=K": n, "ab": "f16" if ab == F16 else "f32",
                              "c": "f16" if cdt == F16 else "f32", "bias_relu": epi, "ms": round(ms, 4),
                              "tflops": round(tf, 1), "frac_of_peak": round(tf / PEAK_TF, 3),
                              "note": "one kernel: B read by TMA as it lies (row-major = MN-major operand)"}), flush=True)


def conv(n=32):
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for c, hw in ((64, 64), (128, 32), (256, 16), (512, 8)):
        w = (torch.randn((c, c, 3, 3)) * (2.0 / (9 * c)) ** 0.5).numpy().astype(np.float32)
        X = torch.randn((n, hw, hw, c), device="cuda", dtype=torch.float16)
        Y = torch.empty((n, hw, hw, c), device="cuda", dtype=torch.float16)
        sc = torch.rand(c, device="cuda") + 0.5
        sh = torch.randn(c, device="cuda") * 0.1
        for algo, name in ((2, "shifted-view conv3x3"), (0, "per-tap TMA tconv"), (1, "winograd F(2x2,3x3) 3-stage")):
            h = lib().nncv_b200_conv_create(w.ctypes.data, F32, c, c, 3, 3, 1, 1, F16, algo)
            assert h
            call = lambda: check(lib().nncv_b200_conv_run(h, _p(X), _p(Y), n, hw, hw, _p(sc), _p(sh), None, 1, st))
            call()
            torch.cuda.synchronize()
            rt.profile(True)
            for _ in range(5):
                _flush_fill()
                call()
            torch.cuda.synchronize()
            recs = [r for r in rt.profile_records() if r["kind"] in (2, 5, 6, 7)]
            rt.profile(False)
            ms = sorted(r["ms"] for r in recs)[len(recs) // 2]
            tf = recs[0]["flops"] / ms / 1e9
            print(json.dumps({"sweep": "conv3x3", "N": n, "C=K": c, "H=W": hw, "kernel": name, "us": round(ms * 1e3, 1),
                              "tflops_direct_conv": round(tf, 1), "frac_of_peak": round(tf / PEAK_TF, 3)}), flush=True)
            lib().nncv_b200_conv_destroy(h)


def _flush_fill():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    _flush.zero_()


def nets():
    from .netspec import conv_macs
    from .split_params import random_state_dict, to_flat_array
    s = torch.cuda.current_stream().cuda_stream
    for depth, dt, n, hw, name in ((18, F32, 1, 256, "R18 fp32 N=1 @256"), (18, F16, 256, 224, "R18 fp16 N=256 @224"),
                                   (50, F16, 512, 224, "R50 fp16 N=512 @224")):
        np_dt = np.float32 if dt == F32 else np.float16
        blob = to_flat_array(depth, random_state_dict(depth, 0), np_dt).blob()
        rt.load_blob(f"resnet{depth}", blob, dt)
        x = torch.randn((n, 3, hw, hw), device="cuda").to(torch.float32 if dt == F32 else torch.float16)
        out = torch.empty((n, 1000), device="cuda", dtype=x.dtype)
        ms = _time(lambda: rt.forward_device(out, x, s), reps=5)
        gf = 2.0 * conv_macs(depth, hw, hw) * n / 1e9
        print(json.dumps({"sweep": "nets", "config": name, "ms": round(ms, 3), "images_per_s": round(n / ms * 1e3, 1),
                          "tflops": round(gf / ms, 1)}), flush=True)
        rt.unload()


PEAK_GBS = 6540.5


def hbm_ops():
    """(name, GB/s, fraction of the measured HBM bandwidth) of the memory-bound operators."""
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = []
    L = lib()

    def rec(name, nbytes, fn):
        ms = _time(fn, reps=9)
        gbs = nbytes / ms / 1e6
        out.append({"sweep": "hbm", "op": name, "mb": round(nbytes / 1e6, 1), "us": round(ms * 1e3, 1), "gbs": round(gbs, 1),
                    "frac_of_hbm": round(gbs / PEAK_GBS, 3)})
        print(json.dumps(out[-1]), flush=True)

    n, c, hw = 64, 96, 112            # a MobileNetV3-large expansion layer at batch 64
    X = torch.randn((n, hw, hw, c), device="cuda", dtype=torch.float16)
    Y = torch.empty_like(X)
    W = torch.randn((c, 3, 3), device="cuda")
    sc, sh = torch.rand(c, device="cuda") + 0.5, torch.randn(c, device="cuda") * 0.1
    rec("depthwise 3x3 s1 + BN + hard-swish, 64x112x112x96 fp16", 2 * X.numel() * 2,
        lambda: check(L.nncv_b200_depthwise_conv_nhwc(_p(X), _p(W), F32, _p(sc), _p(sh), _p(Y), F16, n, hw, hw, c, 3, 3, 1, 1, 3, st)))
    rec("hard-swish, 77 M fp16 elements", 2 * X.numel() * 2, lambda: check(L.nncv_b200_activation(_p(X), _p(Y), F16, X.numel(), 3, st)))
    rec("SiLU, 77 M fp16 elements", 2 * X.numel() * 2, lambda: check(L.nncv_b200_activation(_p(X), _p(Y), F16, X.numel(), 5, st)))
    G8 = torch.rand((n, c), device="cuda", dtype=torch.float16)
    rec("SE channel scaling, 64x112x112x96 fp16", 2 * X.numel() * 2,
        lambda: check(L.nncv_b200_scale_channels_nhwc(_p(X), _p(G8), _p(Y), F16, n, hw * hw, c, st)))
    A = torch.randn((n, 80, 80, 128), device="cuda", dtype=torch.float16)    # YOLOv5s neck at batch 64
    B = torch.randn((n, 80, 80, 128), device="cuda", dtype=torch.float16)
    Cc = torch.empty((n, 80, 80, 256), device="cuda", dtype=torch.float16)
    ptrs = (ctypes.c_void_p * 2)(A.data_ptr(), B.data_ptr())
    ch = (ctypes.c_int * 2)(128, 128)
    rec("concat 2 x (64x80x80x128) fp16", 2 * Cc.numel() * 2,
        lambda: check(L.nncv_b200_concat_channels_nhwc(ptrs, ch, 2, _p(Cc), F16, n * 80 * 80, st)))
    S = torch.randn((n, 40, 40, 256), device="cuda", dtype=torch.float16)
    U = torch.empty((n, 80, 80, 256), device="cuda", dtype=torch.float16)
    rec("upsample 2x, 64x40x40x256 fp16", (S.numel() + U.numel()) * 2, lambda: check(L.nncv_b200_upsample2x_nhwc(_p(S), _p(U), F16, n, 40, 40, 256, st)))
    M = torch.randn((256, 112, 112, 64), device="cuda", dtype=torch.float16)
    Mo = torch.empty((256, 56, 56, 64), device="cuda", dtype=torch.float16)
    rec("max-pool 3x3 s2, 256x112x112x64 fp16", (M.numel() + Mo.numel()) * 2,
        lambda: check(L.nncv_b200_maxpool_nhwc(_p(M), _p(Mo), F16, 256, 112, 112, 64, 3, 2, 1, st)))
    Pq = torch.empty((256, 64), device="cuda", dtype=torch.float16)
    rec("global average pool, 256x112x112x64 fp16", M.numel() * 2, lambda: check(L.nncv_b200_avgpool_nhwc(_p(M), _p(Pq), F16, 256, 112 * 112, 64, st)))
    return out


def mobilenet(batch=256, plan_path=None):
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    plan_path = plan_path or os.path.join(root, "tests", "golden", "mobilenetv3_from_mlir.plan")
    text = open(plan_path).read()
    g = np.random.default_rng(0)
    total = int(next(l for l in text.splitlines() if l.startswith("params")).split()[1])
    blob = (g.standard_normal(total) * 0.05).astype(np.float32)
    for line in text.splitlines():          # batch-norm scales and variances must be positive
        f = dict(t.split("=") for t in line.split()[1:] if "=" in t)
        c = int(f.get("cout", f.get("c", 0)))
        for role in ("gamma", "var"):
            if role in f:
                blob[int(f[role]):int(f[role]) + c] = g.uniform(0.5, 1.5, c)
    rt.load_blob("plan:" + text, blob.astype(np.float16), F16)
    x = torch.randn((batch, 3, 224, 224), device="cuda").to(torch.float16)
    o = torch.empty((batch, 1000), device="cuda", dtype=x.dtype)
    s = torch.cuda.current_stream().cuda_stream
    rt.forward_device(o, x, s)
    torch.cuda.synchronize()
    ms = _time(lambda: rt.forward_device(o, x, s))
    print(json.dumps({"sweep": "mobilenet", "config": "MobileNetV3-small fp16 @224, imported plan", "batch": batch, "ms": round(ms, 4),
                      "images_per_s": round(batch / ms * 1e3, 1), "finite": bool(torch.isfinite(o.float()).all())}), flush=True)
    rt.unload()


if __name__ == "__main__":
    which = sys.argv[1:] or ["gemm", "conv", "nets"]
    if "mobilenet" in which:
        nums = [int(a) for a in which if a.isdigit()]
        mobilenet(nums[0] if nums else 256)
        which = [a for a in which if a != "mobilenet" and not a.isdigit()]
        if not which:
            sys.exit(0)
    sizes = tuple(int(a) for a in which if a.isdigit())
    if "gemm" in which:
        gemm(sizes or (512, 1024, 2048, 4096))
    if "hbm" in which:
        hbm_ops()
    if "conv" in which:
        conv()
    if "conv256" in which:
        conv(256)
    if "nets" in which:
        nets()
