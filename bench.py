#!/usr/bin/env python
"""Benchmark of the compiled-forward hot path: ResNet-18 fp16 inference, batch 256 of 3x224x224.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

One "step" is one forward over the (global) batch, sharded by contiguous image ranges over N
ranks (one process per GPU, launched by torchrun for N > 1), logits gathered to rank 0.
  value : images/s with the input already in HBM (nncv_b200_forward_device), CUDA events on the
          launching stream, an L2 flush between steps, max over ranks.
  e2e   : images/s through `_mlir_ciface_forward` with pinned HOST input: the host->device copy of
          the images and the device->host copy of the logits (at N > 1: of the gathered logits, on
          rank 0) are inside the timed region.
  roofline : algorithmic direct-convolution FLOPs of one step / the step time OF THE TIMED REGION
          (every kernel of the step, helpers included), vs the measured dense bf16/fp16 tensor
          peak.  `per_launch_pass` is a separate pass with events around every launch (it
          serialises the launches, so its sum exceeds the step time); it attributes time to kernels.
  split : forward and gather time of the timed steps, from two event pairs per step.
  secondary : the other benchmark configs (GEMM sweep, 3x3 conv sweep, ResNet-18 fp32, ResNet-50)
          measured after the headline on one GPU, each with its own clock window.
  cpu_baseline : the CPU oracle (a port of the reference's linalg graph; the reference's own
          HostWParallel build needs an MLIR/LLVM toolchain that is absent) on the host cores,
          on a bounded sample of images; `torch_cpu` beside it is PyTorch's CPU operators
          (oneDNN) on the same sample, for context.
--impl reference times that CPU path alone (rank 0 only).
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "resnet18_fp16_images_per_s"
UNIT = "images/s"
H = W = 224


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", 0)), float(p["hbm_gbs"]), "measured"
    except Exception:
        return 1590.0, 1400.0, 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons (query only) while timed regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpus):
        self.gpus = set(gpus)
        self.proc = None
        self.lines = []

    def start(self):
        """Starts nvidia-smi and a thread that collects its lines (NVML start-up can take longer than a
        short timed region, so callers start it before the warm-up and wait for the first sample)."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return

        def pump():
            try:
                for line in self.proc.stdout:
                    self.lines.append(line)
            except Exception:
                pass
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def wait_ready(self, timeout=10.0):
        t0 = time.perf_counter()
        while self.proc is not None and not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.005)

    def pos(self):
        return len(self.lines)

    def window(self, i0, i1=None):
        """Clock statistics of the samples taken between two pos() marks."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        sm, smax, reasons = [], [], set()
        for line in self.lines[i0:i1]:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[0].isdigit() or int(f[0]) not in self.gpus:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.thread.join(timeout=2)


_CPU_STATE = {}


def cpu_oracle_images_per_s(n_images):
    """One oracle forward (fp32, every host core) of n_images of 3x224x224: (images/s, cores, seconds)."""
    from oracle import binding as ob
    from nncv_b200.split_params import random_input, random_state_dict, to_flat_array
    if "blob" not in _CPU_STATE:
        ob.use_all_cores()
        _CPU_STATE["blob"] = to_flat_array(18, random_state_dict(18, 0)).blob()
        ob.resnet_forward(18, random_input(1, H, W, 0, "normal"), _CPU_STATE["blob"])  # page everything in
    x = _CPU_STATE.setdefault(("x", n_images), random_input(n_images, H, W, 0, "normal"))
    t0 = time.perf_counter()
    ob.resnet_forward(18, x, _CPU_STATE["blob"])
    dt = time.perf_counter() - t0
    return n_images / dt, ob.num_threads(), dt


def cpu_torch_images_per_s(n_images):
    """The same network and weights on PyTorch's CPU operators (oneDNN), fp32, every host core:
    a stronger CPU number for context, not the reference and not the oracle."""
    import torch
    import torch.nn.functional as F
    from nncv_b200.netspec import conv_groups
    from nncv_b200.split_params import random_input, random_state_dict
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sd = {k: torch.from_numpy(v) for k, v in random_state_dict(18, 0).items()}
    groups = {g.name: g for g in conv_groups(18)}

    def cbr(x, g, relu):
        y = F.conv2d(x, sd[f"{g.name}.weight"], stride=g.stride, padding=g.pad)
        y = F.batch_norm(y, sd[f"{g.bn}.running_mean"], sd[f"{g.bn}.running_var"], sd[f"{g.bn}.weight"],
                         sd[f"{g.bn}.bias"], training=False, eps=1e-5)
        return F.relu(y) if relu else y

    def fwd(x):
        x = F.max_pool2d(cbr(x, groups["conv1"], True), 3, 2, 1)
        for l in range(4):
            for b in range(2):
                p = f"layer{l + 1}.{b}"
                y = cbr(cbr(x, groups[f"{p}.conv1"], True), groups[f"{p}.conv2"], False)
                idn = cbr(x, groups[f"{p}.downsample.0"], False) if f"{p}.downsample.0" in groups else x
                x = F.relu(y + idn)
        return x.mean(dim=(2, 3)) @ sd["fc.weight"].T + sd["fc.bias"]

    x = torch.from_numpy(random_input(n_images, H, W, 0, "normal"))
    with torch.no_grad():
        fwd(x[:2])
        t0 = time.perf_counter()
        fwd(x)
        dt = time.perf_counter() - t0
    return n_images / dt, cores, dt


def run_reference(args):
    """The CPU arm: each step is one oracle forward over a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 32
    for _ in range(args.warmup):
        cpu_oracle_images_per_s(4)
    times, cores = [], 1
    for _ in range(args.steps):
        _, cores, dt = cpu_oracle_images_per_s(sample)
        times.append(dt)
    mean = sum(times) / len(times)
    ips = sample / mean
    line = {
        "impl": "reference", "metric": METRIC, "value": ips, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "ResNet-18 inference, batch 256 of 3x224x224 ~N(0,1), seeded random-init weights "
                               f"(config 3); the CPU arm runs a bounded sample of {sample} images per step, fp32",
                   "global_batch": args.batch, "image": [3, H, W]},
        "cpu_baseline": {"value": ips, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{sample} images of 3x224x224 per step, oracle/nncv_oracle.cpp (a plain loop nest, no "
                                   "blocking) with OpenMP on every host core; the reference's own HostWParallel build "
                                   "needs MLIR/LLVM 18, absent here"},
        "e2e": {"value": ips, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _timed_loop(torch, flush, fn, min_ms=150.0, min_reps=7, max_reps=3000):
    """Median CUDA-event time of fn() on the current stream, L2 flushed before every call; repeats
    until about min_ms of kernel time has run so that clock samples fall inside the window."""
    fn()
    torch.cuda.synchronize()
    ts, total = [], 0.0
    while len(ts) < min_reps or (total < min_ms and len(ts) < max_reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
        total += ts[-1]
    return statistics.median(ts), len(ts)


def secondary_configs(torch, rt, flush, sampler, tf_peak):
    """The benchmark configs other than the headline one, on one GPU: GEMM sweep (config 1), 3x3
    stride-1 conv sweep at batch 32 (config 2), ResNet-18 fp32 N=1 @256 (config 0), ResNet-50 fp16
    (config 4).  Each entry: median ms, TFLOP/s (algorithmic), fraction of the tensor peak, and the
    clocks sampled while it ran."""
    from nncv_b200._lib import F16, F32, check, lib
    from nncv_b200.netspec import conv_macs
    from nncv_b200.split_params import random_state_dict, to_flat_array
    L = lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    out = {"gemm": [], "conv3x3_n32": [], "nets": [], "hbm_ops": []}

    def entry(ms, reps, flops, i0, **kw):
        tf = flops / ms / 1e9
        e = dict(kw, ms=round(ms, 5), reps=reps, tflops=round(tf, 2), frac=round(tf / tf_peak, 4),
                 clocks=sampler.window(i0, sampler.pos()) if sampler else None)
        return e

    for n in (512, 1024, 2048, 4096):
        for ab, name in ((F16, "f16 in / f32 acc"), (F32, "f32")):
            tdt = torch.float16 if ab == F16 else torch.float32
            A = (torch.rand((n, n), device="cuda") * 2 - 1).to(tdt)
            B = (torch.rand((n, n), device="cuda") * 2 - 1).to(tdt)
            C = torch.empty((n, n), device="cuda", dtype=torch.float32)
            for epi in (False, True):
                bias = torch.randn(n, device="cuda") if epi else None
                i0 = sampler.pos() if sampler else 0
                ms, reps = _timed_loop(torch, flush, lambda: check(L.nncv_b200_matmul(P(A), P(B), P(C), n, n, n, ab, F32, P(bias), int(epi), st)))
                out["gemm"].append(entry(ms, reps, 2.0 * n ** 3, i0, size=n, dtype=name, bias_relu=epi))
    for c, hw in ((64, 64), (128, 32), (256, 16), (512, 8)):
        n = 32
        w = (torch.randn((c, c, 3, 3)) * (2.0 / (9 * c)) ** 0.5).numpy().astype(np.float32)
        X = torch.randn((n, hw, hw, c), device="cuda", dtype=torch.float16)
        Y = torch.empty((n, hw, hw, c), device="cuda", dtype=torch.float16)
        sc = torch.rand(c, device="cuda") + 0.5
        sh = torch.randn(c, device="cuda") * 0.1
        h = L.nncv_b200_conv_create(w.ctypes.data, F32, c, c, 3, 3, 1, 1, F16, 2)
        if not h:
            continue
        try:
            call = lambda: check(L.nncv_b200_conv_run(h, P(X), P(Y), n, hw, hw, P(sc), P(sh), None, 1, st))
            call()
            torch.cuda.synchronize()
            # the entry point converts dense NHWC <-> the kernel's layout around the conv: time the conv
            # launch itself through the per-launch records
            i0 = sampler.pos() if sampler else 0
            rt.profile(True)
            t_end = time.perf_counter() + 0.15
            k = 0
            while k < 7 or (time.perf_counter() < t_end and k < 2000):
                flush.zero_()
                call()
                k += 1
            torch.cuda.synchronize()
            recs = [r for r in rt.profile_records() if r["kind"] in (2, 5, 7)]
            rt.profile(False)
            ms = statistics.median(r["ms"] for r in recs)
            out["conv3x3_n32"].append(entry(ms, len(recs), recs[0]["flops"], i0, c=c, hw=hw, batch=n, kernel_kind=recs[0]["kind"],
                                            note="fp16, fused scale/shift + ReLU; the conv launch alone"))
        finally:
            L.nncv_b200_conv_destroy(h)
    try:
        from nncv_b200 import sweeps
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):     # the sweep prints its own lines; this run prints one
            out["hbm_ops"] = sweeps.hbm_ops()
    except Exception as ex:
        out["hbm_ops"] = [{"error": str(ex)[:200]}]
    s = torch.cuda.current_stream().cuda_stream
    for depth, dt, n, hw, name in ((18, F32, 1, 256, "ResNet-18 fp32 N=1 @256 (config 0)"),
                                   (50, F16, 512, 224, "ResNet-50 fp16 N=512 @224 (config 4)")):
        np_dt = np.float32 if dt == F32 else np.float16
        blob = to_flat_array(depth, random_state_dict(depth, 0), np_dt).blob()
        try:
            rt.load_blob(f"resnet{depth}", blob, dt)
            x = torch.randn((n, 3, hw, hw), device="cuda").to(torch.float32 if dt == F32 else torch.float16)
            o = torch.empty((n, 1000), device="cuda", dtype=x.dtype)
            rt.forward_device(o, x, s)     # first call: tile timing, workspace
            torch.cuda.synchronize()
            i0 = sampler.pos() if sampler else 0
            ms, reps = _timed_loop(torch, flush, lambda: rt.forward_device(o, x, s), min_ms=200.0, min_reps=5)
            e = entry(ms, reps, 2.0 * conv_macs(depth, hw, hw) * n, i0, config=name, batch=n)
            e["images_per_s"] = round(n / ms * 1e3, 1)
            out["nets"].append(e)
            del x, o
        except Exception as ex:   # e.g. not enough free memory for batch 512 beside another tenant
            out["nets"].append({"config": name, "error": str(ex)[:200]})
        finally:
            rt.unload()
            torch.cuda.empty_cache()
    # MobileNetV3-small as nncv's fixture spells it (tests/Nets/MobileNetV3.mlir of the nncv tree), through the plan the importer
    # wrote from that module: fp16, batch 256 @224, seeded random weights
    try:
        name = "MobileNetV3-small fp16 N=256 @224 (imported plan of nncv's fixture)"
        text = open(os.path.join(ROOT, "tests", "golden", "mobilenetv3_from_mlir.plan")).read()
        blob, flops_per_image = _plan_blob_and_flops(text, 224, 224)
        n = 256
        rt.load_blob("plan:" + text, blob.astype(np.float16), F16)
        x = torch.randn((n, 3, 224, 224), device="cuda").to(torch.float16)
        o = torch.empty((n, 1000), device="cuda", dtype=x.dtype)
        rt.forward_device(o, x, s)
        torch.cuda.synchronize()
        i0 = sampler.pos() if sampler else 0
        ms, reps = _timed_loop(torch, flush, lambda: rt.forward_device(o, x, s), min_ms=200.0, min_reps=5)
        e = entry(ms, reps, flops_per_image * n, i0, config=name, batch=n)
        e["images_per_s"] = round(n / ms * 1e3, 1)
        e["note"] = "memory-bound network (0.11 GFLOP per image): images/s is the figure, the tensor-peak fraction is not a target"
        out["nets"].append(e)
        del x, o
    except Exception as ex:
        out["nets"].append({"config": name, "error": str(ex)[:200]})
    finally:
        rt.unload()
        torch.cuda.empty_cache()
    return out


def _plan_blob_and_flops(text, h, w):
    """Seeded parameters for a plan text (conv weights ~ N(0, 2/fan_in), batch-norm scale and variance in [0.5, 1.5], the
    rest small) and the multiply-add FLOPs of one image."""
    g = np.random.default_rng(0)
    total, nodes = 0, []
    for line in text.splitlines():
        t = line.split("#")[0].split()
        if not t or t[0] == "nncv_b200_plan":
            continue
        if t[0] == "params":
            total = int(t[1])
            continue
        nodes.append((t[0], {k: int(v) for k, v in (f.split("=") for f in t[1:])}))
    blob = (g.standard_normal(total) * 0.05).astype(np.float32)
    shape = {0: (h, w)}
    flops = 0.0
    for kind, f in nodes:
        ih, iw = shape.get(f["in"], (1, 1))
        if kind in ("conv", "dwconv"):
            cout = f.get("cout", f.get("c"))
            cin = 1 if kind == "dwconv" else f["cin"]
            k = f["k"]
            oh, ow = (ih + 2 * f["pad"] - k) // f["stride"] + 1, (iw + 2 * f["pad"] - k) // f["stride"] + 1
            nw = cout * cin * k * k
            blob[f["w"]:f["w"] + nw] = g.standard_normal(nw) * np.sqrt(2.0 / (cin * k * k))
            for role in ("gamma", "var"):
                if role in f:
                    blob[f[role]:f[role] + cout] = g.uniform(0.5, 1.5, cout)
            flops += 2.0 * nw * oh * ow
            shape[f["id"]] = (oh, ow)
        elif kind == "maxpool":
            shape[f["id"]] = ((ih + 2 * f["pad"] - f["k"]) // f["stride"] + 1, (iw + 2 * f["pad"] - f["k"]) // f["stride"] + 1)
        elif kind == "se":
            for wk, cnt in (("w1", f["c"] * f["cr"]), ("w2", f["c"] * f["cr"])):
                blob[f[wk]:f[wk] + cnt] = g.standard_normal(cnt) * np.sqrt(1.0 / f["c"])
            flops += 4.0 * f["c"] * f["cr"]
            shape[f["id"]] = (ih, iw)
        elif kind == "fc":
            cnt = f["cin"] * f["cout"]
            blob[f["w"]:f["w"] + cnt] = g.standard_normal(cnt) * np.sqrt(1.0 / f["cin"])
            flops += 2.0 * cnt
            shape[f["id"]] = (1, 1)
        else:
            shape[f["id"]] = (1, 1)
    return blob, flops


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nncv_b200 import runtime as rt
    from nncv_b200._lib import F16, lib
    from nncv_b200.netspec import conv_macs
    from nncv_b200.shard import gather_logits, shard_range
    from nncv_b200.split_params import random_state_dict, to_flat_array

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    B = args.batch
    lo, hi = shard_range(B, rank, world)
    nb = hi - lo

    # fp16 params blob (same seeded weights on every rank) -> library
    sd = random_state_dict(18, 0)
    blob = to_flat_array(18, sd, np.float16).blob()
    rt.load_blob("resnet18", blob, F16)

    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    x_host = torch.randn((max(nb, 1), 3, H, W), generator=g, dtype=torch.float32).to(torch.float16).pin_memory()
    out_host = torch.zeros((max(nb, 1), 1000), dtype=torch.float16).pin_memory()
    all_host = torch.zeros((B, 1000), dtype=torch.float16).pin_memory() if rank == 0 else None
    x_dev = x_host.cuda()
    out_dev = torch.zeros((max(nb, 1), 1000), device="cuda", dtype=torch.float16)
    flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)   # > 126 MB L2
    stream = torch.cuda.Stream()
    sptr = stream.cuda_stream

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    mids = []

    def step_device():
        if nb > 0:
            rt.forward_device(out_dev[:nb], x_dev[:nb], sptr)
        if world > 1:
            mid = torch.cuda.Event(enable_timing=True)
            mid.record(stream)
            mids.append(mid)
            gather_logits(out_dev[:nb], B)

    def step_host():
        if world == 1:
            rt.forward(out_host.numpy()[:nb], x_host.numpy()[:nb])   # _mlir_ciface_forward, host buffers both ways
            return
        # host images -> this step's logits on the device -> gather -> rank 0 copies the batch's logits out
        if nb > 0:
            rt.forward(out_dev[:nb], x_host.numpy()[:nb])
        full = gather_logits(out_dev[:nb], B)
        if rank == 0:
            all_host.copy_(full, non_blocking=True)
            stream.synchronize()

    def timed(step, k):
        """k steps, each bracketed by events on the launching stream, L2 flushed in between."""
        evs = []
        for _ in range(k):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            step()
            e1.record(stream)
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return evs

    with torch.cuda.stream(stream):
        rt.set_stream(sptr, True)
        sampler = ClockSampler(range(world)) if rank == 0 else None
        if sampler:
            sampler.start()
        for _ in range(max(args.warmup, 3)):
            step_device()
        if sampler:
            sampler.wait_ready()
        barrier()
        mids.clear()
        c0 = sampler.pos() if sampler else 0
        l0 = rt.launch_count()
        evs = timed(step_device, args.steps)
        launches = rt.launch_count() - l0
        c1 = sampler.pos() if sampler else 0
        ms_dev = sum(a.elapsed_time(b) for a, b in evs)
        ms_fwd = sum(a.elapsed_time(m) for (a, _), m in zip(evs, mids)) if world > 1 else ms_dev
        barrier()
        # The K timed steps last a few tens of milliseconds, shorter than a few sampling periods of
        # nvidia-smi: the same step, timed the same way, runs args.sustain more times so that the clock
        # record covers a timed region of about half a second.  The count is a constant: every rank
        # runs the same number of steps (they contain a collective).
        mids.clear()
        evs_s = timed(step_device, args.sustain)
        c2 = sampler.pos() if sampler else 0
        ms_sus = sum(a.elapsed_time(b) for a, b in evs_s) if args.sustain > 0 else 0.0
        barrier()
        for _ in range(max(args.warmup, 3)):
            step_host()
        barrier()
        c3 = sampler.pos() if sampler else 0
        evs_h = timed(step_host, args.steps)
        c4 = sampler.pos() if sampler else 0
        ms_e2e = sum(a.elapsed_time(b) for a, b in evs_h)
        barrier()
        status = lib().nncv_b200_device_status()
        if status != 0:
            raise SystemExit(f"device status after the timed regions: {lib().nncv_b200_last_error().decode()}")

        # per-kernel attribution of one step (events around every launch), after the timed regions
        prof = []
        if rank == 0 and nb > 0:
            rt.profile(True)
            reps = 5
            for _ in range(reps):
                flush.zero_()
                rt.forward_device(out_dev[:nb], x_dev[:nb], sptr)
            torch.cuda.synchronize()
            prof = rt.profile_records()
            rt.profile(False)

    if world > 1:
        t = torch.tensor([ms_dev, ms_e2e, ms_fwd, ms_sus], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e, ms_fwd, ms_sus = t.tolist()
        tl = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(tl)
        launches = int(tl.item())

    if rank == 0:
        tf_peak, tf_sus, hbm_peak, which = peaks()
        conv_kinds = (0, 2, 4, 5, 7)
        conv = [r for r in prof if r["kind"] in conv_kinds]
        conv_ms = sum(r["ms"] for r in conv)
        conv_fl = sum(r["flops"] for r in conv)
        n_conv = len(conv)
        other_ms = sum(r["ms"] for r in prof if r["kind"] not in conv_kinds)
        gflop_img = 2 * conv_macs(18, H, W) / 1e9
        ms_step = ms_dev / args.steps
        ms_fwd_step = ms_fwd / args.steps
        # rank 0's own share of the FLOPs over the forward part of its timed step
        achieved = nb * gflop_img / ms_fwd_step if ms_fwd_step > 0 else None    # GFLOP / ms = TFLOP/s
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "igemm_traffic.json")) as f:
                tj = json.load(f)
            # measured DRAM bytes per algorithmic byte of the conv launches, scaled to one launch
            alg_bytes = sum(r["bytes"] for r in conv) / max(n_conv, 1)
            traffic = tj["dram_bytes_per_algorithmic_byte"] * alg_bytes
        except Exception:
            pass
        ips = B * args.steps / (ms_dev * 1e-3)
        e2e = B * args.steps / (ms_e2e * 1e-3)
        clocks = None
        if sampler:
            clocks = sampler.window(c0, c2)
            clocks["timed_steps_window"] = sampler.window(c0, c1)
            clocks["sustained_window"] = sampler.window(c1, c2)
            clocks["e2e_window"] = sampler.window(c3, c4)
            clocks["note"] = ("sampled every 20 ms during the K timed steps and the sustained run of "
                              f"{args.sustain} further steps timed the same way")
        line = {
            "metric": METRIC, "value": ips, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "ResNet-18 fp16 inference, batch 256 of 3x224x224 ~N(0,1), seeded random-init "
                                   "weights, batch-sharded over the ranks, logits gathered to rank 0 (config 3)",
                       "global_batch": B, "per_gpu_batch": nb, "image": [3, H, W], "parallelism": f"dp{world}",
                       "l2": "256 MiB buffer rewritten between timed steps (L2 flush)",
                       "gflop_per_image": gflop_img},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(B * 3 * H * W * 2),
                    "d2h_bytes_per_step": int(B * 1000 * 2), "ms_per_step": ms_e2e / args.steps,
                    "api": "_mlir_ciface_forward with pinned host input" +
                           ("; logits to pinned host memory" if world == 1 else
                            "; this step's logits gathered on the device over NCCL, rank 0 copies the batch's logits to pinned host memory")},
            "gpu_launches": launches,
            "clocks": clocks,
            "split": {"forward_ms_per_step": ms_fwd_step, "gather_ms_per_step": ms_step - ms_fwd_step,
                      "note": "max over ranks of each rank's own event pairs"},
            "sustained": ({"steps": args.sustain, "ms_per_step": ms_sus / args.sustain,
                           "value": B * args.sustain / (ms_sus * 1e-3)} if args.sustain > 0 else None),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s",
                         "frac": (achieved / tf_peak) if achieved else None, "traffic": traffic,
                         "peak_source": f"{which} burst bf16/fp16 dense; sustained {tf_sus}",
                         "kernel": "all launches of one step on rank 0 (stem_pool_kernel + conv3x3_kernel + conv3x3_pair_kernel + "
                                   "tconv_kernel + helpers): algorithmic conv/FC FLOPs of rank 0's images / its forward "
                                   "time inside the timed region",
                         "per_launch_pass": {
                             "note": "separate pass after the timed region, CUDA events around every launch (serialised, "
                                     "so the sum exceeds the step time); conv/FC launches only in frac",
                             "launches_per_step": n_conv // 5 if n_conv else 0,
                             "conv_ms_per_step": conv_ms / 5 if conv_ms else None,
                             "other_kernels_ms_per_step": other_ms / 5 if prof else None,
                             "achieved": (conv_fl / (conv_ms * 1e-3) / 1e12) if conv_ms > 0 else None,
                             "frac": (conv_fl / (conv_ms * 1e-3) / 1e12 / tf_peak) if conv_ms > 0 else None}},
        }
        if args.layers and prof:
            with open(args.layers, "w") as f:
                json.dump(prof[: len(prof) // 5], f)
        rt.unload()
        if world == 1:
            cpu_ips, cores, cpu_s = cpu_oracle_images_per_s(64)
            line["cpu_baseline"] = {"value": cpu_ips, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"64 images of 3x224x224, fp32, oracle/nncv_oracle.cpp (a plain loop nest) with OpenMP "
                                              f"on every host core ({cpu_s:.2f} s); the reference's HostWParallel build is unavailable"}
            try:
                t_ips, t_cores, t_s = cpu_torch_images_per_s(64)
                line["cpu_baseline"]["torch_cpu"] = {"value": t_ips, "unit": UNIT, "cores": t_cores,
                                                     "sample": f"the same 64 images on PyTorch CPU operators (oneDNN), fp32 ({t_s:.2f} s); context only"}
            except Exception as ex:
                line["cpu_baseline"]["torch_cpu"] = {"error": str(ex)[:200]}
            if not args.no_secondary:
                with torch.cuda.stream(stream):
                    line["secondary"] = secondary_configs(torch, rt, flush, sampler, tf_peak)
        if sampler:
            sampler.stop()
        print(json.dumps(line), flush=True)
    else:
        rt.unload()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="global batch (the benchmark config uses 256)")
    ap.add_argument("--layers", default="", metavar="FILE",
                    help="also write the per-launch records of one step of the attribution pass to FILE as JSON")
    ap.add_argument("--sustain", type=int, default=300,
                    help="further steps timed the same way after the K timed ones, so that clock samples fall into a timed "
                         "region (0 for a short run under a profiler); the same for every rank")
    ap.add_argument("--no-secondary", action="store_true", help="skip the other benchmark configs (N = 1 only measures them)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
