#!/usr/bin/env python
"""Benchmark of the compiled-forward hot path: ResNet-18 fp16 inference, batch 256 of 3x224x224.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

One "step" is one forward over the (global) batch, sharded by contiguous image ranges over N
ranks (one process per GPU, launched by torchrun for N > 1), logits gathered to rank 0.
  value : images/s with the input already in HBM (nncv_b200_forward_device), CUDA events on the
          launching stream, an L2 flush between steps, max over ranks.
  e2e   : images/s through `_mlir_ciface_forward` with pinned HOST buffers: the host->device
          copy of the images and the device->host copy of the logits are inside the timed region.
  roofline : conv/GEMM (tcgen05 implicit-GEMM) launches of one step, timed one by one with CUDA
          events: algorithmic direct-convolution FLOPs / summed device time, vs the measured
          dense bf16/fp16 tensor peak.
  cpu_baseline : the CPU oracle (a port of the reference's linalg graph; the reference's own
          HostWParallel build needs an MLIR/LLVM toolchain that is absent) on the host cores,
          on a bounded sample of images.
--impl reference times that CPU path alone (rank 0 only).
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
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
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpus):
        self.gpus = set(gpus)
        self.proc = None

    def start(self):
        """Starts nvidia-smi and a thread that collects its lines (NVML start-up can take longer than a
        short timed region, so callers start it before the warm-up and wait for the first sample)."""
        import threading
        self.lines = []
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

    def mark(self):
        """Samples before this point (start-up, warm-up) are dropped."""
        self.skip = len(getattr(self, "lines", []))

    def count(self):
        return len(getattr(self, "lines", [])) - getattr(self, "skip", 0)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.thread.join(timeout=2)
        out = "".join(self.lines[getattr(self, "skip", 0):])
        sm, smax, reasons = [], [], set()
        for line in out.splitlines():
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
        # samples under load: the upper half of the clock samples (idle samples sit at the floor)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons), "samples": len(sm)}


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
                         "sample": f"{sample} images of 3x224x224 per step, oracle/nncv_oracle.cpp with OpenMP on every "
                                   "host core; the reference's own HostWParallel build needs MLIR/LLVM 18, absent here"},
        "e2e": {"value": ips, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nncv_b200 import runtime as rt
    from nncv_b200._lib import F16
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

    def step_device():
        if nb > 0:
            rt.forward_device(out_dev[:nb], x_dev[:nb], sptr)
        if world > 1:
            gather_logits(out_dev[:nb], B)

    def step_host():
        if nb > 0:
            rt.forward(out_host.numpy()[:nb], x_host.numpy()[:nb])   # _mlir_ciface_forward, host buffers
        if world > 1:
            gather_logits(out_dev[:nb], B)

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
        return sum(a.elapsed_time(b) for a, b in evs)

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
        if sampler:
            sampler.mark()
        l0 = rt.launch_count()
        ms_dev = timed(step_device, args.steps)
        launches = rt.launch_count() - l0
        barrier()
        for _ in range(max(args.warmup, 3)):
            step_host()
        barrier()
        ms_e2e = timed(step_host, args.steps)
        barrier()
        # Timed regions shorter than a few sampling periods (20 ms each) leave too few clock samples:
        # keep running the same device step, untimed, for a while.  The number of extra steps depends
        # on the arguments only, never on a rank's own timings: every rank must run the same number
        # of steps, they contain a collective.
        n_extra = 0 if args.steps >= 200 else 200
        for _ in range(n_extra):
            step_device()
        torch.cuda.synchronize()
        barrier()
        clocks = sampler.stop() if sampler else None
        if clocks is not None:
            clocks["extra_untimed_steps_sampled"] = n_extra

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
        t = torch.tensor([ms_dev, ms_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e = t.tolist()
        tl = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(tl)
        launches = int(tl.item())

    if rank == 0:
        tf_peak, tf_sus, hbm_peak, which = peaks()
        conv = [r for r in prof if r["kind"] in (0, 2, 4, 5, 7)]
        conv_ms = sum(r["ms"] for r in conv)
        conv_fl = sum(r["flops"] for r in conv)
        n_conv = len(conv)
        other_ms = sum(r["ms"] for r in prof if r["kind"] not in (0, 2, 4, 5, 7))
        achieved = conv_fl / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else None
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
        cpu_ips, cores, cpu_s = cpu_oracle_images_per_s(64) if world == 1 else (None, None, None)
        line = {
            "metric": METRIC, "value": ips, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "ResNet-18 fp16 inference, batch 256 of 3x224x224 ~N(0,1), seeded random-init "
                                   "weights, batch-sharded over the ranks, logits gathered to rank 0 (config 3)",
                       "global_batch": B, "per_gpu_batch": nb, "image": [3, H, W], "parallelism": f"dp{world}",
                       "l2": "256 MiB buffer rewritten between timed steps (L2 flush)",
                       "gflop_per_image": 2 * conv_macs(18, H, W) / 1e9},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(B * 3 * H * W * 2),
                    "d2h_bytes_per_step": int(B * 1000 * 2), "ms_per_step": ms_e2e / args.steps,
                    "api": "_mlir_ciface_forward with pinned host buffers"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s",
                         "frac": (achieved / tf_peak) if achieved else None, "traffic": traffic,
                         "peak_source": f"{which} burst bf16/fp16 dense; sustained {tf_sus}",
                         "kernel": "stem_pool_kernel + conv3x3_kernel + conv3x3_pair_kernel + tconv_kernel (all tcgen05 conv/FC launches of one step, rank 0)",
                         "launches_per_step": n_conv // 5 if n_conv else 0,
                         "conv_ms_per_step": conv_ms / 5 if conv_ms else None,
                         "other_kernels_ms_per_step": other_ms / 5 if prof else None},
        }
        if cpu_ips is not None:
            line["cpu_baseline"] = {"value": cpu_ips, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"64 images of 3x224x224, fp32, oracle/nncv_oracle.cpp with OpenMP on every host core "
                                              f"({cpu_s:.2f} s); the reference's HostWParallel build is unavailable"}
        if args.layers and prof:
            per = {}
            for i, r in enumerate(prof[: len(prof) // 5]):
                per[i] = r
            os.makedirs(os.path.join(ROOT, "gpurun_out"), exist_ok=True)
            with open(os.path.join(ROOT, "gpurun_out", "layers.json"), "w") as f:
                json.dump(prof, f)
        print(json.dumps(line), flush=True)
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
    ap.add_argument("--layers", action="store_true", help="also dump the per-launch records of the profiling pass as JSON into the run's output folder")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
