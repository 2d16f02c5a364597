#!/usr/bin/env python
"""Headline benchmark: VGG-16 (or SqueezeNet v1.1) fp32 inference throughput in images/s through the
deepRacin C API of libdeepracin.so, batch 64 per GPU, batch-sharded replicas across GPUs.

  python bench.py --gpus N --steps K --warmup W                    this library (CUDA, sm_100a)
  python bench.py --impl reference --gpus N --steps K --warmup W   the reference's own kernels on the host cores

One JSON line on stdout (rank 0).  `value` is whole-job images/s with the inputs already resident in
HBM (CUDA events on the library's stream around K x dR_apply, max over ranks); `e2e` is the same
metric with the pinned-host -> device copy of every step's images and the device -> host read of its
class probabilities inside the timed region.  Inputs are synthetic: uniform[0,255] - 128 images,
seeded He-normal weights of the named architecture.  Activations of one step (GBs) exceed the 126 MB
L2 many times over, so no extra L2 flush is needed between steps.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

VGG_CONVS = [(3, 64, 224), (64, 64, 224), (64, 128, 112), (128, 128, 112), (128, 256, 56), (256, 256, 56), (256, 256, 56),
             (256, 512, 28), (512, 512, 28), (512, 512, 28), (512, 512, 14), (512, 512, 14), (512, 512, 14)]
VGG_FCS = [(25088, 4096), (4096, 4096), (4096, 1000)]


def vgg_flops_per_image():
    conv = sum(2 * 9 * ci * co * hw * hw for ci, co, hw in VGG_CONVS)
    fc = sum(2 * a * b for a, b in VGG_FCS)
    return conv, fc


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                c = [t.strip() for t in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    sm.append(float(c[1]))
                    smax.append(float(c[2]))
                except ValueError:
                    continue
                for nm, v in zip(names, c[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
        os.remove(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons), "samples": len(sm)}


def build_net(dr, nets, env, net, batch, math, size):
    g = env.create_graph("HWC")
    g.batch = batch
    g.math = math
    if net == "vgg16":
        x, out = nets.vgg16(g, size=size)
    else:
        x, out = nets.squeezenet11(g, size=size)
    dr.mark_as_output(out)
    dr.lib.dR_setInterfaceLayout(g.ptr, 1)     # synthetic inputs are N-HWC: no layout conversion in the timed region
    g.feed_overlap = True                      # e2e: the next batch's H2D copy runs on a second stream under the current batch's kernels
    return g, x, out


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    from deepracin_b200 import replicas
    dist = replicas.init("nccl") if world > 1 else None
    import deepracin_b200 as dr
    import nets

    lib = dr.lib
    size = 224
    batch = args.batch
    with dr.Environment(device=local) as env:
        g, x, out = build_net(dr, nets, env, args.net, batch, args.math, size)
        g.autotune = bool(args.autotune)
        dr.prepare(g)
        nclass = out.out_shape[0] * out.out_shape[1] * out.out_shape[2]
        in_floats = batch * size * size * 3
        out_floats = batch * nclass
        pin_in = lib.dR_allocPinned(in_floats * 4)
        pin_out = lib.dR_allocPinned(out_floats * 4)
        host_in = np.ctypeslib.as_array((np.ctypeslib.ctypes.c_float * in_floats).from_address(pin_in))
        host_out = np.ctypeslib.as_array((np.ctypeslib.ctypes.c_float * out_floats).from_address(pin_out))
        host_in[:] = nets.synthetic_images("bench_rank%d" % rank, batch, size).reshape(-1)
        lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in, in_floats)
        lib.dR_synchronize(g.ptr)

        def barrier():
            lib.dR_synchronize(g.ptr)
            if dist is not None:
                import torch
                dist.barrier()
                torch.cuda.synchronize()

        def reduce_max(v):
            return replicas.max_over_ranks(dist, v, cuda=True)

        for _ in range(args.warmup):
            if not lib.dR_apply(g.ptr):
                raise RuntimeError("dR_apply failed")
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        # ---- device-resident throughput: K x dR_apply between events on the library's stream
        lib.dR_timerStart(g.ptr)
        for _ in range(args.steps):
            lib.dR_apply(g.ptr)
        ms = lib.dR_timerStopMs(g.ptr)
        barrier()
        ms = reduce_max(ms)
        clocks = sampler.stop() if rank == 0 else None
        # ---- end to end: pinned host -> device, apply, device -> host, every step
        for _ in range(2):
            lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in, in_floats)
            lib.dR_apply(g.ptr)
            lib.dR_fetchOutputAsync(g.ptr, 0, pin_out, out_floats)
        barrier()
        lib.dR_timerStart(g.ptr)
        for _ in range(args.steps):
            lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in, in_floats)
            lib.dR_apply(g.ptr)
            lib.dR_fetchOutputAsync(g.ptr, 0, pin_out, out_floats)
        ms_e2e = lib.dR_timerStopMs(g.ptr)
        barrier()
        ms_e2e = reduce_max(ms_e2e)
        status = lib.dR_getDeviceStatus(g.ptr)
        probs = host_out.reshape(batch, nclass).copy()
        all_probs = replicas.gather_outputs(dist, probs, batch * world, cuda=True)      # outputs of every replica, in image order
        launches_per_apply = lib.dR_getLaunchCount(g.ptr)

        line = None
        if rank == 0:
            peaks = measured_peaks()
            # per-node kernel times of one profiled apply -> roofline of the dominant (convolution) kernel
            lib.dR_synchronize(g.ptr)
            prof = per_node_profile(dr, lib, g)
            conv_flops, fc_flops = vgg_flops_per_image()
            conv_times = [t for kind, t in prof if kind == "conv"]
            conv_ms = sum(conv_times)
            n_conv = len(conv_times)
            tensor = args.math == "tf32"
            peak = peaks["bf16_sustained"] / 2.0 if tensor else 74.4
            peak_src = ("%s bf16 sustained / 2 (TF32 issues at half the bf16 rate; no TF32 figure in MEASURED_PEAKS.json)" % peaks["source"]) if tensor \
                else "nominal FP32 FFMA 148 SM x 128 lanes x 2 x 1.965 GHz"
            aggregate = conv_flops * batch / (conv_ms * 1e-3) / 1e12 if (args.net == "vgg16" and conv_ms > 0) else None
            roof = {"bound": "tensor", "achieved": aggregate, "peak": peak, "unit": "TFLOP/s", "frac": (aggregate / peak) if aggregate else None,
                    "traffic": None, "kernel": "convolution (%d launches, aggregate)" % n_conv, "peak_source": peak_src}
            if args.net == "vgg16" and n_conv == 13 and conv_times[5] > 0:
                # dominant kernel: the 128..512-channel 3x3 layers (k_umma_conv_swap in TF32 mode); measured live on conv3_2
                ci, co, hw = VGG_CONVS[5]
                one = 2.0 * 9 * ci * co * hw * hw * batch / (conv_times[5] * 1e-3) / 1e12
                roof = {"bound": "tensor", "achieved": one, "peak": peak, "unit": "TFLOP/s", "frac": one / peak,
                        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this layer at batch 64 (ncu capture, see profiles/)
                        "traffic": 368.8e6 if (tensor and batch == 64) else None,
                        "algorithmic_bytes": 4.0 * (batch * hw * hw * (ci + co) + 9 * ci * co),
                        "kernel": "conv3_2 256->256 @56x56 (%s), %.4f ms per launch" % ("k_umma_conv_swap" if tensor else "FP32 variant chosen at prepare", conv_times[5]),
                        "peak_source": peak_src}
            roof["conv_aggregate"] = {"tflops": aggregate, "frac": (aggregate / peak) if aggregate else None, "launches": n_conv, "ms": round(conv_ms, 4)}
            roof["ms_by_kind"] = {k: round(sum(t for kk, t in prof if kk == k), 4) for k in sorted(set(k for k, _ in prof))}
            roof["ms_per_layer"] = [[k, round(t, 4)] for k, t in prof if t > 0]        # launch order; fused / elided nodes launch nothing
            achieved = aggregate
            value = batch * world * args.steps / (ms * 1e-3)
            e2e = batch * world * args.steps / (ms_e2e * 1e-3)
            line = {
                "metric": "images/sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "tf32" if tensor else "f32", "data": "synthetic",
                "config": {"workload": "%s fp32 inference, batch %d per GPU, 224x224x3 uniform[0,255]-128 inputs, seeded He-normal weights; "
                                       "inputs larger than L2 (no flush)" % ("VGG-16" if args.net == "vgg16" else "SqueezeNet v1.1 (reference example graph)", batch),
                           "global_batch": batch * world, "parallelism": "replicas x%d (batch sharded, no collective)" % world,
                           "math": args.math, "autotune": bool(args.autotune)},
                "e2e": {"value": e2e, "unit": "images/s", "h2d_bytes_per_step": in_floats * 4, "d2h_bytes_per_step": out_floats * 4,
                        "ms_per_step": ms_e2e / args.steps},
                "gpu_launches": launches_per_apply * args.steps,
                "clocks": clocks, "roofline": roof,
                "conv_tflops": achieved, "device_status": status,
                "top1_sample": [int(v) for v in probs.argmax(1)[:4]], "gathered_outputs": list(all_probs.shape),
            }
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline(args.net, budget_s=args.cpu_budget)
        lib.dR_freePinned(pin_in)
        lib.dR_freePinned(pin_out)
    replicas.finish(dist)
    if line is not None:
        print(json.dumps(line))


def per_node_profile(dr, lib, g):
    """One apply with per-kernel events; returns [(kind, ms)] per node."""
    res = []
    lib.dR_config(g.ptr, b"", 1, 0, 1, 0, (g.env.model_path).encode())
    # the C library prints a summary line per apply when profiling; keep stdout clean for the JSON line
    fd = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    sys.stdout.flush()
    os.dup2(devnull, 1)
    try:
        lib.dR_apply(g.ptr)
        lib.dR_synchronize(g.ptr)
    finally:
        os.dup2(fd, 1)
        os.close(fd)
        os.close(devnull)
    for node in g.nodes:
        kind = {"Conv2D": "conv", "FullyConnected": "fc", "Pooling": "pool", "Softmax": "softmax"}.get(node.desc, "other")
        res.append((kind, lib.dR_getNodeGpuMs(node.ptr)))
    lib.dR_config(g.ptr, b"", 1, 0, 0, 0, (g.env.model_path).encode())
    return res


# ------------------------------------------------------------------ CPU side (oracle is the checker / baseline only)
def _ref_vgg_layers():
    import cases
    layers = []
    for i, (ci, co, hw) in enumerate(VGG_CONVS):
        x, w, b = cases.conv_case("cpu_vgg_conv%d" % i, 1, ci, co, hw, hw, 3)
        layers.append(("conv", x, w, b, 2 * 9 * ci * co * hw * hw))
    for i, (a, bb) in enumerate(VGG_FCS):
        g = cases.rng("cpu_vgg_fc%d" % i)
        x = g.standard_normal((1, a, 1, 1), dtype=np.float32)
        w = g.standard_normal((a, bb), dtype=np.float32) * np.float32(np.sqrt(2.0 / a))
        layers.append(("fc", x, w, np.zeros(bb, np.float32), 2 * a * bb))
    return layers


def cpu_step(oracle, layers, use_ref):
    for kind, x, w, b, _ in layers:
        if kind == "conv":
            if use_ref:
                oracle.ref_conv2d_winograd(x, w, b, 1)
            else:
                oracle.conv2d_winograd(x, w, b, 1)
        else:
            if use_ref:
                oracle.ref_fc(x, w, b, 1)
            else:
                oracle.fc(x, w, b, 1)


def choose_cpu_sample(oracle, layers, use_ref, steps, budget_s):
    """Largest sample (whole image, or a FLOP-weighted subset of its layers) whose `steps` repetitions fit the budget."""
    total = sum(l[4] for l in layers)
    t0 = time.time()
    cpu_step(oracle, layers, use_ref)
    t_full = time.time() - t0
    if t_full * steps <= budget_s:
        return layers, 1.0, "1 image through all 13 conv + 3 FC layers per step"
    subset = [layers[i] for i in (1, 5, 8, 11)]     # one layer of each resolution: conv1_2, conv3_2, conv4_2, conv5_2
    frac = sum(l[4] for l in subset) / total
    if t_full * frac * steps <= budget_s:
        return subset, frac, "1 image through conv1_2, conv3_2, conv4_2, conv5_2 per step (%.0f%% of the image's FLOPs), scaled by FLOPs" % (100 * frac)
    subset = [layers[5]]
    frac = subset[0][4] / total
    return subset, frac, "1 image through conv3_2 per step (%.0f%% of the image's FLOPs), scaled by FLOPs" % (100 * frac)


def cpu_baseline(net, budget_s=20.0, steps=3):
    import oracle
    from oracle import build_oracle
    build_oracle.build_restatement()
    use_ref = oracle.ref_available()
    cores = oracle.set_threads()
    layers = _ref_vgg_layers()
    sample, frac, what = choose_cpu_sample(oracle, layers, use_ref, steps + 1, budget_s)
    t0 = time.time()
    for _ in range(steps):
        cpu_step(oracle, sample, use_ref)
    dt = (time.time() - t0) / steps
    return {"value": frac / dt, "unit": "images/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": what + "; VGG-16 layer shapes; " + ("reference OpenCL C kernels compiled as C (Winograd + FC), OpenMP over work-groups"
                                                          if use_ref else "C restatement of the reference's Winograd arithmetic")}


def run_reference(args):
    """The reference's own CPU-runnable implementation of the path: its kernel sources compiled as C
    (oracle/_ref), all host cores.  PoCL / any OpenCL runtime is unavailable on this box."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from oracle import build_oracle
    build_oracle.build_restatement()
    use_ref = oracle.ref_available()
    cores = oracle.set_threads()
    layers = _ref_vgg_layers()
    sample, frac, what = choose_cpu_sample(oracle, layers, use_ref, args.steps + args.warmup + 1, 170.0)
    for _ in range(args.warmup):
        cpu_step(oracle, sample, use_ref)
    t0 = time.time()
    for _ in range(args.steps):
        cpu_step(oracle, sample, use_ref)
    dt = time.time() - t0
    value = frac * args.steps / dt
    kind = "reference" if use_ref else "port"
    sample_txt = what + "; " + ("reference OpenCL C kernels compiled as C, OpenMP over work-groups" if use_ref else "C restatement (port)")
    line = {"impl": "reference", "metric": "images/sec", "value": value, "unit": "images/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "VGG-16 fp32 inference, batch 64 per GPU, 224x224x3 inputs (CPU arm: bounded sample per step)",
                       "global_batch": 64, "parallelism": "host cores"},
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample_txt},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--net", default="vgg16", choices=["vgg16", "squeezenet"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--math", default=os.environ.get("DR_BENCH_MATH", "tf32"), choices=["fp32", "tf32"])
    ap.add_argument("--autotune", type=int, default=-1, help="time conv variants at prepare; default: only in fp32 mode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.autotune < 0:
        args.autotune = 1 if args.math == "fp32" else 0
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
