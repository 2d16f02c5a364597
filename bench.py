#!/usr/bin/env python
"""Headline benchmark: VGG-16 (and SqueezeNet v1.1) inference throughput in images/s through the deepRacin C API of
libdeepracin.so, batch 64 per GPU, batch-sharded replicas across GPUs.

  python bench.py --gpus N --steps K --warmup W                    this library (CUDA, sm_100a)
  python bench.py --impl reference --gpus N --steps K --warmup W   the reference's own kernels on the host cores

One JSON line on stdout (rank 0).  The headline (`value`, `e2e`, `roofline`) is VGG-16 at batch 64 per GPU in the TF32
tensor-core class (fp32 storage, TF32 operands, FP32 accumulation; tolerance 3e-3 per layer).  `value` is whole-job
images/s with the inputs already resident in HBM (CUDA events on the library's stream around K x dR_apply, max over
ranks); `e2e` is the same metric with the pinned-host -> device copy of every step's images and the device -> host read
of its class probabilities inside the timed region.  The same line carries, as objects of their own:

  fp32_exact   VGG-16 batch 64 in the reference's own arithmetic (FP32 FFMA kernels, tolerance 1e-4 per layer)
  fp32_accurate_tensor  VGG-16 batch 64 in math mode fp32x3: FP32-class error bound from three TF32 tensor-core passes per product
  e2e_u8       the headline's end-to-end loop fed with 8-bit image samples (dR_feedDataU8Async: a quarter of the host-link bytes)
  squeezenet   SqueezeNet v1.1 (the reference's example graph) at batch 64 in the headline's class and in FP32 mode (every N), and at batch 1 (N = 1)
  sustained    >= 3 s of back-to-back dR_apply with the clock sampler running (N = 1)
  e2e_dropin   the reference-shaped blocking calls: dR_feedData ([C][H][W], pageable host memory) + dR_apply +
               dR_downloadArray, as examples/vgg16/vgg_deployed.c:141-166 makes them (N = 1)
  tf32_yardstick  a TF32 torch.matmul 8192^3, burst and 4 s back to back: a library GEMM as a yardstick for the roofline's
               denominator, never part of the measured path (N = 1)
  cpu_baseline the reference's kernels compiled as C on the host cores (N = 1)

Inputs are synthetic: uniform[0,255] - 128 images, seeded He-normal weights of the named architecture.  Activations of
one step (GBs) exceed the 126 MB L2 many times over, so no extra L2 flush is needed between steps.
"""
import argparse
import ctypes
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
VGG_POOL_AFTER = (1, 3, 6, 9, 12)
VGG_FCS = [(25088, 4096), (4096, 4096), (4096, 1000)]
SQUEEZENET_CONV_FLOPS = 0.905e9     # per image, the reference's example graph (conv1 at stride 1)
FFMA_PEAK_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12        # 74.4 TFLOP/s
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch, from the ncu capture summarised in the named file
NCU_TRAFFIC = {("tf32", 64): (368.8e6, "profiles/k_umma_conv_swap_256to256_56x56_b64.md")}


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
    """nvidia-smi clock / power / throttle-reason samples during a timed region (read-only queries)."""
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
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                c = [t.strip() for t in line.split(",")]
                if len(c) < 9:
                    continue
                try:
                    sm.append(float(c[1]))
                    smax.append(float(c[2]))
                    power.append(float(c[3]))
                except ValueError:
                    continue
                for nm, v in zip(names, c[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
        os.remove(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": float(max(power))}


class Ctx:
    """Process-wide pieces of one benchmark run: rank layout, the library, barrier and max-over-ranks."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        from deepracin_b200 import replicas
        self.replicas = replicas
        self.dist = replicas.init("nccl") if self.world > 1 else None
        import deepracin_b200 as dr
        import nets
        self.dr, self.nets, self.lib = dr, nets, dr.lib

    def barrier(self, g):
        self.lib.dR_synchronize(g.ptr)
        if self.dist is not None:
            import torch
            self.dist.barrier()
            torch.cuda.synchronize()

    def reduce_max(self, v):
        return self.replicas.max_over_ranks(self.dist, v, cuda=True)


def check(ok, what):
    if not ok:
        raise RuntimeError(what + " failed")


def measure(ctx, net, math, batch, steps, warmup, overlap=True, cuda_graph=False, autotune=False, sampler=None, want_profile=False, min_seconds=0.0):
    """Builds `net`, prepares it, and times `steps` x dR_apply device-resident and end to end (async pinned copies).
    Every rank runs it; times are the max over ranks.  Returns a dict (rank 0 adds the per-node profile when asked)."""
    dr, nets, lib = ctx.dr, ctx.nets, ctx.lib
    size = 224
    with dr.Environment(device=ctx.local) as env:
        g = env.create_graph("HWC")
        g.batch = batch
        g.math = math
        g.autotune = autotune
        g.cuda_graph = cuda_graph
        x, out = nets.vgg16(g, size=size) if net == "vgg16" else nets.squeezenet11(g, size=size)
        dr.mark_as_output(out)
        lib.dR_setInterfaceLayout(g.ptr, 1)         # synthetic inputs are N-HWC: no layout conversion in the timed region
        g.feed_overlap = overlap and not cuda_graph  # e2e: the next batch's H2D copy runs on a second stream under this batch's kernels
        dr.prepare(g)
        nclass = out.out_shape[0] * out.out_shape[1] * out.out_shape[2]
        in_floats, out_floats = batch * size * size * 3, batch * nclass
        pin_in, pin_out = lib.dR_allocPinned(in_floats * 4), lib.dR_allocPinned(out_floats * 4)
        host_in = np.ctypeslib.as_array((ctypes.c_float * in_floats).from_address(pin_in))
        host_out = np.ctypeslib.as_array((ctypes.c_float * out_floats).from_address(pin_out))
        host_in[:] = nets.synthetic_images("bench_rank%d" % ctx.rank, batch, size).reshape(-1)
        check(lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in, in_floats), "dR_feedDataAsync")
        lib.dR_synchronize(g.ptr)
        for _ in range(warmup):
            check(lib.dR_apply(g.ptr), "dR_apply")
        ctx.barrier(g)
        if sampler is not None and ctx.rank == 0:
            sampler.start()
        # ---- device-resident: K x dR_apply between events on the library's stream
        lib.dR_timerStart(g.ptr)
        ok = True
        for _ in range(steps):
            ok &= bool(lib.dR_apply(g.ptr))
        ms = lib.dR_timerStopMs(g.ptr)
        check(ok and ms > 0, "dR_apply (timed)")
        ctx.barrier(g)
        ms = ctx.reduce_max(ms)
        clocks = sampler.stop() if (sampler is not None and ctx.rank == 0) else None
        # ---- end to end: pinned host -> device, apply, device -> host, every step
        for _ in range(2):
            ok &= bool(lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in, in_floats)) and bool(lib.dR_apply(g.ptr)) and bool(lib.dR_fetchOutputAsync(g.ptr, 0, pin_out, out_floats))
        ctx.barrier(g)
        lib.dR_timerStart(g.ptr)
        for _ in range(steps):
            ok &= bool(lib.dR_feedDataAsync(g.ptr, x.ptr, pin_in, in_floats)) and bool(lib.dR_apply(g.ptr)) and bool(lib.dR_fetchOutputAsync(g.ptr, 0, pin_out, out_floats))
        ms_e2e = lib.dR_timerStopMs(g.ptr)
        check(ok and ms_e2e > 0, "feed / apply / fetch (timed)")
        ctx.barrier(g)
        ms_e2e = ctx.reduce_max(ms_e2e)
        probs = host_out.reshape(batch, nclass).copy()
        # ---- end to end from 8-bit samples (decoded image bytes): a quarter of the bytes cross the host link, cast on the device
        pin_u8 = lib.dR_allocPinned(in_floats)
        host_u8 = np.ctypeslib.as_array((ctypes.c_uint8 * in_floats).from_address(pin_u8))
        host_u8[:] = np.random.default_rng(1234 + ctx.rank).integers(0, 256, size=in_floats, dtype=np.uint8)
        for _ in range(2):
            ok &= bool(lib.dR_feedDataU8Async(g.ptr, x.ptr, pin_u8, in_floats)) and bool(lib.dR_apply(g.ptr)) and bool(lib.dR_fetchOutputAsync(g.ptr, 0, pin_out, out_floats))
        ctx.barrier(g)
        lib.dR_timerStart(g.ptr)
        for _ in range(steps):
            ok &= bool(lib.dR_feedDataU8Async(g.ptr, x.ptr, pin_u8, in_floats)) and bool(lib.dR_apply(g.ptr)) and bool(lib.dR_fetchOutputAsync(g.ptr, 0, pin_out, out_floats))
        ms_u8 = lib.dR_timerStopMs(g.ptr)
        check(ok and ms_u8 > 0, "8-bit feed / apply / fetch (timed)")
        ctx.barrier(g)
        ms_u8 = ctx.reduce_max(ms_u8)
        lib.dR_freePinned(pin_u8)
        status = lib.dR_getDeviceStatus(g.ptr)
        check(status == 0, "device status %d: a kernel's bounded wait ran out" % status)
        res = {"images_per_s": batch * ctx.world * steps / (ms * 1e-3), "ms_per_step": ms / steps,
               "e2e_images_per_s": batch * ctx.world * steps / (ms_e2e * 1e-3), "e2e_ms_per_step": ms_e2e / steps,
               "h2d_bytes_per_step": in_floats * 4, "d2h_bytes_per_step": out_floats * 4, "steps": steps, "batch_per_gpu": batch,
               "e2e_u8_images_per_s": batch * ctx.world * steps / (ms_u8 * 1e-3), "e2e_u8_ms_per_step": ms_u8 / steps, "e2e_u8_h2d_bytes_per_step": in_floats,
               "clocks": clocks, "probs": probs, "status": status}
        # ---- sustained: back-to-back applies for at least min_seconds, clocks sampled (rank 0 of a single-GPU run)
        if min_seconds > 0:
            n_sus = max(steps, int(min_seconds * 1e3 / res["ms_per_step"]) + 1)
            s2 = ClockSampler(ctx.local)
            s2.start()
            lib.dR_timerStart(g.ptr)
            for _ in range(n_sus):
                ok &= bool(lib.dR_apply(g.ptr))
            ms_s = lib.dR_timerStopMs(g.ptr)
            check(ok and ms_s > 0, "dR_apply (sustained)")
            res["sustained"] = {"seconds": ms_s * 1e-3, "steps": n_sus, "ms_per_step": ms_s / n_sus, "images_per_s": batch * n_sus / (ms_s * 1e-3),
                                "clocks": s2.stop()}
        res["launches_per_apply"] = lib.dR_getLaunchCount(g.ptr)
        if want_profile and ctx.rank == 0:
            lib.dR_synchronize(g.ptr)
            res["profile"] = per_node_profile(dr, lib, g)
            if math == "fp32":
                # the FP32 FMA rate this GPU reaches from registers (the library's own probe kernel): the measured
                # denominator for the FFMA kernels' fractions
                rate = {}
                for name, packed in (("ffma2", 1), ("ffma", 0)):
                    t = ctypes.c_double(0.0)
                    if lib.dR_probeFfmaRate(g.ptr, packed, ctypes.byref(t)) and t.value > 0:
                        rate[name] = t.value
                res["ffma_rate"] = rate
        lib.dR_freePinned(pin_in)
        lib.dR_freePinned(pin_out)
    return res


def measure_dropin(ctx, steps, warmup, batch=64, math="tf32"):
    """The reference-shaped calls (examples/vgg16/vgg_deployed.c:141-166): blocking dR_feedData of [C][H][W] images from
    pageable host memory, dR_apply, blocking dR_downloadArray -- including the CHW <-> HWC conversion kernels."""
    dr, nets, lib = ctx.dr, ctx.nets, ctx.lib
    size = 224
    with dr.Environment(device=ctx.local) as env:
        g = env.create_graph("HWC")                 # layout of the Python-side shapes only; the C interface stays [C][H][W]
        g.batch = batch
        g.math = math
        x, out = nets.vgg16(g, size=size)
        dr.mark_as_output(out)
        dr.prepare(g)
        imgs = np.ascontiguousarray(nets.synthetic_images("bench_dropin", batch, size).transpose(0, 3, 1, 2))
        outbufs = (ctypes.c_void_p * 1)()
        check(lib.dR_getOutputBuffers(g.ptr, outbufs) == 1, "dR_getOutputBuffers")
        probs = np.empty((batch, 1000), np.float32)

        def step():
            lib.dR_feedData(g.ptr, x.ptr, imgs.ctypes.data_as(dr._FP), 0, imgs.size)
            check(lib.dR_apply(g.ptr), "dR_apply")
            lib.dR_downloadArray(g.ptr, b"", outbufs[0], 0, probs.nbytes, probs.ctypes.data_as(ctypes.c_void_p))
        for _ in range(warmup):
            step()
        lib.dR_synchronize(g.ptr)
        t0 = time.perf_counter()
        for _ in range(steps):
            step()                                   # every call blocks: wall clock is the honest timer here
        dt = time.perf_counter() - t0
        check(lib.dR_getDeviceStatus(g.ptr) == 0, "device status")
        return {"value": batch * steps / dt, "unit": "images/s", "ms_per_step": dt / steps * 1e3, "steps": steps,
                "h2d_bytes_per_step": int(imgs.nbytes), "d2h_bytes_per_step": int(probs.nbytes),
                "calls": "dR_feedData (CHW, pageable host memory, blocking) + dR_apply + dR_downloadArray (blocking); wall clock",
                "top1_distinct": int(len(set(probs.argmax(1).tolist())))}


def per_node_profile(dr, lib, g):
    """One apply with per-kernel events; returns [(kind, ms, output shape WxHxC, kernel family of a convolution or None)] per node."""
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
        sh = lib.dR_getOutputShape(node.ptr).contents
        res.append((kind, lib.dR_getNodeGpuMs(node.ptr), "%dx%dx%d" % (sh.s0, sh.s1, sh.s2), lib.dR_getConvAlgo(node.ptr) if kind == "conv" else None))
    lib.dR_config(g.ptr, b"", 1, 0, 0, 0, (g.env.model_path).encode())
    return res


def tf32_yardstick(seconds=4.0):
    """A library TF32 GEMM (torch.matmul, 8192^3) as a yardstick for the tensor roofline: best of 10 single launches (burst) and
    a back-to-back loop of `seconds` (sustained, under the power cap).  Never part of the measured path."""
    try:
        import torch
        torch.backends.cuda.matmul.allow_tf32 = True
        n = 8192
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        for _ in range(3):
            torch.matmul(a, b)
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        best = 1e30
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(seconds * 1e3 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b)
        e1.record()
        e1.synchronize()
        sus = e0.elapsed_time(e1) / reps
        del a, b
        torch.cuda.empty_cache()
        return {"burst_tflops": flops / (best * 1e-3) / 1e12, "sustained_tflops": flops / (sus * 1e-3) / 1e12, "what": "torch.matmul TF32 8192^3 (library GEMM)"}
    except Exception as e:      # noqa: BLE001 -- the yardstick is optional; the roofline falls back to bf16 / 2
        return {"unavailable": str(e)[:200]}


def vgg_roofline(math, batch, prof, peaks, yard):
    """Roofline of the dominant kernel (conv3_2's launch) and of the 13 convolution launches together, from the per-node
    event times of one profiled apply.  Per-launch times are sub-millisecond, so the denominator is the BURST peak."""
    conv_flops, _ = vgg_flops_per_image()
    prof = [(p[0], p[1]) for p in prof]
    conv_times = [t for kind, t in prof if kind == "conv"]
    conv_ms, n_conv = sum(conv_times), len(conv_times)
    tensor = math in ("tf32", "fp32x3")
    if tensor:
        peak, peak_sus = peaks["bf16"] / 2.0, peaks["bf16_sustained"] / 2.0
        peak_src = "%s bf16 cuBLAS burst / 2 (TF32 issues at half the bf16 rate; MEASURED_PEAKS.json holds no TF32 figure)" % peaks["source"]
    else:
        peak = peak_sus = FFMA_PEAK_NOMINAL
        peak_src = "nominal FP32 FFMA: 148 SMs x 128 lanes x 2 flop x 1.965 GHz (no measured FFMA figure in MEASURED_PEAKS.json)"
    aggregate = conv_flops * batch / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else None
    roof = {"bound": "tensor" if tensor else "fp32-ffma", "achieved": aggregate, "peak": peak, "unit": "TFLOP/s", "frac": (aggregate / peak) if aggregate else None,
            "traffic": None, "kernel": "convolution (%d launches, aggregate)" % n_conv, "peak_source": peak_src}
    if n_conv == 13 and conv_times[5] > 0:
        ci, co, hw = VGG_CONVS[5]
        one = 2.0 * 9 * ci * co * hw * hw * batch / (conv_times[5] * 1e-3) / 1e12
        traffic = NCU_TRAFFIC.get((math, batch))
        roof = {"bound": "tensor" if tensor else "fp32-ffma", "achieved": one, "peak": peak, "unit": "TFLOP/s", "frac": one / peak,
                "traffic": traffic[0] if traffic else None, "traffic_source": traffic[1] if traffic else None,
                "algorithmic_bytes": 4.0 * (batch * hw * hw * (ci + co) + 9 * ci * co),
                "kernel": "conv3_2 256->256 @56x56 (%s), %.4f ms per launch" % ("k_umma_conv_swap" if tensor else "FP32 variant chosen at prepare", conv_times[5]),
                "peak_source": peak_src}
    roof["peak_sustained"] = peak_sus
    if tensor and yard and "burst_tflops" in yard:
        roof["frac_of_tf32_matmul_burst"] = roof["achieved"] / yard["burst_tflops"] if roof["achieved"] else None
    roof["conv_aggregate"] = {"tflops": aggregate, "frac": (aggregate / peak) if aggregate else None, "launches": n_conv, "ms": round(conv_ms, 4)}
    roof["ms_by_kind"] = {k: round(sum(t for kk, t in prof if kk == k), 4) for k in sorted(set(k for k, _ in prof))}
    roof["ms_per_layer"] = [[k, round(t, 4)] for k, t in prof if t > 0]        # launch order; fused / elided nodes launch nothing
    return roof, aggregate, conv_ms / max(sum(t for _, t in prof), 1e-9)


def run_ours(args):
    ctx = Ctx()
    batch, single = args.batch, None
    main = measure(ctx, args.net, args.math, batch, args.steps, args.warmup, sampler=ClockSampler(ctx.local), want_profile=True,
                   autotune=bool(args.autotune), min_seconds=(3.0 if (ctx.world == 1 and not args.quick) else 0.0))
    all_probs = ctx.replicas.gather_outputs(ctx.dist, main["probs"], batch * ctx.world, cuda=True)      # outputs of every replica, in image order
    extra = {}
    if not args.quick and args.net == "vgg16":
        k2 = max(3, min(args.steps, 10))
        fp = measure(ctx, "vgg16", "fp32", batch, k2, 3, autotune=True, want_profile=True)
        sq = measure(ctx, "squeezenet", args.math, batch, max(args.steps, 20), 3)
        extra["fp32_exact"], extra["squeezenet_b64"] = fp, sq
        extra["fp32x3"] = measure(ctx, "vgg16", "fp32x3", batch, k2, 3, want_profile=True)
        if args.math != "fp32":
            extra["squeezenet_b64_fp32"] = measure(ctx, "squeezenet", "fp32", batch, k2, 3)
        if ctx.world == 1:
            extra["squeezenet_b1"] = measure(ctx, "squeezenet", args.math, 1, max(args.steps, 50), 5, cuda_graph=True)
            single = measure_dropin(ctx, k2, 3, batch, args.math)
    line = None
    if ctx.rank == 0:
        peaks = measured_peaks()
        yard = tf32_yardstick() if (ctx.world == 1 and not args.quick) else None
        tensor = args.math == "tf32"
        conv_flops, fc_flops = vgg_flops_per_image()
        roof, aggregate = {"bound": "tensor", "achieved": None, "peak": None, "unit": "TFLOP/s", "frac": None, "traffic": None}, None
        conv_share = None
        if args.net == "vgg16":
            roof, aggregate, conv_share = vgg_roofline(args.math, batch, main["profile"], peaks, yard)
        else:
            roof["ms_per_layer"] = [[k, sh, round(t, 4)] for k, t, sh, _ in main["profile"] if t > 0]      # launch order; fused nodes launch nothing
            roof["note"] = "SqueezeNet: per-node event times of one profiled apply (each carries ~5 us of event overhead); no single dominant kernel"
        klass = ("TF32 tensor-core class (fp32 storage, TF32 operands, FP32 accumulate)" if tensor else
                 "FP32-accurate tensor-core class (three TF32 passes per product)" if args.math == "fp32x3" else "exact FP32 class (FFMA)")
        line = {
            "metric": "images/sec", "value": main["images_per_s"], "unit": "images/s", "n_gpus": ctx.world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32" if tensor else ("3xtf32" if args.math == "fp32x3" else "f32"), "data": "synthetic",
            "config": {"workload": "%s inference, %s, batch %d per GPU, 224x224x3 uniform[0,255]-128 inputs, seeded He-normal weights; "
                                   "inputs larger than L2 (no flush)" % ("VGG-16" if args.net == "vgg16" else "SqueezeNet v1.1 (reference example graph)", klass, batch),
                       "global_batch": batch * ctx.world, "parallelism": "replicas x%d (batch sharded, no collective)" % ctx.world,
                       "math": args.math, "autotune": bool(args.autotune)},
            "e2e": {"value": main["e2e_images_per_s"], "unit": "images/s", "h2d_bytes_per_step": main["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": main["d2h_bytes_per_step"], "ms_per_step": main["e2e_ms_per_step"],
                    "calls": "dR_feedDataAsync (pinned, second stream) + dR_apply + dR_fetchOutputAsync, N-HWC interface"},
            "e2e_u8": {"value": main["e2e_u8_images_per_s"], "unit": "images/s", "h2d_bytes_per_step": main["e2e_u8_h2d_bytes_per_step"],
                       "d2h_bytes_per_step": main["d2h_bytes_per_step"], "ms_per_step": main["e2e_u8_ms_per_step"],
                       "calls": "dR_feedDataU8Async (8-bit samples 0..255, pinned; cast to float on the device) + dR_apply + dR_fetchOutputAsync"},
            "gpu_launches": main["launches_per_apply"] * args.steps,
            "clocks": main["clocks"], "roofline": roof,
            "conv_tflops": aggregate, "device_status": main["status"],
            "top1_distinct": int(len(set(all_probs.argmax(1).tolist()))), "gathered_outputs": list(all_probs.shape),
        }
        if "sustained" in main:
            s = main["sustained"]
            mhz = s["clocks"].get("sm_mhz")
            sus = {"seconds": round(s["seconds"], 3), "steps": s["steps"], "images_per_s": s["images_per_s"], "ms_per_step": s["ms_per_step"],
                   "sm_mhz_median": mhz, "power_w_max": s["clocks"].get("power_w_max"), "reasons": s["clocks"].get("reasons"),
                   "ms_x_mhz_per_step": (s["ms_per_step"] * mhz) if mhz else None}
            if conv_share:
                est = conv_flops * batch / (s["ms_per_step"] * conv_share * 1e-3) / 1e12
                sus["conv_tflops_est"] = est
                sus["conv_frac_of_sustained_peak"] = est / roof["peak_sustained"]
                sus["note"] = "conv TFLOP/s estimated from this loop's step time x the convolutions' share of the profiled apply (%.3f)" % conv_share
            line["sustained"] = sus
        if "fp32_exact" in extra:
            fp = extra["fp32_exact"]
            froof, fagg, _ = vgg_roofline("fp32", batch, fp["profile"], peaks, None) if "profile" in fp else ({}, None, None)
            # FFMA work really executed: a Winograd layer multiplies 16 (F(2x2,3x3)) or 36 (F(4x4,3x3)) transform-domain values per
            # tile of 4 or 16 outputs (whole tiles, so 14x14 planes pay for 16x16 under F(4x4)) instead of 9 per output
            real, families = None, None
            convs = [(t, algo) for kind, t, _, algo in fp["profile"] if kind == "conv" and t > 0] if "profile" in fp else []
            if fagg and len(convs) == len(VGG_CONVS):
                executed, conv_ms, families = 0.0, 0.0, []
                for (ci, co, hw), (t, algo) in zip(VGG_CONVS, convs):
                    if algo == 2:
                        per_image = 2.0 * 16 * ci * co * ((hw + 1) // 2) ** 2
                    elif algo == 6:
                        per_image = 2.0 * 36 * ci * co * ((hw + 3) // 4) ** 2
                    else:
                        per_image = 2.0 * 9 * ci * co * hw * hw
                    executed += per_image * batch
                    conv_ms += t
                    families.append({1: "direct", 2: "winograd F(2x2,3x3)", 3: "1x1", 6: "winograd F(4x4,3x3)"}.get(algo, str(algo)))
                real = executed / (conv_ms * 1e-3) / 1e12
            line["fp32_exact"] = {"images_per_s": fp["images_per_s"], "ms_per_step": fp["ms_per_step"], "e2e_images_per_s": fp["e2e_images_per_s"],
                                  "steps": fp["steps"], "dtype": "f32", "conv_tflops_direct_equivalent": fagg, "conv_tflops_executed_ffma": real,
                                  "frac_of_ffma_peak_executed": (real / FFMA_PEAK_NOMINAL) if real else None, "ffma_peak": FFMA_PEAK_NOMINAL,
                                  "ffma_peak_source": "nominal 148 SMs x 128 lanes x 2 x 1.965 GHz",
                                  "ffma_rate_measured": fp.get("ffma_rate"),
                                  "frac_of_ffma_rate_measured_executed": (real / max(fp["ffma_rate"].values())) if real and fp.get("ffma_rate") else None,
                                  "ffma_rate_source": "dR_probeFfmaRate: 8 x 8 register outer product per thread, no memory traffic, every SM filled; best of three launches",
                                  "ms_per_layer": froof.get("ms_per_layer"),
                                  "conv_kernel_family_per_layer": families,
                                  "tolerance": "1e-4 x max|ref| per layer (FP32 FFMA arithmetic; F(4x4,3x3) layers measure about 2e-5, F(2x2,3x3) -- the reference's transform -- 1e-6)"}
        if "fp32x3" in extra:
            x3 = extra["fp32x3"]
            xroof, xagg, _ = vgg_roofline("tf32", batch, x3["profile"], peaks, None) if "profile" in x3 else ({}, None, None)
            # executed tensor-core work: three MMAs per product; a Winograd F(4x4,3x3) layer has 36 products per whole tile of 16 outputs
            xexec, xfam = None, None
            xconvs = [(t, algo) for kind, t, _, algo in x3["profile"] if kind == "conv" and t > 0] if "profile" in x3 else []
            if xagg and len(xconvs) == len(VGG_CONVS):
                ex, ms_t, xfam = 0.0, 0.0, []
                for (ci, co, hw), (t, algo) in zip(VGG_CONVS, xconvs):
                    if algo == 5:
                        ex += 3 * 2.0 * 36 * ci * co * ((hw + 3) // 4) ** 2 * batch
                        ms_t += t
                    elif algo == 4:
                        ex += 3 * 2.0 * 9 * ci * co * hw * hw * batch
                        ms_t += t
                    xfam.append({1: "FP32 direct (FFMA)", 4: "direct, 3 passes", 5: "winograd F(4x4,3x3), 3 passes", 6: "FP32 winograd F(4x4,3x3) (FFMA)"}.get(algo, str(algo)))
                xexec = ex / (ms_t * 1e-3) / 1e12 if ms_t > 0 else None
            line["fp32_accurate_tensor"] = {"images_per_s": x3["images_per_s"], "ms_per_step": x3["ms_per_step"], "e2e_images_per_s": x3["e2e_images_per_s"],
                                            "steps": x3["steps"], "dtype": "3xtf32", "conv_tflops_direct_equivalent": xagg,
                                            "conv_tflops_executed_tf32_tensor_layers": xexec, "conv_kernel_family_per_layer": xfam,
                                            "ms_per_layer": xroof.get("ms_per_layer"),
                                            "what": "math mode fp32x3: 3x3 layers with >= 8 input channels evaluate every product as hi*hi + hi*lo + lo*hi in three TF32 "
                                                    "tensor-core passes (FP32-class error bound 1e-4 x max|ref| per layer) -- the deep layers as Winograd F(4x4,3x3) "
                                                    "with its 36 transform-domain products on the tensor cores, the others directly, FC as a three-pass split-K GEMM; first layer, pooling, softmax on the FP32 kernels"}
        if "squeezenet_b64" in extra:
            sq = extra["squeezenet_b64"]
            line["squeezenet"] = {"batch64": {"images_per_s": sq["images_per_s"], "ms_per_step": sq["ms_per_step"], "e2e_images_per_s": sq["e2e_images_per_s"],
                                              "e2e_u8_images_per_s": sq["e2e_u8_images_per_s"], "launches_per_apply": sq["launches_per_apply"], "conv_tflops": SQUEEZENET_CONV_FLOPS * sq["images_per_s"] / 1e12 / ctx.world,
                                              "h2d_bytes_per_step": sq["h2d_bytes_per_step"]},
                                  "graph": "reference example graph (conv1 3x3 stride 1 + 2x2 average pool, 8 Fire modules, conv10, global average pool, softmax)",
                                  "math": args.math}
            if "squeezenet_b64_fp32" in extra:
                sf = extra["squeezenet_b64_fp32"]
                line["squeezenet"]["batch64_fp32_mode"] = {"images_per_s": sf["images_per_s"], "ms_per_step": sf["ms_per_step"], "e2e_images_per_s": sf["e2e_images_per_s"],
                                                           "launches_per_apply": sf["launches_per_apply"], "dtype": "f32",
                                                           "conv_tflops": SQUEEZENET_CONV_FLOPS * sf["images_per_s"] / 1e12 / ctx.world}
            if "squeezenet_b1" in extra:
                s1 = extra["squeezenet_b1"]
                line["squeezenet"]["batch1"] = {"images_per_s": s1["images_per_s"], "ms_per_image": s1["ms_per_step"], "e2e_images_per_s": s1["e2e_images_per_s"],
                                                "launches_per_apply": s1["launches_per_apply"], "cuda_graph_replay": True}
        if single is not None:
            line["e2e_dropin"] = single
        if yard is not None:
            line["tf32_yardstick"] = yard
        if ctx.world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_budget)
    ctx.replicas.finish(ctx.dist)
    if line is not None:
        print(json.dumps(line))


# ------------------------------------------------------------------ CPU side (oracle is the checker / baseline only)
def _cpu_vgg_weights():
    import cases
    convs, fcs = [], []
    for i, (ci, co, hw) in enumerate(VGG_CONVS):
        _, w, b = cases.conv_case("cpu_vgg_conv%d" % i, 1, ci, co, 4, 4, 3)
        convs.append((w, b, 2 * 9 * ci * co * hw * hw))
    for i, (a, bb) in enumerate(VGG_FCS):
        g = cases.rng("cpu_vgg_fc%d" % i)
        w = g.standard_normal((a, bb), dtype=np.float32) * np.float32(np.sqrt(2.0 / a))
        fcs.append((w * np.float32(0.05) if i == 2 else w, np.zeros(bb, np.float32), 2 * a * bb))
    return convs, fcs


def cpu_image(oracle, convs, fcs, x, use_ref):
    """One image through the whole of VGG-16 on the host: 13 convolutions (the reference's Winograd kernel), 5 max pools,
    3 fully connected layers (its two FC kernels), softmax -- each layer fed with the previous one's output."""
    for i, (w, b, _) in enumerate(convs):
        x = oracle.ref_conv2d_winograd(x, w, b, 1) if use_ref else oracle.conv2d_winograd(x, w, b, 1)
        if i in VGG_POOL_AFTER:
            x = oracle.pool(x, (2, 2, 1), (2, 2, 1), 0)     # the reference generates this kernel at run time; restated in C
    for i, (w, b, _) in enumerate(fcs):
        act = 0 if i == 2 else 1
        x = (oracle.ref_fc(x, w, b, act) if use_ref else oracle.fc(x, w, b, act))
    return oracle.ref_softmax(x) if use_ref else oracle.softmax(x)


def cpu_conv3_2(oracle, convs, use_ref, x):
    w, b, _ = convs[5]
    return oracle.ref_conv2d_winograd(x, w, b, 1) if use_ref else oracle.conv2d_winograd(x, w, b, 1)


def cpu_plan(oracle, use_ref, steps, budget_s):
    """What one CPU step runs: a whole image if `steps` of them fit the budget, else conv3_2 alone scaled by FLOPs."""
    import nets
    convs, fcs = _cpu_vgg_weights()
    img = np.ascontiguousarray(nets.synthetic_images("cpu_img", 1, 224).transpose(0, 3, 1, 2))
    t0 = time.time()
    cpu_image(oracle, convs, fcs, img, use_ref)
    t_full = time.time() - t0
    total = sum(c[2] for c in convs) + sum(f[2] for f in fcs)
    if t_full * steps <= budget_s:
        return (lambda: cpu_image(oracle, convs, fcs, img, use_ref)), 1.0, "1 image through the whole network per step (13 conv + 5 max pool + 3 FC + softmax, layers chained)"
    import cases
    x = cases.act_case("cpu_conv3_2_in", 1, 256, 56, 56)
    frac = convs[5][2] / total
    return (lambda: cpu_conv3_2(oracle, convs, use_ref, x)), frac, "1 image through conv3_2 per step (%.0f%% of the image's FLOPs), scaled by FLOPs" % (100 * frac)


def cpu_describe(oracle, use_ref, what):
    if use_ref:
        return (what + "; reference OpenCL C kernels compiled as C (conv2dwinograd2, matrixVectorMultFirst/Second, computeExp), OpenMP over "
                "work-groups, scheduled for an emulated device with local memory %d KiB and max work-group size %d; 2x2 max pooling by the C restatement"
                % (oracle.REF_LMS // 1024, oracle.REF_MWS))
    return what + "; C restatement of the reference's Winograd arithmetic (port)"


def cpu_baseline(budget_s=20.0, steps=3):
    import oracle
    from oracle import build_oracle
    build_oracle.build_restatement()
    use_ref = oracle.ref_available()
    cores = oracle.set_threads()
    step, frac, what = cpu_plan(oracle, use_ref, steps + 1, budget_s)
    t0 = time.time()
    for _ in range(steps):
        step()
    dt = (time.time() - t0) / steps
    return {"value": frac / dt, "unit": "images/s", "cores": cores, "kind": "reference" if use_ref else "port", "sample": cpu_describe(oracle, use_ref, what)}


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
    step, frac, what = cpu_plan(oracle, use_ref, args.steps + args.warmup + 1, 170.0)
    for _ in range(args.warmup):
        step()
    t0 = time.time()
    for _ in range(args.steps):
        step()
    dt = time.time() - t0
    value = frac * args.steps / dt
    kind = "reference" if use_ref else "port"
    line = {"impl": "reference", "metric": "images/sec", "value": value, "unit": "images/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "VGG-16 inference, exact FP32 (the reference's arithmetic), 224x224x3 inputs (CPU arm: one image per step)",
                       "global_batch": 64, "parallelism": "host cores"},
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "sample": cpu_describe(oracle, use_ref, what)},
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
    ap.add_argument("--math", default=os.environ.get("DR_BENCH_MATH", "tf32"), choices=["fp32", "tf32", "fp32x3"])
    ap.add_argument("--autotune", type=int, default=-1, help="time conv variants at prepare; default: only in fp32 mode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    ap.add_argument("--quick", action="store_true", help="headline measurement only (no fp32_exact / squeezenet / sustained / yardstick objects)")
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
