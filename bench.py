#!/usr/bin/env python3
"""Headline benchmark: ResNet-50 forward, batch 64 per GPU, through libcaffe.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one Net::Forward over one batch of synthetic input (seeded
U(0,255) minus the channel means; random He-normal weights, identity
BatchNorm).  For N > 1 launch under torch.distributed.run: one process per
GPU, each with a full weight replica and its own batch (weak scaling), no
collective in the timed loop; only the final class scores are gathered, after
timing.  Rank 0 prints one JSON line.

  value      images/s with the input already resident in device memory
             (CUDA events on the engine's stream, max over ranks)
  e2e        images/s through the C API with the input in (pinned) host memory:
             every step uploads the batch and downloads the class scores
  roofline   the tensor-core convolution kernel, timed live with CUDA events
             around every launch: algorithmic bytes / time against the measured
             HBM copy bandwidth (the binding limit for fp32 activations; the
             achieved TF32 rate is reported beside it)
  cpu_baseline  mini-caffe's own CPU path (oracle/_ref, OpenBLAS threads = host
             cores) on a bounded sample of the same workload

--impl reference times that CPU path as the measured arm instead.
"""
import argparse
import ctypes
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ENGINE_LIB = os.path.join(ROOT, "mini-caffe_b200", "lib", "libcaffe.so")
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcaffe_ref.so")
BATCH_PER_GPU = 64
E2E_THREADS = 2        # host threads per GPU in the end-to-end leg, each with its own Net
# DRAM bytes per convolution launch (read + write, averaged over the 54 launches of one pass at
# batch 64) from one ncu capture of this workload: 3589 MB read + 1139 MB written per pass.  Below
# the algorithmic 126 MB per launch because small activations stay in L2 between layers.
CONV_DRAM_BYTES_PER_LAUNCH = 87.61e6
METRIC = "resnet50_images_per_sec"
UNIT = "images/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.first_sample = threading.Event()
        self.stop_flag = threading.Event()
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            if self.stop_flag.is_set():
                break
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sample = (time.monotonic(), float(parts[0]), float(parts[1]))
            except ValueError:
                continue
            active = [name for name, flag in zip(names, parts[3:7]) if flag.lower().startswith("active")]
            self.samples.append(sample + (active,))
            self.first_sample.set()

    def wait_ready(self, timeout=5.0):
        """Blocks until nvidia-smi has delivered its first line (its start-up takes a while)."""
        self.first_sample.wait(timeout)

    def finish(self, windows):
        """Summary over the samples that fall inside the timed windows [(t0, t1), ...] (time.monotonic)."""
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()   # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        inside = [s for s in self.samples if any(t0 <= s[0] <= t1 for t0, t1 in windows)]
        scope = "timed regions"
        if not inside:   # regions shorter than the sampling period: take the samples around them
            lo, hi = min(t0 for t0, _ in windows) - 0.05, max(t1 for _, t1 in windows) + 0.05
            inside = [s for s in self.samples if lo <= s[0] <= hi] or self.samples
            scope = "around the timed regions"
        reasons = sorted({r for s in inside for r in s[3]})
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": max(s[2] for s in inside),
                "reasons": reasons, "samples": len(inside), "scope": scope}


def build_resnet(capi, wl, library, batch):
    builder = wl.resnet50(batch)
    net = capi.Net(library, builder.text(), None, from_buffer=True)
    net.set_params(wl.init_params(builder.params, seed=0))
    return net


def cpu_reference_rate(capi, wl, steps, warmup, budget_s):
    """images/s of the reference CPU build on a sample sized to fit `budget_s` seconds."""
    if not os.path.isfile(REF_LIB):
        return None
    cores = os.cpu_count() or 1
    os.environ.setdefault("OPENBLAS_NUM_THREADS", str(cores))
    ref = capi.CaffeLibrary(REF_LIB)
    probe_batch = 4
    net = build_resnet(capi, wl, ref, probe_batch)
    x = wl.image_input(probe_batch, seed=0)
    net.forward(**x)
    t0 = time.perf_counter()
    net.forward()
    probe_rate = probe_batch / (time.perf_counter() - t0)
    net.close()
    per_step = int(max(1, min(BATCH_PER_GPU, probe_rate * budget_s / max(1, steps + warmup))))
    net = build_resnet(capi, wl, ref, per_step)
    net.forward(**wl.image_input(per_step, seed=0))
    for _ in range(max(0, warmup - 1)):
        net.forward()
    t0 = time.perf_counter()
    for _ in range(steps):
        net.forward()
    dt = time.perf_counter() - t0
    net.close()
    return {"value": per_step * steps / dt, "unit": UNIT, "cores": cores, "kind": "reference",
            "sample": "%d forward passes of ResNet-50 at batch %d (workload batch is %d) on %d OpenBLAS threads; only "
                      "SGEMM is multi-threaded in the reference" % (steps, per_step, BATCH_PER_GPU, cores),
            "ms_per_step": dt / steps * 1e3, "batch": per_step}


def time_forwards(engine, L, net, stream, torch, reps, warmup=3):
    """Milliseconds per CaffeNetForward (inputs resident on the device), CUDA events on the engine's stream."""
    for _ in range(warmup):
        engine.check(L.CaffeNetForward(net.handle))
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(reps):
        engine.check(L.CaffeNetForward(net.handle))
    ev1.record(stream)
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / reps


def proposal_figure(capi, wl, engine, L, stream, torch, reps=10, images=32):
    """RPN Proposal stress case: 63x38 map, 15 anchors, pre-NMS 6000, post-NMS 300, `images` images in one
    call.  boxes/s := images * min(pre_nms_topn, A*H*W) / time of the whole layer forward (decode, top-k,
    NMS, gather, counts back to the host)."""
    import numpy as np
    b = wl.proposal(num_anchors=15)
    text = b.text().replace("dim: 1 dim: 30", "dim: %d dim: 30" % images).replace(
        "dim: 1 dim: 60", "dim: %d dim: 60" % images).replace("dim: 1 dim: 3 }", "dim: %d dim: 3 }" % images)
    net = capi.Net(engine, text, None, from_buffer=True)
    batches = [wl.proposal_input(num_anchors=15, seed=i)[0] for i in range(images)]
    feed = {k: np.concatenate([x[k] for x in batches], axis=0) for k in batches[0]}
    net.forward(**feed)
    ms = time_forwards(engine, L, net, stream, torch, reps)
    n_all = 15 * 63 * 38
    out = {"images_per_call": images, "ms_per_call": ms, "rois": int(net.blob("rois").shape[0]),
           "nms_boxes_per_s": images * min(6000, n_all) / (ms * 1e-3),
           "decoded_boxes_per_s": images * n_all / (ms * 1e-3),
           "iou_pairs_upper_bound_per_image": 6000 * 5999 // 2,
           "algorithmic_bytes_per_image": 4 * n_all + 16 * n_all + 12 + 24 * 300}
    net.close()
    return out


def detection_output_figure(capi, wl, engine, L, stream, torch, reps=10, images=32):
    """SSD300 post-processing: 8732 priors, 21 classes, confidence 0.01, NMS 0.45, top_k 400, keep 200,
    near-uniform class scores (what random-init heads give: every class of every prior passes the
    threshold, the top_k cut does the work).  boxes/s := 8732 * 20 * images / time."""
    b = wl.detection_head(batch=images, num_priors=8732, num_classes=21, conf_thr=0.01, nms_thr=0.45, top_k=400,
                          keep_top_k=200)
    net = capi.Net(engine, b.text(), None, from_buffer=True)
    net.forward(**wl.detection_head_input(images, 8732, 21, seed=0))
    ms = time_forwards(engine, L, net, stream, torch, reps)
    out = {"images_per_call": images, "ms_per_call": ms, "rows": int(net.blob("detection_out").shape[0]),
           "boxes_per_s": 8732 * 20 * images / (ms * 1e-3),
           "algorithmic_bytes_per_image": 4 * (8732 * 4 + 8732 * 21) + 28 * 200}
    net.close()
    return out


def roi_pooling_figure(capi, wl, engine, L, stream, torch, reps=20):
    """R-FCN head: 300 rois over 21 x 7 x 7 position-sensitive score maps of 63 x 38."""
    b = wl.roi_pooling("PSROIPooling", batch=1, height=63, width=38, num_rois=300, output_dim=21, group_size=7)
    net = capi.Net(engine, b.text(), None, from_buffer=True)
    net.forward(**wl.roi_pooling_input(1, 21 * 49, 63, 38, 300, seed=0))
    ms = time_forwards(engine, L, net, stream, torch, reps)
    out = {"rois": 300, "ms_per_call": ms, "rois_per_s": 300 / (ms * 1e-3),
           "algorithmic_bytes": 4 * (21 * 49 * 63 * 38 + 300 * 5 + 300 * 21 * 49)}
    net.close()
    return out


def secondary_figures(capi, wl, engine, L, stream, torch):
    """The other figures the benchmark definition names, measured after the headline: NMS boxes/s of
    the RPN Proposal stress case and the TF32 rate of the single 3x3 64->64 convolution at batch 32."""
    out = {"proposal": proposal_figure(capi, wl, engine, L, stream, torch)}
    # Config 1: Convolution(64, 3x3, pad 1) + ReLU on [32, 64, 56, 56]
    cb = wl.conv_relu(32)
    net = capi.Net(engine, cb.text(), None, from_buffer=True)
    net.set_params(wl.init_params(cb.params, seed=0))
    net.forward(**wl.conv_relu_input(32, seed=0))
    L.mcb200_kernel_timing_begin()
    for _ in range(20):
        engine.check(L.CaffeNetForward(net.handle))
    conv_ms = ctypes.c_double(0.0)
    n = int(L.mcb200_kernel_timing_end(ctypes.byref(conv_ms)))
    flops = 2 * 32 * 64 * 56 * 56 * 64 * 9
    out["conv_relu_b32"] = {"kernel_ms": conv_ms.value / max(1, n), "tf32_tflops": flops / (conv_ms.value / max(1, n) * 1e-3) / 1e12,
                            "algorithmic_bytes": 4 * (2 * 32 * 64 * 56 * 56 + 64 * 64 * 9 + 64)}
    net.close()
    out["resnet50_bf16_storage"] = bf16_storage_figure(capi, wl, engine, L, stream, torch)
    return out


def bf16_storage_figure(capi, wl, engine, L, stream, torch, batch=BATCH_PER_GPU, reps=30):
    """The engine's precision opt-in (MINICAFFE_PRECISION=bf16 while the net is constructed): the same
    ResNet-50 pass with bfloat16 operands in the tensor-core convolutions and bfloat16 storage of the
    blobs between them.  Input resident on the device; not the headline (which is fp32 storage / TF32)."""
    previous = os.environ.get("MINICAFFE_PRECISION")
    os.environ["MINICAFFE_PRECISION"] = "bf16"
    try:
        net = build_resnet(capi, wl, engine, batch)
    finally:
        if previous is None:
            del os.environ["MINICAFFE_PRECISION"]
        else:
            os.environ["MINICAFFE_PRECISION"] = previous
    net.forward(**wl.image_input(batch, seed=0))
    ms = time_forwards(engine, L, net, stream, torch, reps)
    net.close()
    return {"images_per_s": batch / (ms * 1e-3), "ms_per_step": ms, "batch": batch, "dtype": "bf16 operands and storage, fp32 accumulation",
            "how": "MINICAFFE_PRECISION=bf16 at net construction"}


def run_tail_workload(args, capi, wl):
    """`--workload proposal | detection_output | psroi_pooling`: the detection-tail layers on their own
    (one GPU), for profiler captures and the figures in profiles/.  Prints one JSON line."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: the engine has no CPU path")
    engine = capi.CaffeLibrary(ENGINE_LIB)
    L = engine.lib
    L.mcb200_current_stream.restype = ctypes.c_void_p
    L.mcb200_launch_count.restype = ctypes.c_longlong
    engine.set_mode(True, 0)
    stream = torch.cuda.ExternalStream(L.mcb200_current_stream(), device=torch.device("cuda", 0))
    fn = {"proposal": proposal_figure, "detection_output": detection_output_figure,
          "psroi_pooling": roi_pooling_figure}[args.workload]
    L.mcb200_launch_count_reset()
    res = fn(capi, wl, engine, L, stream, torch, reps=args.steps)
    res.update({"workload": args.workload, "steps": args.steps, "gpu_launches": int(L.mcb200_launch_count())})
    print(json.dumps(res))


def run_reference_arm(args, capi, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": "resnet50 forward, batch %d per GPU, 224x224" % BATCH_PER_GPU}}
    res = cpu_reference_rate(capi, wl, args.steps, args.warmup, budget_s=150.0)
    if res is None:
        base["unavailable"] = "oracle/_ref/libcaffe_ref.so is not built (needs the reference checkout at build time)"
        print(json.dumps(base))
        return
    base.update({"value": res["value"], "ms_per_step": res["ms_per_step"], "cpu_baseline": res, "gpu_launches": 0,
                 "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    base["config"]["sample_batch"] = res["batch"]
    print(json.dumps(base))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU,
                    help="images per GPU (the headline metric is quoted at the default; smaller values are for "
                         "profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU reference leg (profiler captures)")
    ap.add_argument("--workload", default="resnet50",
                    choices=["resnet50", "proposal", "detection_output", "psroi_pooling"],
                    help="resnet50 is the benchmark; the others time one detection-tail layer on its own")
    ap.add_argument("--precision", default="tf32", choices=["tf32", "bf16"],
                    help="tf32 (default, the benchmark: fp32 storage, TF32 tensor cores) or the engine's bfloat16 "
                         "storage opt-in for the whole run (profiler captures of that mode)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    # The engine reads the opt-in from the environment when a net is constructed.
    if args.precision == "bf16":
        os.environ["MINICAFFE_PRECISION"] = "bf16"
    else:
        os.environ.pop("MINICAFFE_PRECISION", None)

    capi = importlib.import_module("mini-caffe_b200.capi")
    wl = importlib.import_module("mini-caffe_b200.workloads")
    if args.impl == "reference":
        run_reference_arm(args, capi, wl)
        return
    if args.workload != "resnet50":
        run_tail_workload(args, capi, wl)
        return

    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE is %d: launch with torch.distributed.run" % (args.gpus, world))
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    engine = capi.CaffeLibrary(ENGINE_LIB)
    L = engine.lib
    L.mcb200_current_stream.restype = ctypes.c_void_p
    L.mcb200_launch_count.restype = ctypes.c_longlong
    L.mcb200_kernel_timing_end.restype = ctypes.c_longlong
    L.mcb200_kernel_timing_end.argtypes = [ctypes.POINTER(ctypes.c_double)]
    engine.set_mode(True, local_rank)
    stream_ptr = L.mcb200_current_stream()
    if not stream_ptr:
        raise SystemExit("engine stream: " + L.CaffeGetLastError().decode())
    stream = torch.cuda.ExternalStream(stream_ptr, device=torch.device("cuda", local_rank))

    batch = args.batch
    net = build_resnet(capi, wl, engine, batch)
    x = wl.image_input(batch, seed=rank)["data"]
    data_blob = net.blob("data")
    data_blob.reshape(*x.shape)
    data_blob.data[...] = x
    prob_blob = net.blob("prob")

    def forward():
        engine.check(L.CaffeNetForward(net.handle))

    # ---- device-resident throughput: the input blob's device copy stays valid ----
    for _ in range(args.warmup):
        forward()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.wait_ready()
    windows = []
    barrier()
    L.mcb200_launch_count_reset()
    w0 = time.monotonic()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        forward()
    ev1.record(stream)
    barrier()
    windows.append((w0, time.monotonic()))
    launches = int(L.mcb200_launch_count())
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    ms_per_step = ms_total / args.steps
    value = world * batch * args.steps / (ms_total * 1e-3)

    # ---- end to end: host input -> device, forward, scores -> host, every step ----
    # One caller first (what a single application thread sees), then the K steps
    # dealt out to E2E_THREADS host threads, each with its own Net on this GPU
    # (the engine keeps stream, pool and mode per thread, like mini-caffe):
    # one thread's input copy overlaps the other's kernels.  Every step still
    # copies its input from pinned host memory and reads its scores back.
    for _ in range(2):
        data_blob.data  # marks the pinned host copy as the current one
        forward()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        data_blob.data
        forward()
        prob_blob.data
    barrier()
    e2e_single_s = max_over_ranks(time.perf_counter() - t0)

    import threading
    start_line = threading.Barrier(E2E_THREADS + 1)
    finish_line = threading.Barrier(E2E_THREADS + 1)
    errors = []

    def e2e_worker(tid):
        try:
            engine.set_mode(True, local_rank)      # this thread's own stream and memory pool
            own = build_resnet(capi, wl, engine, batch)
            blob = own.blob("data")
            blob.reshape(*x.shape)
            blob.data[...] = x
            out = own.blob("prob")
            for _ in range(2):
                blob.data
                engine.check(L.CaffeNetForward(own.handle))
            start_line.wait()
            for _ in range(args.steps // E2E_THREADS + (1 if tid < args.steps % E2E_THREADS else 0)):
                blob.data
                engine.check(L.CaffeNetForward(own.handle))
                out.data
            finish_line.wait()
            own.close()
        except Exception as exc:   # surfaced by the main thread
            errors.append(exc)
            for line in (start_line, finish_line):
                line.abort()

    workers = [threading.Thread(target=e2e_worker, args=(t,)) for t in range(E2E_THREADS)]
    for w in workers:
        w.start()
    try:
        barrier()
        start_line.wait()          # the workers are warmed up and leave this line together with the clock
        w0 = time.monotonic()
        t0 = time.perf_counter()
        finish_line.wait()
        e2e_local = time.perf_counter() - t0
    except threading.BrokenBarrierError:
        e2e_local = float("nan")
    for w in workers:
        w.join()
    if errors:
        raise errors[0]
    barrier()
    e2e_s = max_over_ranks(e2e_local)
    windows.append((w0, time.monotonic()))
    clocks = sampler.finish(windows) if sampler else None
    e2e_value = world * batch * args.steps / e2e_s
    e2e_single_value = world * batch * args.steps / e2e_single_s
    h2d = int(np.prod(x.shape)) * 4
    d2h = int(np.prod(prob_blob.shape)) * 4

    # ---- the convolution kernel on its own clock ----
    barrier()
    # (Events around every convolution launch keep consecutive launches from
    # overlapping, so this is each kernel's own duration; in the timed loops above
    # a launch's set-up overlaps the end of the launch before it.)
    # Three sessions, the quickest counts: a session slowed by something else on
    # the machine says nothing about the kernel.
    timed_steps = min(args.steps, 5)
    conv_ms, conv_launches = None, 0
    for _ in range(3):
        L.mcb200_kernel_timing_begin()
        for _ in range(timed_steps):
            forward()
        session_ms = ctypes.c_double(0.0)
        session_launches = int(L.mcb200_kernel_timing_end(ctypes.byref(session_ms)))
        if conv_ms is None or session_ms.value < conv_ms.value:
            conv_ms, conv_launches = session_ms, session_launches
    peaks = load_peaks()
    conv_bytes = wl.resnet50_conv_bytes(batch, bf16_storage=args.precision == "bf16")   # per forward pass
    conv_flops = wl.resnet50_flops_per_image() * batch
    conv_s_per_step = conv_ms.value * 1e-3 / timed_steps
    launches_per_step = conv_launches / timed_steps
    achieved_gbs = conv_bytes / conv_s_per_step / 1e9
    roofline = {
        "kernel": "conv_tc_kernel (tcgen05 implicit GEMM, %d launches per forward)" % round(launches_per_step),
        "bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": achieved_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
        "traffic": CONV_DRAM_BYTES_PER_LAUNCH if (batch == BATCH_PER_GPU and args.precision == "tf32") else None,
        "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum averaged over the 54 launches of a pass, from "
                        "the ncu capture summarised in profiles/conv_tc_kernel_resnet50_b64.md (same workload)",
        "algorithmic_bytes_per_launch": conv_bytes / launches_per_step,
        "avg_launch_ms": conv_ms.value / max(1, conv_launches),
        "tf32_tflops_achieved": conv_flops / conv_s_per_step / 1e12,
        "tf32_peak_tflops_assumed": peaks["bf16_tflops"] / 2.0,
        "kernel_ms_per_step": conv_s_per_step * 1e3,
        "share_of_step": min(1.0, conv_s_per_step * 1e3 / ms_per_step),
        "share_of_step_note": "sum of the kernel's own launch durations / time of a step; launches overlap by "
                              "their set-up (programmatic dependent launch), so the ratio is capped at 1",
    }

    # ---- secondary figures of the benchmark definition (rank 0, after the headline) ----
    extras = secondary_figures(capi, wl, engine, L, stream, torch) if rank == 0 else None

    # ---- final output gather (outside the timed loops) ----
    probs = torch.from_numpy(prob_blob.data.copy()).cuda()
    if world > 1:
        gathered = [torch.empty_like(probs) for _ in range(world)] if rank == 0 else None
        dist.gather(probs, gathered, dst=0)
        gathered_rows = sum(int(g.shape[0]) for g in gathered) if rank == 0 else 0
    else:
        gathered_rows = int(probs.shape[0])

    if rank == 0:
        cpu = None if args.no_cpu_baseline else cpu_reference_rate(capi, wl, steps=2, warmup=1, budget_s=20.0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": args.precision, "data": "synthetic",
            "config": {"workload": "resnet50 forward (Caffe layout conv+BN+Scale+ReLU, Eltwise residuals), batch %d "
                                   "per GPU, 3x224x224 fp32 input" % batch,
                       "global_batch": world * batch, "parallelism": "replica per GPU, batch sharded, no collective",
                       "l2": "activations of one pass (%.1f GB of convolution traffic) exceed the 126 MB L2"
                             % (conv_bytes / 1e9),
                       "flops_per_image": wl.resnet50_flops_per_image(), "gathered_output_rows": gathered_rows},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "host_threads": E2E_THREADS, "single_thread_value": e2e_single_value,
                    "how": "CaffeNetForward on host buffers; %d host threads per GPU, one Net each, K steps in total"
                           % E2E_THREADS},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "secondary": extras,
            "cpu_baseline": cpu if cpu else {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                             "sample": "skipped (--no-cpu-baseline)" if args.no_cpu_baseline
                                             else "oracle/_ref not built"},
        }
        print(json.dumps(line))
    net.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
