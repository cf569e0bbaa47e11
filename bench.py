#!/usr/bin/env python3
"""Headline benchmark: ResNet-50 forward, batch 64 per GPU, through libcaffe.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl reference]

One "step" is one Net::Forward over one batch of synthetic input (seeded
U(0,255) minus the channel means; random He-normal weights, identity
BatchNorm).  For N > 1 launch under torch.distributed.run: one process per
GPU, each with a full weight replica and its own batch (weak scaling), no
collective in the timed loop; only the final class scores are gathered, after
timing.  Rank 0 prints one JSON line.

  value      images/s with the input already resident in device memory: exactly
             K steps between CUDA events on the engine's stream, max over ranks;
             the K-step loop is repeated R times and the median counts (all R
             figures are printed under "repeats")
  e2e        images/s through the C API with the input in (pinned) host memory:
             every step uploads the batch and downloads the class scores
  roofline   the tensor-core convolution kernel, timed live with CUDA events
             around every launch: algorithmic bytes / time against the measured
             HBM copy bandwidth (the binding limit for fp32 activations), the
             achieved TF32 rate against the tcgen05 kind::tf32 issue rate measured
             in the same run, and a per-layer table saying which of the two
             bounds each layer
  secondary  the other configurations of the benchmark definition (single
             convolution, MobileNet-v1, SSD300, DetectionOutput, Proposal), each
             with its bound and with the reference's CPU code timed beside it
  cpu_baseline  mini-caffe's own CPU path (oracle/_ref, OpenBLAS threads = host
             cores) on a bounded sample of the same workload

--impl reference times that CPU path as the measured arm instead.
"""
import argparse
import ctypes
import hashlib
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
KERNEL_SOURCES = [os.path.join(ROOT, "mini-caffe_b200", "csrc", "kernels", f) for f in ("conv_tc.cu", "sm100.cuh")]
BATCH_PER_GPU = 64
def _e2e_threads():
    """Host threads per GPU in the end-to-end leg, each with its own Net and stream.  Three where the
    host has the cores for it: the third net's kernels run on the SMs that the under-filled launches
    of the other two leave idle (measured on one B200: 31 500 images/s with two threads, 35 200 with
    three or four); two when eight ranks share sixteen cores."""
    forced = os.environ.get("MCB200_E2E_THREADS")
    if forced:
        return max(1, int(forced))
    per_rank = (os.cpu_count() or 2) // max(1, int(os.environ.get("WORLD_SIZE", "1")))
    return 3 if per_rank >= 3 else 2


E2E_THREADS = _e2e_threads()
# DRAM bytes per convolution launch (dram__bytes_read.sum + dram__bytes_write.sum, averaged over
# the 54 launches of one pass at batch 64) from one ncu launch-list capture of this workload, and
# the hash of the kernel sources the capture was made with.  A different hash means the figure is
# stale: the line then carries null until the capture is repeated.
CONV_TRAFFIC = {"bytes_per_launch": 87.96e6, "kernel_sha16": "fb7a1d4658a37bed"}
METRIC = "resnet50_images_per_sec"
UNIT = "images/s"


def workload_name(batch):
    return ("resnet50 forward (Caffe layout conv+BN+Scale+ReLU, Eltwise residuals), batch %d per GPU, "
            "3x224x224 fp32 input" % batch)


def kernel_sha16():
    h = hashlib.sha256()
    for path in KERNEL_SOURCES:
        with open(path, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


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


def build_net(capi, library, builder, weights=None):
    net = capi.Net(library, builder.text(), None, from_buffer=True)
    if weights is not None:
        net.set_params(weights)
    return net


def build_resnet(capi, wl, library, batch):
    builder = wl.resnet50(batch)
    return build_net(capi, library, builder, wl.init_params(builder.params, seed=0))


# ----------------------------------------------------------------------------- CPU reference legs

def reference_library(capi):
    """The reference's CPU build with all host cores given to OpenBLAS, or None when it is not there."""
    if not os.path.isfile(REF_LIB):
        return None
    os.environ.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
    return capi.CaffeLibrary(REF_LIB)


def cpu_reference_rate(capi, wl, steps, warmup, budget_s, engine_check=None):
    """images/s of the reference CPU build on a sample sized to fit `budget_s` seconds.  With
    `engine_check` (a function batch, input -> fc1000 of the engine) the sample's class scores are
    also compared with the engine's: the error figures against the literal tolerance are returned."""
    ref = reference_library(capi)
    if ref is None:
        return None
    cores = os.cpu_count() or 1
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
    x = wl.image_input(per_step, seed=0)
    net.forward(**x)
    for _ in range(max(0, warmup - 1)):
        net.forward()
    t0 = time.perf_counter()
    for _ in range(steps):
        net.forward()
    dt = time.perf_counter() - t0
    want = net.blob("fc1000").data.copy()
    net.close()
    out = {"value": per_step * steps / dt, "unit": UNIT, "cores": cores, "kind": "reference",
           "sample": "%d forward passes of ResNet-50 at batch %d (workload batch is %d) on %d OpenBLAS threads; only "
                     "SGEMM is multi-threaded in the reference" % (steps, per_step, BATCH_PER_GPU, cores),
           "ms_per_step": dt / steps * 1e3, "batch": per_step}
    if engine_check is not None:
        out["parity_of_sample"] = literal_bound_stats(engine_check(per_step, x), want, "fc1000")
    return out


def literal_bound_stats(got, want, blob):
    """How a blob fares against the stated tolerance read literally (|a-b| <= 2e-2 + 1e-2 |b|) and
    against the bound the tests assert (absolute term in units of the blob's RMS when that is > 1)."""
    import numpy as np
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    ref = np.abs(want.astype(np.float64))
    rms = float(np.sqrt(np.mean(ref ** 2)))
    return {"blob": blob, "elements": int(err.size), "max_abs_err": float(err.max()), "rms_ref": rms,
            "max_abs_err_over_peak": float(err.max() / ref.max()) if ref.max() > 0 else 0.0,
            "outside_literal_bound": int((err > 2e-2 + 1e-2 * ref).sum()),
            "outside_asserted_bound": int((err > 2e-2 * max(1.0, rms) + 1e-2 * ref).sum())}


def cpu_forward_ms(capi, ref, builder, weights, feed, passes=1):
    """Milliseconds per forward pass of a net on the reference CPU build (one warm-up pass, then `passes`)."""
    box = {}

    def body():
        net = build_net(capi, ref, builder, weights)
        net.forward(**feed)
        t0 = time.perf_counter()
        for _ in range(passes):
            net.forward()
        box["ms"] = (time.perf_counter() - t0) / passes * 1e3
        net.close()
        ref.memory_pool_clear()

    t = threading.Thread(target=body)   # the reference's memory pool is per thread: leave nothing behind
    t.start()
    t.join()
    return box["ms"]


# ----------------------------------------------------------------------------- GPU timing helpers

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


def bound_of(flops, nbytes, ms, peaks, tf32_peak_tflops):
    """Which roofline bounds a piece of work (the larger of the two floor times) and the fraction reached."""
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    t_tensor = flops / (tf32_peak_tflops * 1e12) if tf32_peak_tflops else 0.0
    bound = "tensor" if t_tensor > t_hbm else "hbm"
    floor_ms = max(t_hbm, t_tensor) * 1e3
    return {"bound": bound, "floor_ms": floor_ms, "frac": floor_ms / ms if ms > 0 else None,
            "hbm_gbs_achieved": nbytes / (ms * 1e-3) / 1e9, "tf32_tflops_achieved": flops / (ms * 1e-3) / 1e12}


def proposal_net_text(wl, images, anchors=15):
    b = wl.proposal(num_anchors=anchors)
    return b.text().replace("dim: 1 dim: %d" % (2 * anchors), "dim: %d dim: %d" % (images, 2 * anchors)).replace(
        "dim: 1 dim: %d" % (4 * anchors), "dim: %d dim: %d" % (images, 4 * anchors)).replace(
        "dim: 1 dim: 3 }", "dim: %d dim: 3 }" % images)


def proposal_figure(capi, wl, engine, L, stream, torch, reps=10, images=32, seed0=0, reduce_max=None, world=1):
    """RPN Proposal stress case: 63x38 map, 15 anchors, pre-NMS 6000, post-NMS 300, `images` images in one
    call on every GPU.  boxes/s := images * min(pre_nms_topn, A*H*W) / time of the whole layer forward
    (decode, top-k, NMS, gather, counts back to the host); with several GPUs the images of all ranks over
    the slowest rank's time."""
    import numpy as np
    net = capi.Net(engine, proposal_net_text(wl, images), None, from_buffer=True)
    batches = [wl.proposal_input(num_anchors=15, seed=seed0 + i)[0] for i in range(images)]
    feed = {k: np.concatenate([x[k] for x in batches], axis=0) for k in batches[0]}
    net.forward(**feed)
    ms = time_forwards(engine, L, net, stream, torch, reps)
    if reduce_max is not None:
        ms = reduce_max(ms)
    n_all = 15 * 63 * 38
    total = images * world
    out = {"images_per_call": images, "n_gpus": world, "images_total": total, "ms_per_call": ms,
           "rois": int(net.blob("rois").shape[0]),
           "nms_boxes_per_s": total * min(6000, n_all) / (ms * 1e-3),
           "decoded_boxes_per_s": total * n_all / (ms * 1e-3),
           "iou_pairs_upper_bound_per_image": 6000 * 5999 // 2,
           "algorithmic_bytes_per_image": 4 * n_all + 16 * n_all + 12 + 24 * 300}
    out["hbm_gbs_achieved"] = out["algorithmic_bytes_per_image"] * total / (ms * 1e-3) / 1e9 / max(1, world)
    net.close()
    return out


def proposal_cpu(capi, wl, ref, images=8):
    """The reference's ProposalLayer::Forward_cpu on `images` single-image calls (it takes one image per call)."""
    b = wl.proposal(num_anchors=15)
    feeds = [wl.proposal_input(num_anchors=15, seed=i)[0] for i in range(images)]
    box = {}

    def body():
        net = build_net(capi, ref, b)
        net.forward(**feeds[0])
        t0 = time.perf_counter()
        for f in feeds:
            net.forward(**f)
        box["s"] = time.perf_counter() - t0
        net.close()

    t = threading.Thread(target=body)
    t.start()
    t.join()
    return {"nms_boxes_per_s": images * 6000 / box["s"], "ms_per_image": box["s"] / images * 1e3, "cores": 1,
            "kind": "reference", "sample": "%d images, one call each (proposal_layer.cpp is single-threaded)" % images}


def detection_output_figure(capi, wl, engine, L, stream, torch, reps=10, images=32):
    """SSD300 post-processing: 8732 priors, 21 classes, confidence 0.01, NMS 0.45, top_k 400, keep 200,
    near-uniform class scores (what random-init heads give: every class of every prior passes the
    threshold, the top_k cut does the work).  boxes/s := 8732 * 20 * images / time."""
    b = wl.detection_head(batch=images, num_priors=8732, num_classes=21, conf_thr=0.01, nms_thr=0.45, top_k=400,
                          keep_top_k=200)
    net = capi.Net(engine, b.text(), None, from_buffer=True)
    net.forward(**wl.detection_head_input(images, 8732, 21, seed=0))
    ms = time_forwards(engine, L, net, stream, torch, reps)
    nbytes = 4 * (8732 * 4 + 8732 * 21) + 28 * 200
    out = {"images_per_call": images, "ms_per_call": ms, "rows": int(net.blob("detection_out").shape[0]),
           "boxes_per_s": 8732 * 20 * images / (ms * 1e-3), "algorithmic_bytes_per_image": nbytes,
           "hbm_gbs_achieved": nbytes * images / (ms * 1e-3) / 1e9}
    net.close()
    return out


def detection_output_cpu(capi, wl, ref, images=4):
    b = wl.detection_head(batch=images, num_priors=8732, num_classes=21, conf_thr=0.01, nms_thr=0.45, top_k=400,
                          keep_top_k=200)
    ms = cpu_forward_ms(capi, ref, b, None, wl.detection_head_input(images, 8732, 21, seed=0), passes=2)
    return {"boxes_per_s": 8732 * 20 * images / (ms * 1e-3), "ms_per_image": ms / images, "cores": 1,
            "kind": "reference", "sample": "2 passes over %d images (detection_output_layer.cpp is single-threaded)" % images}


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


def dense_net_figure(capi, wl, engine, L, stream, torch, builder, feed, batch, peaks, tf32_peak, reps):
    """A whole generated network, input resident: ms per pass, images/s, FLOPs and algorithmic bytes of
    its Convolution / InnerProduct layers, and the bound those give."""
    net = build_net(capi, engine, builder, wl.init_params(builder.params, seed=0))
    net.forward(**feed)
    work = wl.conv_work(builder, {name: blob.shape for name, blob in net.blobs()})
    ms = time_forwards(engine, L, net, stream, torch, reps)
    # each tensor-core convolution launch's own duration, in launch order (median of five passes)
    passes = []
    for _ in range(5):
        L.mcb200_kernel_timing_begin()
        engine.check(L.CaffeNetForward(net.handle))
        total = ctypes.c_double(0.0)
        each = (ctypes.c_double * 512)()
        n = int(L.mcb200_kernel_timing_end_each(ctypes.byref(total), each, 512))
        passes.append([each[i] * 1e3 for i in range(min(n, 512))])
    conv_tc_us = ([round(sorted(p[i] for p in passes)[2], 1) for i in range(len(passes[0]))]
                  if all(len(p) == len(passes[0]) for p in passes) else [])
    net.close()
    out = {"batch": batch, "ms_per_step": ms, "images_per_s": batch / (ms * 1e-3), "conv_flops": work["flops"],
           "conv_algorithmic_bytes": work["bytes"], "conv_layers": work["layers"], "conv_tc_launch_us": conv_tc_us}
    out.update(bound_of(work["flops"], work["bytes"], ms, peaks, tf32_peak))
    return out


def measured_peaks(L, stream_ptr, torch):
    """The tensor pipe's issue rate and the L2 -> shared memory rate, measured now on this device
    (probe kernels of the library: all SMs, operands resident in shared memory / in L2)."""
    L.mcb200_probe_mma_peak.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double), ctypes.c_void_p]
    L.mcb200_probe_tma_l2_pull.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                                           ctypes.c_void_p]
    out = {"how": "tcgen05.mma issued back to back by one thread per SM on one shared-memory stage (M=128 per "
                  "CTA), about 1 ms per launch, quickest of 3; TMA pulls of 16 KiB tiles from a 64 MiB tensor"}
    ms, rate = ctypes.c_double(0.0), ctypes.c_double(0.0)
    for key, bf16, n, pair in (("tf32_n256", 0, 256, 0), ("tf32_n128", 0, 128, 0), ("tf32_n64", 0, 64, 0),
                               ("tf32_n256_cta_pair", 0, 256, 1), ("bf16_n256", 1, 256, 0)):
        rc = L.mcb200_probe_mma_peak(bf16, n, pair, 4096, 3, ctypes.byref(ms), ctypes.byref(rate), stream_ptr)
        out[key + "_tflops"] = rate.value if rc == 0 else None
        if rc != 0:
            out[key + "_error"] = rc
    buf = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    rc = L.mcb200_probe_tma_l2_pull(ctypes.c_void_p(buf.data_ptr()), buf.numel(), 4096, 8, 3, ctypes.byref(ms),
                                    ctypes.byref(rate), stream_ptr)
    out["l2_to_smem_gbs"] = rate.value if rc == 0 else None
    if rc != 0:
        out["l2_to_smem_error"] = rc
    del buf
    return out


def secondary_figures(capi, wl, engine, L, stream, torch, peaks, tf32_peak, rank, world, max_over_ranks, with_cpu):
    """The other figures the benchmark definition names, measured after the headline.  The Proposal
    stress case runs on every rank (its 256 images are split over the GPUs, 32 per call); the rest on
    rank 0.  Each figure carries the reference's CPU code on a bounded sample of the same work."""
    import numpy as np
    proposal = proposal_figure(capi, wl, engine, L, stream, torch, seed0=32 * rank, reduce_max=max_over_ranks, world=world)
    if rank != 0:
        return None
    out = {"proposal": proposal}
    ref = reference_library(capi) if with_cpu else None

    # Config 1: Convolution(64, 3x3, pad 1) + ReLU on [32, 64, 56, 56]
    cb = wl.conv_relu(32)
    conv_weights = wl.init_params(cb.params, seed=0)
    net = build_net(capi, engine, cb, conv_weights)
    net.forward(**wl.conv_relu_input(32, seed=0))
    L.mcb200_kernel_timing_begin()
    for _ in range(20):
        engine.check(L.CaffeNetForward(net.handle))
    conv_ms = ctypes.c_double(0.0)
    n = int(L.mcb200_kernel_timing_end(ctypes.byref(conv_ms)))
    net.close()
    flops = 2 * 32 * 64 * 56 * 56 * 64 * 9
    nbytes = 4 * (2 * 32 * 64 * 56 * 56 + 64 * 64 * 9 + 64)
    kernel_ms = conv_ms.value / max(1, n)
    fig = {"kernel_ms": kernel_ms, "tf32_tflops": flops / (kernel_ms * 1e-3) / 1e12, "algorithmic_bytes": nbytes}
    fig.update(bound_of(flops, nbytes, kernel_ms, peaks, tf32_peak))
    out["conv_relu_b32"] = fig

    # Config 3: MobileNet-v1 at batch 64; config 4: SSD300 at batch 32 (DetectionOutput included)
    mb = wl.mobilenet_v1(64)
    out["mobilenet_v1_b64"] = dense_net_figure(capi, wl, engine, L, stream, torch, mb, wl.normal_image_input(64, seed=0),
                                               64, peaks, tf32_peak, reps=30)
    sb = wl.ssd300_vgg16(32)
    out["ssd300_b32"] = dense_net_figure(capi, wl, engine, L, stream, torch, sb, wl.ssd_input(32, seed=0), 32, peaks,
                                         tf32_peak, reps=10)
    out["detection_output"] = detection_output_figure(capi, wl, engine, L, stream, torch)
    out["resnet50_bf16_storage"] = bf16_storage_figure(capi, wl, engine, L, stream, torch)
    # The other batch sizes the benchmark definition names for ResNet-50 (64 is the headline)
    sweep = {}
    for b in (1, 16, 256):
        rnet = build_resnet(capi, wl, engine, b)
        rnet.forward(**wl.image_input(b, seed=0))
        ms = time_forwards(engine, L, rnet, stream, torch, 30 if b < 256 else 10)
        rnet.close()
        sweep[str(b)] = {"ms_per_step": ms, "images_per_s": b / (ms * 1e-3)}
    out["resnet50_batch_sweep"] = sweep
    # The shipped WGAN generator's structure at its own batch (64): five Deconvolution layers on the
    # tensor-core kernel (stride-1 convolution, reversed filter, of the input spread over zeros).
    gb = wl.wgan_generator(64)
    gnet = build_net(capi, engine, gb, wl.init_params(gb.params, seed=0, bn_identity=False))
    gnet.forward(**wl.wgan_noise(64))
    gms = time_forwards(engine, L, gnet, stream, torch, 30)
    gnet.close()
    # useful FLOPs of a transposed convolution: every input element meets every filter tap once
    gflops, cin, side = 0, 100, 1
    for i, cout in enumerate((512, 256, 128, 64, 3)):
        gflops += 2 * 64 * side * side * cin * cout * 16
        side, cin = (4 if i == 0 else side * 2), cout
    out["wgan_g"] = {"batch": 64, "ms_per_step": gms, "images_per_s": 64 / (gms * 1e-3), "deconv_flops": gflops,
                     "tf32_tflops_achieved": gflops / (gms * 1e-3) / 1e12, "deconvolution_layers": 5}

    if ref is not None:
        out["proposal"]["cpu_baseline"] = proposal_cpu(capi, wl, ref)
        out["detection_output"]["cpu_baseline"] = detection_output_cpu(capi, wl, ref)
        ms = cpu_forward_ms(capi, ref, cb, conv_weights, wl.conv_relu_input(32, seed=0), passes=3)
        out["conv_relu_b32"]["cpu_baseline"] = {"ms_per_step": ms, "gflops": flops / (ms * 1e-3) / 1e9, "batch": 32,
                                                "cores": os.cpu_count(), "kind": "reference", "sample": "3 passes at batch 32"}
        small = wl.mobilenet_v1(4)
        ms = cpu_forward_ms(capi, ref, small, wl.init_params(small.params, seed=0), wl.normal_image_input(4, seed=0))
        out["mobilenet_v1_b64"]["cpu_baseline"] = {"images_per_s": 4 / (ms * 1e-3), "batch": 4, "cores": os.cpu_count(),
                                                   "kind": "reference", "sample": "1 pass at batch 4"}
        ms = cpu_forward_ms(capi, ref, gb, wl.init_params(gb.params, seed=0, bn_identity=False), wl.wgan_noise(64))
        out["wgan_g"]["cpu_baseline"] = {"images_per_s": 64 / (ms * 1e-3), "batch": 64, "cores": os.cpu_count(),
                                         "kind": "reference", "sample": "1 pass at batch 64"}
        small = wl.ssd300_vgg16(1)
        ms = cpu_forward_ms(capi, ref, small, wl.init_params(small.params, seed=0), wl.ssd_input(1, seed=0))
        out["ssd300_b32"]["cpu_baseline"] = {"images_per_s": 1 / (ms * 1e-3), "batch": 1, "cores": os.cpu_count(),
                                             "kind": "reference", "sample": "1 pass at batch 1"}
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


def open_engine(capi, local_rank):
    import torch
    engine = capi.CaffeLibrary(ENGINE_LIB)
    L = engine.lib
    L.mcb200_current_stream.restype = ctypes.c_void_p
    L.mcb200_launch_count.restype = ctypes.c_longlong
    L.mcb200_kernel_timing_end.restype = ctypes.c_longlong
    L.mcb200_kernel_timing_end.argtypes = [ctypes.POINTER(ctypes.c_double)]
    L.mcb200_kernel_timing_end_each.restype = ctypes.c_longlong
    L.mcb200_kernel_timing_end_each.argtypes = [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                                               ctypes.c_longlong]
    engine.set_mode(True, local_rank)
    stream_ptr = L.mcb200_current_stream()
    if not stream_ptr:
        raise SystemExit("engine stream: " + L.CaffeGetLastError().decode())
    stream = torch.cuda.ExternalStream(stream_ptr, device=torch.device("cuda", local_rank))
    return engine, L, stream_ptr, stream


def init_ranks(args):
    """(torch, rank, local_rank, world, barrier, max_over_ranks) for a one-process-per-GPU launch."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE is %d: launch with torch.distributed.run" % (args.gpus, world))
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL writes its version banner to file descriptor 1 when the first communicator comes up;
        # stdout carries the one JSON line, so descriptor 1 points at stderr until that has happened.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

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

    return torch, dist, rank, local_rank, world, barrier, max_over_ranks


def run_tail_workload(args, capi, wl):
    """`--workload proposal | detection_output | psroi_pooling | mobilenet_v1 | ssd300`: one of the other
    configurations on its own (for profiler captures and the figures in profiles/).  The Proposal
    workload also runs under torch.distributed.run: 32 images per rank, boxes/s summed over the ranks
    against the slowest rank's time.  Prints one JSON line."""
    torch, dist, rank, local_rank, world, barrier, max_over_ranks = init_ranks(args)
    if world > 1 and args.workload != "proposal":
        raise SystemExit("--workload %s runs on one GPU" % args.workload)
    engine, L, stream_ptr, stream = open_engine(capi, local_rank)
    peaks = load_peaks()
    L.mcb200_launch_count_reset()
    barrier()
    if args.workload == "proposal":
        res = proposal_figure(capi, wl, engine, L, stream, torch, reps=args.steps, seed0=32 * rank,
                              reduce_max=max_over_ranks, world=world)
    elif args.workload == "detection_output":
        res = detection_output_figure(capi, wl, engine, L, stream, torch, reps=args.steps)
    elif args.workload == "psroi_pooling":
        res = roi_pooling_figure(capi, wl, engine, L, stream, torch, reps=args.steps)
    else:
        batch = args.batch
        builder, feed = ((wl.mobilenet_v1(batch), wl.normal_image_input(batch, seed=0)) if args.workload == "mobilenet_v1"
                         else (wl.ssd300_vgg16(batch), wl.ssd_input(batch, seed=0)))
        res = dense_net_figure(capi, wl, engine, L, stream, torch, builder, feed, batch, peaks, None, reps=args.steps)
    res.update({"workload": args.workload, "steps": args.steps, "gpu_launches": int(L.mcb200_launch_count())})
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference_arm(args, capi, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": workload_name(BATCH_PER_GPU)}}
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
    ap.add_argument("--repeats", type=int, default=5,
                    help="how many times the timed K-step loop is run; the median counts, all are printed")
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--batch", type=int, default=None,
                    help="images per GPU (the headline metric is quoted at the default, 64; smaller values are for "
                         "profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU reference legs (profiler captures)")
    ap.add_argument("--no-secondary", action="store_true", help="headline only (profiler captures)")
    ap.add_argument("--workload", default="resnet50",
                    choices=["resnet50", "proposal", "detection_output", "psroi_pooling", "mobilenet_v1", "ssd300"],
                    help="resnet50 is the benchmark; the others time one of the other configurations on its own")
    ap.add_argument("--precision", default="tf32", choices=["tf32", "bf16"],
                    help="tf32 (default, the benchmark: fp32 storage, TF32 tensor cores) or the engine's bfloat16 "
                         "storage opt-in for the whole run (profiler captures of that mode)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    if args.batch is None:
        args.batch = {"mobilenet_v1": 64, "ssd300": 32}.get(args.workload, BATCH_PER_GPU)
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
    torch, dist, rank, local_rank, world, barrier, max_over_ranks = init_ranks(args)
    engine, L, stream_ptr, stream = open_engine(capi, local_rank)

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
    loop_ms = []
    launches = 0
    for _ in range(args.repeats):
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
        loop_ms.append(max_over_ranks(ev0.elapsed_time(ev1)))
    ms_total = statistics.median(loop_ms)
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

    e2e_repeats = min(args.repeats, 3)
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
            share = args.steps // E2E_THREADS + (1 if tid < args.steps % E2E_THREADS else 0)
            for _ in range(e2e_repeats):
                start_line.wait()
                for _ in range(share):
                    blob.data
                    engine.check(L.CaffeNetForward(own.handle))
                    out.data
                finish_line.wait()
            # the same nets with the input left on the device: what the concurrency alone is worth
            for _ in range(e2e_repeats):
                start_line.wait()
                for _ in range(share):
                    engine.check(L.CaffeNetForward(own.handle))
                out.data                     # one read at the end: waits for this thread's stream
                finish_line.wait()
            own.close()
        except Exception as exc:   # surfaced by the main thread
            errors.append(exc)
            for line in (start_line, finish_line):
                line.abort()

    workers = [threading.Thread(target=e2e_worker, args=(t,)) for t in range(E2E_THREADS)]
    for w in workers:
        w.start()
    e2e_loops = []
    resident_loops = []
    try:
        for _ in range(e2e_repeats):
            barrier()
            start_line.wait()          # the workers are warmed up and leave this line together with the clock
            w0 = time.monotonic()
            t0 = time.perf_counter()
            finish_line.wait()
            e2e_local = time.perf_counter() - t0
            windows.append((w0, time.monotonic()))
            e2e_loops.append(max_over_ranks(e2e_local))
        for _ in range(e2e_repeats):
            barrier()
            start_line.wait()
            t0 = time.perf_counter()
            finish_line.wait()
            resident_loops.append(max_over_ranks(time.perf_counter() - t0))
    except threading.BrokenBarrierError:
        e2e_loops.append(float("nan"))
    for w in workers:
        w.join()
    if errors:
        raise errors[0]
    barrier()
    e2e_s = statistics.median(e2e_loops)
    clocks = sampler.finish(windows) if sampler else None
    e2e_value = world * batch * args.steps / e2e_s
    concurrent_value = (world * batch * args.steps / statistics.median(resident_loops)) if resident_loops else None
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
    table = wl.resnet50_conv_table()
    conv_ms, conv_launches, per_launch = None, 0, None
    for _ in range(3):
        L.mcb200_kernel_timing_begin()
        for _ in range(timed_steps):
            forward()
        session_ms = ctypes.c_double(0.0)
        each = (ctypes.c_double * (timed_steps * len(table)))()
        session_launches = int(L.mcb200_kernel_timing_end_each(ctypes.byref(session_ms), each, len(each)))
        if conv_ms is None or session_ms.value < conv_ms.value:
            conv_ms, conv_launches, per_launch = session_ms, session_launches, list(each)
    peaks = load_peaks()
    probes = measured_peaks(L, stream_ptr, torch) if rank == 0 else {}
    tf32_peak = probes.get("tf32_n256_tflops")
    conv_bytes = wl.resnet50_conv_bytes(batch, bf16_storage=args.precision == "bf16")   # per forward pass
    conv_flops = wl.resnet50_flops_per_image() * batch
    conv_s_per_step = conv_ms.value * 1e-3 / timed_steps
    launches_per_step = conv_launches / timed_steps
    achieved_gbs = conv_bytes / conv_s_per_step / 1e9
    achieved_tflops = conv_flops / conv_s_per_step / 1e12
    sha = kernel_sha16()
    traffic_ok = (batch == BATCH_PER_GPU and args.precision == "tf32" and CONV_TRAFFIC["kernel_sha16"] == sha)
    roofline = {
        "kernel": "conv_tc_kernel (tcgen05 implicit GEMM, %d launches per forward)" % round(launches_per_step),
        "bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": achieved_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
        "traffic": CONV_TRAFFIC["bytes_per_launch"] if traffic_ok else None,
        "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum averaged over the convolution launches of a "
                        "pass, from an ncu launch-list capture of this workload made with kernel sources of hash %s "
                        "(current sources: %s%s)" % (CONV_TRAFFIC["kernel_sha16"], sha,
                                                     "" if traffic_ok else "; stale or another configuration, so null"),
        "algorithmic_bytes_per_launch": conv_bytes / launches_per_step,
        "avg_launch_ms": conv_ms.value / max(1, conv_launches),
        "tf32_tflops_achieved": achieved_tflops,
        "tf32_peak_tflops_measured": tf32_peak,
        "tf32_frac_of_measured": achieved_tflops / tf32_peak if tf32_peak else None,
        "measured_peaks": probes,
        "kernel_ms_per_step": conv_s_per_step * 1e3,
        "share_of_step": min(1.0, conv_s_per_step * 1e3 / ms_per_step),
        "share_of_step_note": "sum of the kernel's own launch durations / time of a step; launches overlap by "
                              "their set-up (programmatic dependent launch), so the ratio is capped at 1",
    }
    if rank == 0 and per_launch and conv_launches == timed_steps * len(table) and args.precision == "tf32":
        roofline.update(layer_table(table, per_launch, timed_steps, batch, peaks, tf32_peak))

    # ---- secondary figures of the benchmark definition (after the headline) ----
    extras = None
    if not args.no_secondary:
        extras = secondary_figures(capi, wl, engine, L, stream, torch, peaks, tf32_peak, rank, world, max_over_ranks,
                                   with_cpu=not args.no_cpu_baseline)

    # ---- final output gather (outside the timed loops) ----
    probs = torch.from_numpy(prob_blob.data.copy()).cuda()
    if world > 1:
        gathered = [torch.empty_like(probs) for _ in range(world)] if rank == 0 else None
        dist.gather(probs, gathered, dst=0)
        gathered_rows = sum(int(g.shape[0]) for g in gathered) if rank == 0 else 0
    else:
        gathered_rows = int(probs.shape[0])

    if rank == 0:
        def engine_scores(sample_batch, sample_input):
            probe = build_resnet(capi, wl, engine, sample_batch)
            probe.forward(**sample_input)
            scores = probe.blob("fc1000").data.copy()
            probe.close()
            return scores

        cpu = None if args.no_cpu_baseline else cpu_reference_rate(capi, wl, steps=2, warmup=1, budget_s=20.0,
                                                                    engine_check=engine_scores)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": args.precision, "data": "synthetic",
            "config": {"workload": workload_name(batch),
                       "global_batch": world * batch, "parallelism": "replica per GPU, batch sharded, no collective",
                       "l2": "activations of one pass (%.1f GB of convolution traffic) exceed the 126 MB L2"
                             % (conv_bytes / 1e9),
                       "flops_per_image": wl.resnet50_flops_per_image(), "gathered_output_rows": gathered_rows},
            "repeats": {"n": args.repeats, "steps_each": args.steps, "ms_per_step": [m / args.steps for m in loop_ms],
                        "value_min": world * batch * args.steps / (max(loop_ms) * 1e-3),
                        "value_max": world * batch * args.steps / (min(loop_ms) * 1e-3),
                        "how": "value and ms_per_step are the median of the repeated K-step loops"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "host_threads": E2E_THREADS, "single_thread_value": e2e_single_value,
                    "loops_s": e2e_loops,
                    "how": "CaffeNetForward on host buffers; %d host threads per GPU, one Net each, K steps in total "
                           "per loop, median of %d loops" % (E2E_THREADS, e2e_repeats)},
            "concurrent_nets": {"value": concurrent_value, "unit": UNIT, "nets_per_gpu": E2E_THREADS,
                                "how": "the end-to-end leg's nets and threads with the input left on the device: K steps "
                                       "in total per loop, one Net and stream per thread; kernels of one net run on the "
                                       "SMs an under-filled launch of another leaves idle, so this exceeds `value`, "
                                       "which is one Net on one stream"},
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


def layer_table(table, per_launch, timed_steps, batch, peaks, tf32_peak):
    """Per convolution / inner-product launch of a pass: mean duration over the timed passes, FLOPs,
    algorithmic bytes, which roofline bounds it and the fraction of that bound it reaches; plus the
    summary over the tensor-bound layers (the ones a tensor-pipe target applies to)."""
    n = len(table)
    rows = []
    tensor_flops = tensor_s = hbm_bytes = hbm_s = 0.0
    for i, (name, cin, cout, k, _, hi, ho, res) in enumerate(table):
        ms = sum(per_launch[p * n + i] for p in range(timed_steps)) / timed_steps
        flops = 2.0 * batch * cout * ho * ho * cin * k * k
        nbytes = 4.0 * (batch * cin * hi * hi + cout * cin * k * k + batch * cout * ho * ho * (2 if res else 1) + cout)
        b = bound_of(flops, nbytes, ms, peaks, tf32_peak)
        rows.append([name, round(ms * 1e3, 1), b["bound"], round(b["frac"], 3), round(b["tf32_tflops_achieved"], 1),
                     round(b["hbm_gbs_achieved"], 0)])
        if b["bound"] == "tensor":
            tensor_flops += flops
            tensor_s += ms * 1e-3
        else:
            hbm_bytes += nbytes
            hbm_s += ms * 1e-3
    out = {"layers_columns": ["layer", "us", "bound", "frac_of_bound", "tf32_tflops", "hbm_gbs"], "layers": rows}
    if tensor_s > 0:
        out["tensor_bound_layers"] = {"count": sum(1 for r in rows if r[2] == "tensor"),
                                      "tf32_tflops": tensor_flops / tensor_s / 1e12,
                                      "frac_of_measured_tf32_peak": tensor_flops / tensor_s / 1e12 / tf32_peak if tf32_peak else None}
    if hbm_s > 0:
        out["hbm_bound_layers"] = {"count": sum(1 for r in rows if r[2] == "hbm"), "gbs": hbm_bytes / hbm_s / 1e9,
                                   "frac_of_measured_hbm": hbm_bytes / hbm_s / 1e9 / peaks["hbm_gbs"]}
    return out


if __name__ == "__main__":
    main()
