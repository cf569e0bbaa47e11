#!/usr/bin/env python3
"""Where the tensor-core convolution kernel's time goes, from cycle counters inside the kernel.

    make -C mini-caffe_b200/csrc trace            # builds lib/libcaffe_trace.so
    python mini-caffe_b200/conv_trace.py --n 64 --c 64 --hw 56 --cout 64 --k 3 --pad 1

Runs one layer through the kernel-level C ABI of the trace build and prints, for CTA 0, how the
single-thread roles spend a k-iteration (cycles of the SM clock):

  producer A / B   wait for a free stage, time to issue the loads
  MMA issuer       wait for a full stage (this is where load latency shows), time to issue
  epilogue warp 0  wait for the accumulator per tile, time to store the tile, and the phases of a chunk

A diagnostic, not part of the engine; needs a GPU.
"""
import argparse
import ctypes
import os
import statistics

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
SLOTS = 2048
ROLES = 5


class ConvShape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("n", "h", "w", "c", "c_stride", "cout", "kh", "kw", "stride_h", "stride_w",
                 "pad_h", "pad_w", "dil_h", "dil_w", "group", "ho", "wo")]


class Epilogue(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_void_p), ("shift", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("residual_ld", ctypes.c_int), ("residual_coeff", ctypes.c_float), ("act", ctypes.c_int),
                ("slope", ctypes.c_float), ("prelu", ctypes.c_void_p), ("prelu_shared", ctypes.c_int),
                ("round_tf32", ctypes.c_int)]


class ConvPlan(ctypes.Structure):
    _fields_ = [("tma_a", ctypes.c_uint64 * 16), ("tma_b", ctypes.c_uint64 * 16),
                ("tma_out", ctypes.c_uint64 * 16), ("tma_res", ctypes.c_uint64 * 16), ("shape", ConvShape),
                ("m", ctypes.c_int), ("k_iters", ctypes.c_int), ("c_blocks", ctypes.c_int),
                ("block_n", ctypes.c_int), ("im2col", ctypes.c_int), ("out_ld", ctypes.c_int),
                ("res_ld", ctypes.c_int), ("cta_pair", ctypes.c_int), ("operand_bf16", ctypes.c_int),
                ("out_bf16", ctypes.c_int), ("out_ptr", ctypes.c_void_p), ("res_ptr", ctypes.c_void_p),
                ("m_virtual", ctypes.c_int), ("strip_rows", ctypes.c_int)]


def summary(name, values):
    if not values:
        return "%-34s -" % name
    q = statistics.quantiles(values, n=10) if len(values) >= 10 else [min(values)] * 9
    return "%-34s median %7.0f   p10 %7.0f   p90 %7.0f   n %d" % (name, statistics.median(values), q[0], q[8], len(values))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=64)
    ap.add_argument("--c", type=int, default=64)
    ap.add_argument("--hw", type=int, default=56)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=1)
    ap.add_argument("--residual", action="store_true")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--dump", type=int, default=0, help="print the first N k-iterations of every role, stamp by stamp")
    ap.add_argument("--lib", default=os.path.join(ROOT, "lib", "libcaffe_trace.so"))
    args = ap.parse_args()
    L = ctypes.CDLL(args.lib)
    L.mcb200_conv_packed_weight_count.restype = ctypes.c_size_t
    s = ConvShape(args.n, args.hw, args.hw, args.c, args.c, args.cout, args.k, args.k, args.stride, args.stride, args.pad,
                  args.pad, 1, 1, 1, 0, 0)
    assert L.mcb200_conv_out_shape(ctypes.byref(s)) == 0
    g = torch.Generator().manual_seed(0)
    w = (torch.randn((args.cout, args.c, args.k, args.k), generator=g) * 0.05).cuda()
    raw = ctypes.create_string_buffer(ctypes.sizeof(ConvPlan) + 64)
    plan = ConvPlan.from_address((ctypes.addressof(raw) + 63) & ~63)
    if args.c <= 4:
        # an image in front of the first layer: row mode over a zero-bordered copy with 4 floats per pixel
        assert L.mcb200_conv_rows_supported(ctypes.byref(s)) == 1
        L.mcb200_conv_rows_packed_weight_count.restype = ctypes.c_size_t
        image = torch.randn((args.n, args.c, args.hw, args.hw), generator=g).cuda()
        hp, wp = ctypes.c_int(), ctypes.c_int()
        assert L.mcb200_conv_rows_padded_dims(ctypes.byref(s), ctypes.byref(hp), ctypes.byref(wp)) == 0
        x = torch.zeros((args.n, hp.value, wp.value, 4), device="cuda")
        assert L.mcb200_conv_rows_pad_input(ctypes.byref(s), ctypes.c_void_p(image.data_ptr()), ctypes.c_void_p(x.data_ptr()), None) == 0
        packed = torch.empty(L.mcb200_conv_rows_packed_weight_count(ctypes.byref(s)), device="cuda")
        assert L.mcb200_conv_rows_pack_weights(ctypes.byref(s), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(packed.data_ptr()), None) == 0
        assert L.mcb200_conv_rows_plan(ctypes.byref(s), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(packed.data_ptr()),
                                       ctypes.byref(plan)) == 0
    else:
        x = torch.randn((args.n, args.hw, args.hw, args.c), generator=g).cuda()
        packed = torch.empty(L.mcb200_conv_packed_weight_count(ctypes.byref(s)), device="cuda")
        assert L.mcb200_conv_pack_weights(ctypes.byref(s), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(packed.data_ptr()), None) == 0
        assert L.mcb200_conv_tc_plan(ctypes.byref(s), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(packed.data_ptr()),
                                     ctypes.byref(plan)) == 0
    out = torch.empty((args.n, s.ho, s.wo, args.cout), device="cuda")
    res = torch.randn((args.n, s.ho, s.wo, args.cout), generator=g).cuda() if args.residual else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ep = Epilogue()
    ep.residual_coeff = 1.0
    ep.act = 1
    if res is not None:
        ep.residual, ep.residual_ld = res.data_ptr(), args.cout
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    trace = (ctypes.c_longlong * (ROLES * SLOTS))()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for rep in range(args.reps):
        flush.zero_()                      # the layer's input comes from DRAM, as inside a network
        torch.cuda.synchronize()
        L.mcb200_conv_trace_read(trace)    # clears the device array
        ev0.record()
        rc = L.mcb200_conv_tc_launch(ctypes.byref(plan), ctypes.c_void_p(out.data_ptr()), args.cout, ctypes.byref(ep),
                                     ctypes.c_void_p(status.data_ptr()), None)
        ev1.record()
        assert rc == 0, rc
        torch.cuda.synchronize()
        slots = L.mcb200_conv_trace_read(trace)
        if slots == 0 and rep == args.reps - 1:
            print("layer n=%d c=%d %dx%d cout=%d k=%d: %.1f us (library without the trace: time only)"
                  % (args.n, args.c, args.hw, args.hw, args.cout, args.k, ev0.elapsed_time(ev1) * 1e3))
            return
    t = np.ctypeslib.as_array(trace).reshape(ROLES, SLOTS)
    mode = {0: "matrix", 1: "im2col", 2: "rows", 3: "halo"}[plan.im2col]
    print("layer n=%d c=%d %dx%d cout=%d k=%d stride=%d pad=%d: mode %s, tile width %d, cta pair %d, k-iterations %d, %.1f us"
          % (args.n, args.c, args.hw, args.hw, args.cout, args.k, args.stride, args.pad, mode, plan.block_n, plan.cta_pair,
             plan.k_iters, ev0.elapsed_time(ev1) * 1e3))
    for role, name in ((0, "producer A"), (1, "producer B"), (2, "MMA issuer")):
        v = t[role][t[role] > 0]
        pairs = v[: len(v) // 2 * 2].reshape(-1, 2)
        if len(pairs) < 2:
            continue
        work = (pairs[:, 1] - pairs[:, 0]).tolist()               # first stamp (wait over) -> second (issued)
        wait = (pairs[1:, 0] - pairs[:-1, 1]).tolist()            # issued -> next wait over
        print(summary(name + ": wait for the stage", wait))
        print(summary(name + ": issue", work))
        print("%-34s %d k-iterations in %d cycles = %.0f cycles each" % (name + ": overall", len(pairs), pairs[-1, 1] - pairs[0, 0],
                                                                      (pairs[-1, 1] - pairs[0, 0]) / max(1, len(pairs) - 1)))
    v = t[3][t[3] > 0]
    pairs = v[: len(v) // 2 * 2].reshape(-1, 2)
    if len(pairs) >= 2:
        print(summary("epilogue: wait for accumulator", (pairs[1:, 0] - pairs[:-1, 1]).tolist()))
        print(summary("epilogue: store the tile", (pairs[:, 1] - pairs[:, 0]).tolist()))
        print("epilogue: %d tiles, %.0f cycles per tile" % (len(pairs), (pairs[-1, 1] - pairs[0, 0]) / max(1, len(pairs) - 1)))
    c = t[4][t[4] > 0]
    c = c[: len(c) // 5 * 5].reshape(-1, 5)
    if len(c) >= 2:
        print("epilogue warp 0, per 32 x 32 chunk (staged epilogue), %d chunks:" % len(c))
        for name, col in (("  accumulator -> registers (tcgen05.ld)", 1), ("  wait for the slot / the residual", 2),
                          ("  tail arithmetic + write to the slot", 3), ("  fence + store issue", 4)):
            print(summary(name, (c[:, col] - c[:, col - 1]).tolist()))
        print(summary("  from store issue to the next chunk", (c[1:, 0] - c[:-1, 4]).tolist()))
    if args.dump:
        origin = min(int(t[r][0]) for r in range(4) if t[r][0] > 0)
        print("k-iteration  A: free issued | B: free issued | MMA: full issued   (cycles since the first stamp)")
        for i in range(args.dump):
            cells = []
            for r in range(3):
                cells.append("%7d %7d" % (int(t[r][2 * i]) - origin, int(t[r][2 * i + 1]) - origin) if t[r][2 * i + 1] > 0 else "      -       -")
            print("%4d   %s" % (i, " | ".join(cells)))
        ep = t[3][t[3] > 0]
        print("epilogue warp 0 (accumulator ready, tile stored):", [int(v) - origin for v in ep[: 2 * max(2, args.dump // max(1, plan.k_iters))]])
    # load latency: from the later of the two producers' issue stamps of a k-iteration to the MMA issuer seeing the stage full
    a = t[0][t[0] > 0]
    b = t[1][t[1] > 0]
    m = t[2][t[2] > 0]
    n = min(len(a), len(b), len(m)) // 2
    if n > 2:
        issued = np.maximum(a[1:2 * n:2], b[1:2 * n:2])
        full = m[0:2 * n:2]
        print(summary("loads issued -> stage seen full", (full - issued).tolist()))
        first = np.minimum(a[0:2 * n:2], b[0:2 * n:2])
        print(summary("stage free -> stage seen full", (full - first).tolist()))


if __name__ == "__main__":
    main()
