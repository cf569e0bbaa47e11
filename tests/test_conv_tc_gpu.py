"""Parity of the tensor-core convolution kernel, called through the kernel-level
C ABI (include/mcb200_kernels.h), against an fp32 reference of the same op.

Tolerance: TF32 operands (10-bit mantissa) with fp32 accumulation; elementwise
|a-b| <= 2e-2 + 1e-2*|b| as the engine's contract states, and the error
normalised by the output's largest magnitude must stay below 2e-3.
"""
import ctypes
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


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
                ("out_bf16", ctypes.c_int), ("out_ptr", ctypes.c_void_p),
                ("res_ptr", ctypes.c_void_p), ("m_virtual", ctypes.c_int), ("strip_rows", ctypes.c_int)]


def aligned_plan():
    raw = ctypes.create_string_buffer(ctypes.sizeof(ConvPlan) + 64)
    addr = (ctypes.addressof(raw) + 63) & ~63
    plan = ConvPlan.from_address(addr)
    plan._keep = raw
    return plan


def run_conv(lib, x_nchw, w, *, stride=1, pad=0, dil=1, c_stride=None, scale=None, shift=None,
             residual=None, res_coeff=1.0, act=0, slope=0.0, prelu=None, expect_status=0):
    L = lib
    L.mcb200_conv_packed_weight_count.restype = ctypes.c_size_t
    n, c, h, wd = x_nchw.shape
    cout, _, kh, kw = w.shape
    cs = c_stride or c
    x_nhwc = torch.zeros((n, h, wd, cs), device="cuda", dtype=torch.float32)
    x_nhwc[..., :c] = x_nchw.permute(0, 2, 3, 1)
    s = ConvShape(n, h, wd, c, cs, cout, kh, kw, stride, stride, pad, pad, dil, dil, 1, 0, 0)
    assert L.mcb200_conv_out_shape(ctypes.byref(s)) == 0
    packed = torch.empty(L.mcb200_conv_packed_weight_count(ctypes.byref(s)), device="cuda", dtype=torch.float32)
    wdev = w.contiguous().cuda()
    assert L.mcb200_conv_pack_weights(ctypes.byref(s), ctypes.c_void_p(wdev.data_ptr()),
                                      ctypes.c_void_p(packed.data_ptr()), None) == 0
    plan = aligned_plan()
    rc = L.mcb200_conv_tc_plan(ctypes.byref(s), ctypes.c_void_p(x_nhwc.data_ptr()),
                               ctypes.c_void_p(packed.data_ptr()), ctypes.byref(plan))
    assert rc == 0, rc
    out = torch.full((n, s.ho, s.wo, cout), float("nan"), device="cuda", dtype=torch.float32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    ep = Epilogue()
    ep.residual_coeff = res_coeff
    keep = []
    for name, t in (("scale", scale), ("shift", shift), ("prelu", prelu)):
        if t is not None:
            d = t.contiguous().cuda()
            keep.append(d)
            setattr(ep, name, d.data_ptr())
    if residual is not None:
        r = residual.permute(0, 2, 3, 1).contiguous().cuda()
        keep.append(r)
        ep.residual = r.data_ptr()
        ep.residual_ld = cout
    ep.act = act
    ep.slope = slope
    rc = L.mcb200_conv_tc_launch(ctypes.byref(plan), ctypes.c_void_p(out.data_ptr()), cout, ctypes.byref(ep),
                                 ctypes.c_void_p(status.data_ptr()), None)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert int(status.item()) == expect_status, "status word %d (1: a barrier wait timed out)" % int(status.item())
    return out.permute(0, 3, 1, 2).contiguous(), plan


def reference(x, w, *, stride, pad, dil, scale, shift, residual, res_coeff, act, slope, prelu):
    y = torch.nn.functional.conv2d(x.double(), w.double(), None, stride, pad, dil)
    if scale is not None:
        y = y * scale.double().view(1, -1, 1, 1)
    if shift is not None:
        y = y + shift.double().view(1, -1, 1, 1)
    if residual is not None:
        y = y + res_coeff * residual.double()
    if act == 1:
        y = torch.where(y > 0, y, y * slope)
    elif act == 2:
        y = torch.where(y > 0, y, y * prelu.double().view(1, -1, 1, 1))
    return y.float()


CASES = [
    # name, N, C, H, W, Cout, k, stride, pad, dil, c_stride
    ("pointwise_gemm", 1, 64, 25, 40, 64, 1, 1, 0, 1, None),
    ("cfg1_3x3", 2, 64, 56, 56, 64, 3, 1, 1, 1, None),
    ("pointwise_wide", 2, 256, 14, 14, 1000, 1, 1, 0, 1, None),
    ("3x3_stride2", 3, 128, 28, 28, 128, 3, 2, 1, 1, None),
    ("1x1_stride2", 2, 256, 56, 56, 512, 1, 2, 0, 1, None),
    ("7x7_stride2_rgb", 2, 3, 224, 224, 64, 7, 2, 3, 1, 4),
    ("3x3_dilated6", 1, 512, 19, 19, 1024, 3, 1, 6, 6, None),
    ("odd_sizes", 3, 20, 13, 17, 24, 3, 1, 1, 1, None),
    ("tiny_1x1x1", 1, 4, 1, 1, 8, 1, 1, 0, 1, None),
    ("5x5_pad2", 2, 32, 9, 11, 96, 5, 1, 2, 1, None),
    ("inner_product", 16, 2048, 1, 1, 1000, 1, 1, 0, 1, None),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_conv_tc_matches_fp32(kernels, case):
    name, n, c, h, w, cout, k, stride, pad, dil, cs = case
    g = torch.Generator().manual_seed(1234)
    x = torch.randn((n, c, h, w), generator=g)
    wt = torch.randn((cout, c, k, k), generator=g) * (2.0 / (c * k * k)) ** 0.5
    got, plan = run_conv(kernels, x.cuda(), wt, stride=stride, pad=pad, dil=dil, c_stride=cs)
    want = reference(x, wt, stride=stride, pad=pad, dil=dil, scale=None, shift=None, residual=None,
                     res_coeff=1.0, act=0, slope=0.0, prelu=None)
    got = got.cpu()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    err = (got - want).abs()
    assert (err <= 2e-2 + 1e-2 * want.abs()).all(), float(err.max())
    assert float(err.max() / want.abs().max()) < 2e-3


def test_conv_tc_fused_tail(kernels):
    g = torch.Generator().manual_seed(7)
    n, c, h, w, cout = 2, 64, 20, 20, 200
    x = torch.randn((n, c, h, w), generator=g)
    wt = torch.randn((cout, c, 3, 3), generator=g) * 0.05
    scale = torch.rand(cout, generator=g) + 0.5
    shift = torch.randn(cout, generator=g)
    res = torch.randn((n, cout, h, w), generator=g)
    prelu = torch.rand(cout, generator=g) * 0.3
    for act, slope in ((0, 0.0), (1, 0.0), (1, 0.1), (2, 0.0)):
        kw = dict(stride=1, pad=1, dil=1, scale=scale, shift=shift, residual=res, res_coeff=0.75, act=act,
                  slope=slope, prelu=prelu if act == 2 else None)
        got, _ = run_conv(kernels, x.cuda(), wt, **kw)
        want = reference(x, wt, **kw)
        err = (got.cpu() - want).abs()
        assert (err <= 2e-2 + 1e-2 * want.abs()).all(), (act, slope, float(err.max()))


def _with_planner(block_n, pairing, fn, halo="0"):
    """Runs fn() with the planner's tile-width, CTA-pair and halo-mode overrides set (halo mode is
    off unless asked for: the tests that compare variants bit for bit need the same K order)."""
    saved = {k: os.environ.get(k) for k in ("MCB200_BLOCK_N", "MCB200_CTA_PAIR", "MCB200_HALO")}
    os.environ["MCB200_BLOCK_N"] = str(block_n)
    os.environ["MCB200_CTA_PAIR"] = pairing
    os.environ["MCB200_HALO"] = halo
    try:
        return fn()
    finally:
        for k, v in saved.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v


@pytest.mark.parametrize("case", [
    # name, N, C, H, W, Cout, k, tile width, with residual
    ("odd_m_tiles_3x3", 1, 256, 19, 19, 256, 3, 256, False),     # 361 pixels: 3 M tiles, the last CTA of a pair idles
    ("many_tiles_per_cluster", 16, 128, 56, 56, 128, 3, 128, False),  # 196 pair units over at most 74 clusters
    ("pointwise_residual", 4, 512, 28, 28, 256, 1, 256, True),
    ("wide_two_n_tiles", 2, 128, 28, 28, 512, 3, 256, True),
    ("ragged_cout", 2, 64, 20, 20, 200, 3, 128, True),           # last N tile 72 columns wide
], ids=lambda c: c[0])
def test_cta_pairs_match_single_ctas(kernels, case):
    """The two-CTA (tcgen05 cta_group::2) variant accumulates every output element over the same
    K sequence as the one-CTA variant, so the two must agree bit for bit."""
    name, n, c, h, w, cout, k, block_n, with_res = case
    g = torch.Generator().manual_seed(99)
    x = torch.randn((n, c, h, w), generator=g)
    wt = torch.randn((cout, c, k, k), generator=g) * (2.0 / (c * k * k)) ** 0.5
    res = torch.randn((n, cout, h, w), generator=g) if with_res else None
    scale = torch.rand(cout, generator=g) + 0.5
    shift = torch.randn(cout, generator=g)
    kw = dict(stride=1, pad=k // 2, dil=1, scale=scale, shift=shift, residual=res, res_coeff=1.0, act=1, slope=0.0)
    single, plan_single = _with_planner(block_n, "0", lambda: run_conv(kernels, x.cuda(), wt, **kw))
    paired, plan_paired = _with_planner(block_n, "1", lambda: run_conv(kernels, x.cuda(), wt, **kw))
    assert plan_single.block_n == block_n and plan_paired.block_n == block_n
    assert plan_single.cta_pair == 0 and plan_paired.cta_pair == 1
    assert torch.equal(single, paired)
    want = reference(x, wt, prelu=None, **kw)
    err = (paired.cpu() - want).abs()
    assert (err <= 2e-2 + 1e-2 * want.abs()).all(), float(err.max())


@pytest.mark.parametrize("block_n", [64, 128, 256])
def test_every_tile_width_gives_the_same_result(kernels, block_n):
    """Tile width only changes how the output is cut up, not the arithmetic."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn((2, 96, 24, 24), generator=g)
    wt = torch.randn((320, 96, 3, 3), generator=g) * 0.03
    kw = dict(stride=1, pad=1, dil=1, scale=None, shift=None, residual=None, res_coeff=1.0, act=0, slope=0.0)
    base, _ = _with_planner(64, "0", lambda: run_conv(kernels, x.cuda(), wt, **kw))
    got, plan = _with_planner(block_n, "0", lambda: run_conv(kernels, x.cuda(), wt, **kw))
    assert plan.block_n == block_n
    assert torch.equal(base, got)


# ---------------------------------------------------------------- bfloat16 storage (opt-in)

def run_conv_bf16(lib, x_nchw, w, *, out_bf16, stride=1, pad=0, dil=1, scale=None, shift=None, residual=None,
                  act=0):
    """The same kernel on bfloat16 activations / weights / residual (mcb200_conv_tc_plan_bf16 and
    mcb200_conv_tc_launch_bf16); the inputs are converted with the library's own copy kernel."""
    L = lib
    L.mcb200_conv_packed_weight_count_bf16.restype = ctypes.c_size_t
    n, c, h, wd = x_nchw.shape
    cout, _, kh, kw = w.shape
    x32 = x_nchw.permute(0, 2, 3, 1).contiguous().cuda()
    x16 = torch.empty(x32.shape, device="cuda", dtype=torch.bfloat16)
    assert L.mcb200_f32_to_bf16(ctypes.c_void_p(x32.data_ptr()), ctypes.c_void_p(x16.data_ptr()),
                                ctypes.c_size_t(x32.numel()), None) == 0
    assert torch.equal(x16, x32.to(torch.bfloat16))          # round to nearest even, like torch
    s = ConvShape(n, h, wd, c, c, cout, kh, kw, stride, stride, pad, pad, dil, dil, 1, 0, 0)
    assert L.mcb200_conv_out_shape(ctypes.byref(s)) == 0
    packed = torch.empty(L.mcb200_conv_packed_weight_count_bf16(ctypes.byref(s)), device="cuda", dtype=torch.bfloat16)
    wdev = w.contiguous().cuda()
    assert L.mcb200_conv_pack_weights_bf16(ctypes.byref(s), ctypes.c_void_p(wdev.data_ptr()),
                                           ctypes.c_void_p(packed.data_ptr()), None) == 0
    plan = aligned_plan()
    rc = L.mcb200_conv_tc_plan_bf16(ctypes.byref(s), ctypes.c_void_p(x16.data_ptr()),
                                    ctypes.c_void_p(packed.data_ptr()), ctypes.byref(plan))
    assert rc == 0, rc
    assert plan.operand_bf16 == 1
    out = torch.full((n, s.ho, s.wo, cout), float("nan"), device="cuda",
                     dtype=torch.bfloat16 if out_bf16 else torch.float32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    ep = Epilogue()
    ep.residual_coeff = 1.0
    keep = []
    for name, t in (("scale", scale), ("shift", shift)):
        if t is not None:
            d = t.contiguous().cuda()
            keep.append(d)
            setattr(ep, name, d.data_ptr())
    if residual is not None:
        r = residual.permute(0, 2, 3, 1).contiguous().cuda().to(torch.bfloat16)
        keep.append(r)
        ep.residual = r.data_ptr()
        ep.residual_ld = cout
    ep.act = act
    # the fp32 entry point refuses a bfloat16 plan
    assert L.mcb200_conv_tc_launch(ctypes.byref(plan), ctypes.c_void_p(out.data_ptr()), cout, ctypes.byref(ep),
                                   ctypes.c_void_p(status.data_ptr()), None) == -8
    rc = L.mcb200_conv_tc_launch_bf16(ctypes.byref(plan), ctypes.c_void_p(out.data_ptr()), 1 if out_bf16 else 0, cout,
                                      ctypes.byref(ep), ctypes.c_void_p(status.data_ptr()), None)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "kernel reported a timed-out barrier wait"
    if out_bf16:
        widened = torch.empty(out.shape, device="cuda", dtype=torch.float32)
        assert L.mcb200_bf16_to_f32(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(widened.data_ptr()),
                                    ctypes.c_size_t(out.numel()), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(widened, out.float())
        out = widened
    return out.permute(0, 3, 1, 2).contiguous().cpu(), plan


BF16_CASES = [
    # name, N, C, H, W, Cout, k, stride, pad, dil, residual, out_bf16
    ("pointwise_res", 2, 64, 28, 28, 256, 1, 1, 0, 1, True, True),
    ("pointwise_to_fp32", 2, 256, 14, 14, 64, 1, 1, 0, 1, False, False),
    ("res_to_fp32", 1, 512, 7, 7, 2048, 1, 1, 0, 1, True, False),
    ("3x3", 2, 64, 56, 56, 64, 3, 1, 1, 1, False, True),
    ("3x3_stride2_pairs", 3, 128, 28, 28, 128, 3, 2, 1, 1, False, True),
    ("1x1_stride2", 2, 256, 28, 28, 512, 1, 2, 0, 1, False, True),
    ("odd_channels", 3, 24, 13, 17, 40, 3, 1, 1, 1, True, True),      # 24 channels: one partial block of 64
    ("wide_k", 2, 1024, 14, 14, 256, 1, 1, 0, 1, False, True),
    ("unaligned_out", 2, 32, 9, 11, 20, 3, 1, 1, 1, True, True),      # 20 output channels: plain bfloat16 stores
]


@pytest.mark.parametrize("case", BF16_CASES, ids=[c[0] for c in BF16_CASES])
def test_conv_tc_bfloat16_storage(kernels, case):
    """Operands rounded to bfloat16 exactly as the kernel sees them, products accumulated in double:
    what is left is the fp32 accumulation (relative 1e-5 of the largest value) and, for bfloat16 output,
    one rounding of the result (2^-9 relative)."""
    name, n, c, h, w, cout, k, stride, pad, dil, with_res, out_bf16 = case
    g = torch.Generator().manual_seed(4321)
    x = torch.randn((n, c, h, w), generator=g)
    wt = torch.randn((cout, c, k, k), generator=g) * (2.0 / (c * k * k)) ** 0.5
    scale = torch.rand(cout, generator=g) + 0.5
    shift = torch.randn(cout, generator=g)
    ho = (h + 2 * pad - dil * (k - 1) - 1) // stride + 1
    wo = (w + 2 * pad - dil * (k - 1) - 1) // stride + 1
    res = torch.randn((n, cout, ho, wo), generator=g) if with_res else None
    got, plan = run_conv_bf16(kernels, x, wt, out_bf16=out_bf16, stride=stride, pad=pad, dil=dil, scale=scale,
                              shift=shift, residual=res, act=1)
    xr, wr = x.to(torch.bfloat16).float(), wt.to(torch.bfloat16).float()
    rr = res.to(torch.bfloat16).float() if with_res else None
    want = reference(xr, wr, stride=stride, pad=pad, dil=dil, scale=scale, shift=shift, residual=rr, res_coeff=1.0,
                     act=1, slope=0.0, prelu=None)
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    err = (got - want).abs()
    bound = 2e-5 * float(want.abs().max()) + (want.abs() * 2.0 ** -8 if out_bf16 else 0.0)
    assert (err <= bound).all(), (name, float(err.max()), plan.block_n, plan.cta_pair)


HALO_CASES = [
    # name, N, C, H, W, Cout, k, pad, dil
    ("cfg1_3x3", 2, 64, 56, 56, 64, 3, 1, 1),
    ("wide_rows_3x3", 1, 32, 9, 300, 40, 3, 1, 1),       # rows longer than a tile (SSD300's first layers)
    ("seven_wide", 4, 512, 7, 7, 512, 3, 1, 1),          # 2 of 9 virtual positions per row are dropped
    ("odd_sizes", 3, 20, 13, 17, 24, 3, 1, 1),           # partial channel block, ragged Cout
    ("5x5_pad2", 2, 32, 9, 11, 96, 5, 2, 1),
    ("dilated6", 1, 512, 19, 19, 1024, 3, 6, 6),         # SSD fc6: taps 6 pixel rows apart in the strip
    ("no_padding", 2, 64, 20, 20, 200, 3, 0, 1),
    ("one_row", 2, 16, 1, 50, 32, 3, 1, 1),              # H = 1: two of three filter rows read only padding
]


@pytest.mark.parametrize("case", HALO_CASES, ids=[c[0] for c in HALO_CASES])
def test_halo_mode_matches_fp32(kernels, case):
    """Halo mode (the taps of a filter row read one shared strip of input pixels at shifted
    shared-memory addresses; tiles run over a virtual output grid with widened rows) against the
    same fp64 reference as the im2col mode, for every tile width / pairing it can run with."""
    name, n, c, h, w, cout, k, pad, dil = case
    g = torch.Generator().manual_seed(4321)
    x = torch.randn((n, c, h, w), generator=g)
    wt = torch.randn((cout, c, k, k), generator=g) * (2.0 / (c * k * k)) ** 0.5
    want = reference(x, wt, stride=1, pad=pad, dil=dil, scale=None, shift=None, residual=None, res_coeff=1.0, act=0,
                     slope=0.0, prelu=None)
    ran = 0
    for block_n, pairing in ((64, "0"), (128, "0"), (128, "1"), (256, "1")):
        if block_n > 64 and block_n // 2 >= cout:
            continue
        got, plan = _with_planner(block_n, pairing, lambda: run_conv(kernels, x.cuda(), wt, stride=1, pad=pad, dil=dil),
                                  halo="1")
        if plan.im2col != 3:       # this width's stage does not fit three times (wide filters): im2col mode ran
            continue
        ran += 1
        assert plan.block_n == block_n and plan.cta_pair == int(pairing)
        assert plan.strip_rows == 128 + (k - 1) * dil
        got = got.cpu()
        assert torch.isfinite(got).all()        # the output was NaN-filled: every element was stored
        err = (got - want).abs()
        assert (err <= 2e-2 + 1e-2 * want.abs()).all(), (block_n, pairing, float(err.max()))
        assert float(err.max() / want.abs().max()) < 2e-3
    assert ran >= 1


def test_halo_mode_fused_tail_and_unaligned_rows(kernels):
    """Scale / shift / residual / activations through the halo mode's store path, with 16-byte
    aligned rows (128-bit accesses) and with a channel count that is not a multiple of four
    (element-wise accesses)."""
    g = torch.Generator().manual_seed(8)
    for cout in (200, 70):
        n, c, h, w = 2, 64, 20, 20
        x = torch.randn((n, c, h, w), generator=g)
        wt = torch.randn((cout, c, 3, 3), generator=g) * 0.05
        scale = torch.rand(cout, generator=g) + 0.5
        shift = torch.randn(cout, generator=g)
        res = torch.randn((n, cout, h, w), generator=g)
        prelu = torch.rand(cout, generator=g) * 0.3
        for act, slope in ((0, 0.0), (1, 0.0), (1, 0.1), (2, 0.0)):
            kw = dict(stride=1, pad=1, dil=1, scale=scale, shift=shift, residual=res, res_coeff=0.75, act=act,
                      slope=slope, prelu=prelu if act == 2 else None)
            got, plan = _with_planner(128, "0", lambda: run_conv(kernels, x.cuda(), wt, **kw), halo="1")
            assert plan.im2col == 3
            want = reference(x, wt, **kw)
            err = (got.cpu() - want).abs()
            assert (err <= 2e-2 + 1e-2 * want.abs()).all(), (cout, act, slope, float(err.max()))


def test_planner_takes_halo_mode_for_the_benchmark_layers(kernels):
    """Without overrides the 3 x 3 layers of the benchmark networks run in halo mode where it was
    measured to pay (rows of at least 16 or at most 8 output pixels), whatever the batch size: the
    two modes sum over K in different orders, so the choice must not depend on the batch."""
    for c, hw, cout, mode in ((64, 56, 64, 3), (128, 28, 128, 3), (256, 14, 256, 1), (512, 7, 512, 3), (512, 19, 512, 3),
                              (256, 10, 512, 1)):
        for n in (1, 8):
            x = torch.zeros((n, c, hw, hw), device="cuda")
            wt = torch.zeros((cout, c, 3, 3))
            _, plan = run_conv(kernels, x, wt, stride=1, pad=1, dil=1)
            assert plan.im2col == mode, (c, hw, n, plan.im2col)


def test_planner_widths_and_pairing_for_measured_layers(kernels):
    """Planner rules that were set from interleaved runs of the benchmark networks: halo mode keeps to
    128-column tiles (paired where there are two M tiles), 256-column tiles pair from 16
    k-iterations, 128-column tiles from 17, and the 128 -> 512 layers of ResNet-50's third stage take
    128-column tiles.  Width and pairing do not change the order of the sums over K."""
    cases = [
        # n, c, hw, cout, k, stride, pad -> mode, width, pair
        (8, 512, 38, 512, 3, 1, 1, 3, 128, 1),      # VGG conv4_2 at 300 x 300
        (8, 256, 75, 256, 3, 1, 1, 3, 128, 1),      # VGG conv3_2
        (64, 512, 28, 1024, 1, 2, 0, 1, 256, 1),    # ResNet-50 res4a_branch1: 16 k-iterations
        (64, 512, 28, 128, 1, 1, 0, 0, 128, 0),     # res3b_branch2a: 16 k-iterations at 128 columns
        (64, 128, 28, 512, 1, 1, 0, 0, 128, 0),     # res3b_branch2c: four k-iterations, many waves
    ]
    for n, c, hw, cout, k, stride, pad, mode, width, pair in cases:
        x = torch.zeros((n, c, hw, hw), device="cuda")
        wt = torch.zeros((cout, c, k, k))
        _, plan = run_conv(kernels, x, wt, stride=stride, pad=pad, dil=1)
        assert (plan.im2col, plan.block_n, plan.cta_pair) == (mode, width, pair), (c, hw, cout, plan.im2col, plan.block_n,
                                                                                   plan.cta_pair)


@pytest.mark.parametrize("halo", ["0", "1"])
def test_bounded_waits_run_out_and_the_context_stays_usable(kernels, halo):
    """Every barrier wait of the kernel is bounded.  The test hook makes the weight producer leave out
    its last loads, so the stage they belong to never completes: with a short limit the waits on it
    run out, the CTA aborts (roles leave their loops, tensor memory is freed), the status word reads
    1, and the launch returns.  Nothing faults or hangs; the next launch computes correctly."""
    g = torch.Generator().manual_seed(77)
    x = torch.randn((1, 64, 12, 10), generator=g)                 # 120 output pixels: a single tile
    wt = torch.randn((64, 64, 3, 3), generator=g) * 0.05
    kernels.mcb200_conv_set_wait_limit.restype = ctypes.c_longlong
    kernels.mcb200_conv_set_wait_limit.argtypes = [ctypes.c_longlong]
    previous = kernels.mcb200_conv_set_wait_limit(2000000)        # about a millisecond
    try:
        kernels.mcb200_conv_test_drop_weight_load()
        _with_planner(64, "0", lambda: run_conv(kernels, x.cuda(), wt, stride=1, pad=1, dil=1, expect_status=1), halo=halo)
        got, _ = _with_planner(64, "0", lambda: run_conv(kernels, x.cuda(), wt, stride=1, pad=1, dil=1), halo=halo)
    finally:
        assert kernels.mcb200_conv_set_wait_limit(previous) == 2000000
    want = reference(x, wt, stride=1, pad=1, dil=1, scale=None, shift=None, residual=None, res_coeff=1.0, act=0,
                     slope=0.0, prelu=None)
    err = (got.cpu() - want).abs()
    assert (err <= 2e-2 + 1e-2 * want.abs()).all(), float(err.max())


def test_bounded_waits_run_out_in_a_cta_pair(kernels):
    g = torch.Generator().manual_seed(78)
    x = torch.randn((1, 128, 16, 16), generator=g)                # 256 pixels: one pair of tiles
    wt = torch.randn((128, 128, 3, 3), generator=g) * 0.05
    kernels.mcb200_conv_set_wait_limit.restype = ctypes.c_longlong
    kernels.mcb200_conv_set_wait_limit.argtypes = [ctypes.c_longlong]
    previous = kernels.mcb200_conv_set_wait_limit(2000000)
    try:
        kernels.mcb200_conv_test_drop_weight_load()
        _, plan = _with_planner(128, "1", lambda: run_conv(kernels, x.cuda(), wt, stride=1, pad=1, dil=1, expect_status=1))
        assert plan.cta_pair == 1
        got, _ = _with_planner(128, "1", lambda: run_conv(kernels, x.cuda(), wt, stride=1, pad=1, dil=1))
    finally:
        kernels.mcb200_conv_set_wait_limit(previous)
    want = reference(x, wt, stride=1, pad=1, dil=1, scale=None, shift=None, residual=None, res_coeff=1.0, act=0,
                     slope=0.0, prelu=None)
    assert ((got.cpu() - want).abs() <= 2e-2 + 1e-2 * want.abs()).all()
