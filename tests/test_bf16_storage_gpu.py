"""bfloat16 storage, the engine's precision opt-in (environment MINICAFFE_PRECISION=bf16, read when a
net is constructed): blobs that callers cannot see and that only tensor-core convolutions (channel
counts multiples of eight) or 2x2 / 3x3 max pooling read are stored as bfloat16, and a convolution whose
input is such a blob computes on bfloat16 operands.

Stated bound for this mode, looser than the TF32 one: elementwise

    |a - b| <= 1e-1 * max(1, rms(b)) + 4e-2 * |b|

against the reference's fp32 CPU results (bfloat16 carries 8 significant bits, i.e. 2^-9 relative per
rounding, and a 50-layer net rounds every activation once per layer: measured on ResNet-50, the
largest error of a late blob is about 1 % of the blob's peak and 7 % of its RMS, four times the TF32
figure), and the default fp32 / TF32
behaviour must be untouched when the variable is absent.
"""
import numpy as np
import pytest

from conftest import pkg
from parity import assert_close, error_stats, run_net

pytestmark = pytest.mark.gpu

BF16_ATOL = 1e-1
BF16_RTOL = 4e-2


@pytest.fixture(scope="module")
def gpu_engine(engine):
    engine.set_mode(True, 0)
    return engine


def run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, outs, marks=()):
    monkeypatch.delenv("MINICAFFE_PRECISION", raising=False)
    wide = run_net(capi, gpu_engine, b, weights, x, outs, marks=marks)
    monkeypatch.setenv("MINICAFFE_PRECISION", "bf16")
    narrow = run_net(capi, gpu_engine, b, weights, x, outs, marks=marks)
    monkeypatch.delenv("MINICAFFE_PRECISION", raising=False)
    return wide, narrow


def test_single_convolution(monkeypatch, capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.conv_relu(2)
    weights = wl.init_params(b.params, seed=0)
    x = wl.conv_relu_input(2)
    out = "conv"
    wide, narrow = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, [out])
    want = run_net(capi, reflib, b, weights, x, [out])
    assert_close(wide[out], want[out], "tf32")
    # A layer computes on bfloat16 only if its input is a bfloat16-stored blob; here both the input and
    # the output are visible to the caller (fp32), so the mode changes nothing.
    assert np.array_equal(wide[out], narrow[out])


def test_resnet50_batch4(monkeypatch, capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.resnet50(4)
    weights = wl.init_params(b.params, seed=3)
    x = wl.image_input(4, seed=5)
    outs = ["res2c", "res4f", "pool5", "fc1000", "prob"]
    marks = ["res2c", "res4f"]
    wide, narrow = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, outs, marks=marks)
    want = run_net(capi, reflib, b, weights, x, outs, marks=marks)
    assert not np.array_equal(wide["res2c"], narrow["res2c"])      # the two modes really are different arithmetic
    for name in outs:
        st = assert_close(narrow[name], want[name], "bf16 " + name, atol=BF16_ATOL, rtol=BF16_RTOL)
        tf = error_stats(wide[name], want[name])
        print("%-8s bf16 max|err|/peak %.2e   tf32 %.2e" % (name, st["max_abs_over_peak"], tf["max_abs_over_peak"]))
    assert np.array_equal(np.argmax(narrow["prob"], axis=1), np.argmax(want["prob"], axis=1))


def test_mixed_consumers(monkeypatch, capi, gpu_engine, reflib):
    """Blobs that cross the border between bfloat16 and fp32 layers: a convolution output read by a
    pooling layer and by another convolution, a residual that comes from a pooling layer, a grouped
    convolution (direct kernel, fp32) between two tensor-core ones, 20 output channels (not a
    multiple of eight: that layer stays TF32), and a standalone Eltwise."""
    wl = pkg("workloads")
    b = wl.NetBuilder("mixed")
    b.input([("data", (3, 16, 20, 24))])
    b.conv("a", "data", "a", 16, 32, 3, pad=1)
    b.relu("a_relu", "a")
    b.raw("pool", "Pooling", ["a"], ["pool"], "pooling_param { pool: MAX kernel_size: 3 stride: 1 pad: 1 }")
    b.conv("b", "a", "b", 32, 32, 1)
    b.conv("c", "b", "c", 32, 32, 3, pad=1)
    b.raw("sum", "Eltwise", ["c", "pool"], ["sum"], "eltwise_param { operation: SUM }")
    b.relu("sum_relu", "sum")
    b.conv("g", "sum", "g", 32, 32, 3, pad=1, group=4)
    b.conv("d", "g", "d", 32, 20, 1)
    b.conv("e", "d", "e", 20, 16, 3, pad=1)
    b.raw("twice", "Eltwise", ["e", "e"], ["twice"], "eltwise_param { operation: SUM }")
    weights = wl.init_params(b.params, seed=11)
    x = {"data": np.random.default_rng(12).standard_normal((3, 16, 20, 24)).astype(np.float32)}
    outs = ["a", "sum", "g", "d", "twice"]
    marks = ["a", "sum", "g", "d"]
    wide, narrow = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, outs, marks=marks)
    want = run_net(capi, reflib, b, weights, x, outs, marks=marks)
    for name in outs:
        assert_close(wide[name], want[name], "tf32 " + name)
        assert_close(narrow[name], want[name], "bf16 " + name, atol=BF16_ATOL, rtol=BF16_RTOL)
    # nothing marked: more blobs become bfloat16-only; the final result must still agree
    wide2, narrow2 = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, ["twice"])
    assert np.array_equal(wide2["twice"], wide["twice"])
    assert_close(narrow2["twice"], want["twice"], "bf16 unmarked", atol=BF16_ATOL, rtol=BF16_RTOL)


def test_repeated_passes_and_new_input(monkeypatch, capi, gpu_engine):
    """The bfloat16 copies are rebuilt on every pass: a second pass with another input gives that
    input's result, and a repeat of the first input repeats the first result bit for bit."""
    wl = pkg("workloads")
    monkeypatch.setenv("MINICAFFE_PRECISION", "bf16")
    b = wl.resnet50(2)
    net = capi.Net(gpu_engine, b.text(), None, from_buffer=True)
    net.set_params(wl.init_params(b.params, seed=1))
    x1, x2 = wl.image_input(2, seed=1), wl.image_input(2, seed=2)
    net.forward(**x1)
    first = net.blob("fc1000").data.copy()
    net.forward(**x2)
    second = net.blob("fc1000").data.copy()
    net.forward(**x1)
    again = net.blob("fc1000").data.copy()
    net.close()
    assert not np.array_equal(first, second)
    assert np.array_equal(first, again)


def test_vgg_style_trunk_with_pooling(monkeypatch, capi, gpu_engine, reflib):
    """Convolution groups separated by max pooling (2x2 stride 2, ceil-rounded odd sizes; 3x3 stride 1
    pad 1): the pooled blobs stay bfloat16, a first layer with three input channels (row mode, fp32
    image) writes bfloat16 directly, and an average pooling layer in between takes fp32."""
    wl = pkg("workloads")
    b = wl.NetBuilder("vgg_like")
    b.input([("data", (2, 3, 37, 45))])
    b.conv("c1_1", "data", "c1_1", 3, 32, 3, pad=1)
    b.relu("r1_1", "c1_1")
    b.conv("c1_2", "c1_1", "c1_2", 32, 32, 3, pad=1)
    b.relu("r1_2", "c1_2")
    b.raw("p1", "Pooling", ["c1_2"], ["p1"], "pooling_param { pool: MAX kernel_size: 2 stride: 2 }")
    b.conv("c2_1", "p1", "c2_1", 32, 64, 3, pad=1)
    b.relu("r2_1", "c2_1")
    b.raw("p2", "Pooling", ["c2_1"], ["p2"], "pooling_param { pool: MAX kernel_size: 3 stride: 1 pad: 1 }")
    b.conv("c3_1", "p2", "c3_1", 64, 64, 3, pad=2, dilation=2)
    b.relu("r3_1", "c3_1")
    b.raw("p3", "Pooling", ["c3_1"], ["p3"], "pooling_param { pool: AVE kernel_size: 2 stride: 2 }")
    b.conv("c4_1", "p3", "c4_1", 64, 48, 1)
    weights = wl.init_params(b.params, seed=31)
    x = {"data": np.random.default_rng(32).standard_normal((2, 3, 37, 45)).astype(np.float32)}
    for marks in ([], ["p1", "p2", "c3_1"]):
        outs = ["c4_1"] + marks
        wide, narrow = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, outs, marks=marks)
        want = run_net(capi, reflib, b, weights, x, outs, marks=marks)
        for name in outs:
            assert_close(wide[name], want[name], "tf32 " + name)
            assert_close(narrow[name], want[name], "bf16 " + name, atol=BF16_ATOL, rtol=BF16_RTOL)
        assert not np.array_equal(wide["c4_1"], narrow["c4_1"])


def test_ssd300_heads(monkeypatch, capi, gpu_engine, reflib):
    """SSD300 (VGG-16 trunk, dilated fc6, L2Norm, six multibox heads) at batch 1: box regressions and
    class scores in front of DetectionOutput against the reference."""
    wl = pkg("workloads")
    b = wl.ssd300_vgg16(1, with_detection_output=False)
    weights = wl.init_params(b.params, seed=2)
    x = wl.ssd_input(1, seed=4)
    outs = ["mbox_loc", "mbox_conf_flatten"]
    wide, narrow = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, outs, marks=outs)
    want = run_net(capi, reflib, b, weights, x, outs, marks=outs)
    for name in outs:
        assert_close(narrow[name], want[name], "bf16 " + name, atol=BF16_ATOL, rtol=BF16_RTOL)
        print(name, error_stats(narrow[name], want[name]), error_stats(wide[name], want[name]))


def _forward(capi, engine, builder, weights, feed, outs, marks=()):
    net = capi.Net(engine, builder.text(), None, from_buffer=True)
    for m in marks:
        net.mark_output(m)
    net.set_params(weights)
    net.forward(**feed)
    res = {o: net.blob(o).data.copy() for o in outs}
    net.close()
    return res


def test_full_size_batches_are_batch_invariant(monkeypatch, capi, gpu_engine):
    """ResNet-50 at batch 64 and SSD300 at batch 32 with bfloat16 storage: every image comes out bit for
    bit as it does in a small batch (whose results the tests above compare with the reference)."""
    wl = pkg("workloads")
    monkeypatch.setenv("MINICAFFE_PRECISION", "bf16")
    weights = wl.init_params(wl.resnet50(4).params, seed=0)
    x = wl.image_input(64, seed=0)["data"]
    big = _forward(capi, gpu_engine, wl.resnet50(64), weights, {"data": x}, ["fc1000", "prob"])
    ref = _forward(capi, gpu_engine, wl.resnet50(4), weights, {"data": x[60:64]}, ["fc1000"])
    assert np.isfinite(big["fc1000"]).all()
    assert np.abs(big["prob"].sum(axis=1) - 1.0).max() < 1e-4
    assert np.array_equal(big["fc1000"][60:64].view(np.uint32), ref["fc1000"].view(np.uint32))

    weights = wl.init_params(wl.ssd300_vgg16(2).params, seed=0)
    x = wl.ssd_input(32, seed=0)["data"]
    outs = ["mbox_loc", "mbox_conf_flatten"]
    big = _forward(capi, gpu_engine, wl.ssd300_vgg16(32), weights, {"data": x}, outs + ["detection_out"], marks=outs)
    ref = _forward(capi, gpu_engine, wl.ssd300_vgg16(2), weights, {"data": x[30:32]}, outs, marks=outs)
    for name in outs:
        assert np.array_equal(big[name][30:32].view(np.uint32), ref[name].view(np.uint32)), name
    rows = big["detection_out"]
    assert rows.shape[-1] == 7 and np.isfinite(rows).all()


def test_mobilenet_v1_and_depthwise_shapes(monkeypatch, capi, gpu_engine, reflib):
    """Depthwise 3x3 layers (stride 1 and 2, odd sizes) read and write bfloat16 between bfloat16
    pointwise convolutions; MobileNet-v1 end to end."""
    wl = pkg("workloads")
    b = wl.NetBuilder("dw_chain")
    b.input([("data", (2, 16, 23, 17))])
    b.conv("pw0", "data", "pw0", 16, 24, 1)
    b.relu("r0", "pw0")
    b.conv("dw1", "pw0", "dw1", 24, 24, 3, stride=2, pad=1, group=24)
    b.relu("r1", "dw1")
    b.conv("pw1", "dw1", "pw1", 24, 40, 1)
    b.relu("r2", "pw1")
    b.conv("dw2", "pw1", "dw2", 40, 40, 3, stride=1, pad=1, group=40)
    b.conv("pw2", "dw2", "pw2", 40, 16, 1)
    weights = wl.init_params(b.params, seed=41)
    x = {"data": np.random.default_rng(42).standard_normal((2, 16, 23, 17)).astype(np.float32)}
    for marks in ([], ["dw1", "pw1"]):
        outs = ["pw2"] + marks
        wide, narrow = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, outs, marks=marks)
        want = run_net(capi, reflib, b, weights, x, outs, marks=marks)
        for name in outs:
            assert_close(wide[name], want[name], "tf32 " + name)
            assert_close(narrow[name], want[name], "bf16 " + name, atol=BF16_ATOL, rtol=BF16_RTOL)
        assert not np.array_equal(wide["pw2"], narrow["pw2"])

    b = wl.mobilenet_v1(2)
    weights = wl.init_params(b.params, seed=0)
    x = wl.normal_image_input(2, seed=7)
    outs = ["prob"]
    wide, narrow = run_both_precisions(monkeypatch, capi, gpu_engine, b, weights, x, outs)
    want = run_net(capi, reflib, b, weights, x, outs)
    assert_close(narrow["prob"], want["prob"], "bf16 mobilenet prob", atol=BF16_ATOL, rtol=BF16_RTOL)
    assert not np.array_equal(wide["prob"], narrow["prob"])
    print("mobilenet prob", error_stats(narrow["prob"], want["prob"]), error_stats(wide["prob"], want["prob"]))
