"""Per-layer parity on the GPU against the reference CPU build: the layers that
are not exercised (or only in fused form) by the ResNet tests, edge shapes, and
MobileNet-v1 end to end."""
import numpy as np
import pytest

from conftest import pkg
from parity import assert_close, run_net

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_engine(engine):
    engine.set_mode(True, 0)
    return engine


def both(capi, gpu_engine, reflib, b, weights, x, outs, marks=()):
    got = run_net(capi, gpu_engine, b, weights, x, outs, marks=marks)
    want = run_net(capi, reflib, b, weights, x, outs, marks=marks)
    return got, want


def test_depthwise_and_grouped_convolution(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.NetBuilder("dw")
    b.input([("data", (3, 32, 17, 19))])
    b.conv("dw", "data", "dw", 32, 32, 3, stride=2, pad=1, group=32)          # depthwise kernel
    b.relu("dw_relu", "dw")
    b.conv("grp", "dw", "grp", 32, 48, 3, stride=1, pad=1, group=4)           # grouped: block-diagonal tiles
    b.conv("odd", "grp", "odd", 48, 10, 1)                                    # 10 outputs: unaligned rows
    b.conv("odd2", "odd", "odd2", 10, 6, 3, pad=1)                            # 10 input channels: padded copy
    weights = wl.init_params(b.params, seed=1)
    x = {"data": np.random.default_rng(2).standard_normal((3, 32, 17, 19)).astype(np.float32)}
    outs = ["dw", "grp", "odd", "odd2"]
    got, want = both(capi, gpu_engine, reflib, b, weights, x, outs, marks=outs)
    for name in outs:
        assert_close(got[name], want[name], name)
    assert tensor_core_launches(capi, gpu_engine, b, weights, x) == 3       # grp, odd, odd2


def tensor_core_launches(capi, engine, b, weights, x):
    """How many launches of the tensor-core convolution kernel one forward pass makes (the library's
    kernel timer brackets exactly those launches)."""
    import ctypes
    L = engine.lib
    L.mcb200_kernel_timing_end.restype = ctypes.c_longlong
    L.mcb200_kernel_timing_end.argtypes = [ctypes.POINTER(ctypes.c_double)]
    net = capi.Net(engine, b.text(), None, from_buffer=True)
    net.set_params(weights)
    net.forward(**x)
    L.mcb200_kernel_timing_begin()
    net.forward()
    ms = ctypes.c_double(0.0)
    count = int(L.mcb200_kernel_timing_end(ctypes.byref(ms)))
    net.close()
    return count


@pytest.mark.parametrize("case", [
    # name, N, Cin, H, W, Cout, k, stride, pad, dilation, group
    ("two_groups_5x5", 2, 96, 27, 27, 256, 5, 1, 2, 1, 2),          # 48 channels and 128 outputs per group
    ("cardinality_32", 2, 128, 28, 28, 128, 3, 1, 1, 1, 32),        # 4 channels, 4 outputs per group
    ("pointwise_three_groups", 3, 240, 14, 14, 240, 1, 1, 0, 1, 3),  # 80 channels per group: not a multiple of 32
    ("stride2_groups", 2, 64, 19, 23, 96, 3, 2, 1, 1, 8),
    ("channel_multiplier", 2, 24, 16, 16, 48, 3, 1, 1, 1, 24),      # one channel in, two out per group
    ("six_by_six", 2, 6, 12, 12, 6, 3, 1, 1, 1, 6),                 # depthwise with a channel count not divisible by 4
    ("dilated_groups", 1, 64, 20, 20, 64, 3, 1, 2, 2, 4),
    ("ragged_groups", 2, 36, 10, 10, 90, 3, 1, 1, 1, 9),            # 4 channels, 10 outputs per group: tiles cut groups
], ids=lambda c: c[0])
def test_grouped_convolution_on_the_tensor_cores(capi, gpu_engine, reflib, case):
    """Grouped layers (1 < group, not plain depthwise) run the tensor-core kernel: an N tile multiplies
    the channels of the groups it touches by a block-diagonal weight tile.  Against the reference's
    per-group GEMM loop (src/layers/base_conv_layer.cpp:265-270), with the fused tail."""
    name, n, cin, h, w, cout, k, stride, pad, dil, group = case
    wl = pkg("workloads")
    b = wl.NetBuilder("grouped")
    b.input([("data", (n, cin, h, w))])
    b.conv("c", "data", "c", cin, cout, k, stride=stride, pad=pad, dilation=dil, group=group, bias=True,
           bias_init="uniform")
    b.relu("c_relu", "c")
    weights = wl.init_params(b.params, seed=31)
    x = {"data": np.random.default_rng(32).standard_normal((n, cin, h, w)).astype(np.float32)}
    got, want = both(capi, gpu_engine, reflib, b, weights, x, ["c"])
    assert_close(got["c"], want["c"], name)
    assert tensor_core_launches(capi, gpu_engine, b, weights, x) == 1


@pytest.mark.parametrize("channels,size,k,stride,pad,cout", [
    (3, (23, 300), 3, 1, 1, 64),     # output rows of 300 pixels: three segments, the last one partial
    (3, (9, 257), 7, 2, 3, 24),      # 129 pixels per row: a second segment of one pixel
    (1, (6, 128), 5, 1, 2, 16),      # exactly one full segment, single channel
    (4, (5, 140), 3, 1, 0, 72),      # no padding, two N tiles
])
def test_first_layer_convolution_with_wide_rows(capi, gpu_engine, reflib, channels, size, k, stride, pad, cout):
    """Layers with at most four input channels run the tensor-core kernel's row mode; output rows wider
    than an M tile (128 pixels) are cut into segments."""
    wl = pkg("workloads")
    b = wl.NetBuilder("wide")
    b.input([("data", (2, channels) + size)])
    b.conv("c", "data", "c", channels, cout, k, stride=stride, pad=pad)
    b.relu("c_relu", "c")
    weights = wl.init_params(b.params, seed=21)
    x = {"data": np.random.default_rng(22).standard_normal((2, channels) + size).astype(np.float32)}
    got, want = both(capi, gpu_engine, reflib, b, weights, x, ["c"])
    assert got["c"].shape == want["c"].shape
    assert_close(got["c"], want["c"], "wide first layer")


@pytest.mark.parametrize("stride,size", [(1, (14, 14)), (2, (15, 9)), (1, (5, 3)), (2, (2, 2)), (1, (17, 23)),
                                         (2, (33, 19)), (1, (8, 8)), (2, (16, 17))])
def test_depthwise_3x3_sizes(capi, gpu_engine, reflib, stride, size):
    wl = pkg("workloads")
    b = wl.NetBuilder("dw3")
    b.input([("data", (2, 24) + size)])
    b.conv("dw", "data", "dw", 24, 24, 3, stride=stride, pad=1, group=24)
    weights = wl.init_params(b.params, seed=5)
    x = {"data": np.random.default_rng(6).standard_normal((2, 24) + size).astype(np.float32)}
    got, want = both(capi, gpu_engine, reflib, b, weights, x, ["dw"])
    assert np.abs(got["dw"] - want["dw"]).max() <= 2e-5


@pytest.mark.parametrize("method,k,stride,pad,size", [
    ("MAX", 3, 2, 0, (112, 112)), ("MAX", 2, 2, 0, (75, 75)), ("MAX", 3, 1, 1, (19, 19)),
    ("AVE", 3, 2, 1, (14, 15)), ("AVE", 2, 2, 1, (9, 9)), ("MAX", 3, 2, 1, (13, 11)),
])
def test_pooling_variants(capi, gpu_engine, reflib, method, k, stride, pad, size):
    wl = pkg("workloads")
    b = wl.NetBuilder("pool")
    c = 24
    b.input([("data", (2, c, size[0], size[1]))])
    b.pool("p", "data", "p", method, k=k, stride=stride, pad=pad)
    x = {"data": np.random.default_rng(3).standard_normal((2, c, size[0], size[1])).astype(np.float32)}
    got, want = both(capi, gpu_engine, reflib, b, {}, x, ["p"])
    assert got["p"].shape == want["p"].shape
    assert np.abs(got["p"] - want["p"]).max() <= 1e-6


def test_global_pooling_odd_channels(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.NetBuilder("gap")
    b.input([("data", (2, 7, 5, 6))])
    b.pool("g", "data", "g", "AVE", global_pooling=True)
    b.pool("m", "data", "m", "MAX", global_pooling=True)
    x = {"data": np.random.default_rng(4).standard_normal((2, 7, 5, 6)).astype(np.float32)}
    got, want = both(capi, gpu_engine, reflib, b, {}, x, ["g", "m"], marks=["g"])
    assert np.abs(got["g"] - want["g"]).max() <= 1e-6
    assert np.array_equal(got["m"], want["m"])


def test_global_pooling_wide_and_long_softmax_rows(capi, gpu_engine, reflib):
    """A classifier's tail: a pooling window over the whole 7 x 7 image with many channels (a block per
    image and 128 channels, partial sums added in a fixed order) and softmax over rows of hundreds of
    values (a block per row)."""
    wl = pkg("workloads")
    b = wl.NetBuilder("tail")
    b.input([("data", (3, 136, 7, 7)), ("scores", (5, 1000)), ("short", (2, 300))])
    b.pool("g", "data", "g", "AVE", global_pooling=True)
    b.pool("m", "data", "m", "MAX", global_pooling=True)
    b.softmax("p", "scores", "p", axis=1)
    b.softmax("q", "short", "q", axis=1)
    rng = np.random.default_rng(14)
    x = {"data": rng.standard_normal((3, 136, 7, 7)).astype(np.float32),
         "scores": rng.standard_normal((5, 1000)).astype(np.float32) * 4,
         "short": rng.standard_normal((2, 300)).astype(np.float32) * 4}
    got, want = both(capi, gpu_engine, reflib, b, {}, x, ["g", "m", "p", "q"], marks=["g", "p"])
    assert np.abs(got["g"] - want["g"]).max() <= 1e-6
    assert np.array_equal(got["m"], want["m"])
    for name in ("p", "q"):
        assert np.abs(got[name] - want[name]).max() <= 2e-6, name
        assert np.abs(got[name].sum(axis=1) - 1).max() <= 1e-5


def test_softmax_axes(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.NetBuilder("sm")
    b.input([("a", (4, 21, 5, 3)), ("b", (3, 50, 21))])
    b.softmax("s1", "a", "s1", axis=1)
    b.softmax("s2", "b", "s2", axis=2)
    b.softmax("s3", "b", "s3", axis=1)
    rng = np.random.default_rng(5)
    x = {"a": rng.standard_normal((4, 21, 5, 3)).astype(np.float32) * 3,
         "b": rng.standard_normal((3, 50, 21)).astype(np.float32) * 3}
    got, want = both(capi, gpu_engine, reflib, b, {}, x, ["s1", "s2", "s3"], marks=["s1", "s2"])
    for name in ("s1", "s2", "s3"):
        assert np.abs(got[name] - want[name]).max() <= 2e-6, name


def test_standalone_elementwise_layers(capi, gpu_engine, reflib):
    """BatchNorm / Scale / Bias / ReLU / PReLU / Eltwise not behind a convolution (no fusion)."""
    wl = pkg("workloads")
    b = wl.NetBuilder("elt")
    b.input([("x", (2, 12, 7, 9)), ("y", (2, 12, 7, 9))])
    b.batch_norm("bn", "x", 12)
    b.scale("sc", "x", 12)
    b.raw("lrelu", "ReLU", ["x"], ["lrelu"], "relu_param { negative_slope: 0.1 }")
    b.raw("pr", "PReLU", ["y"], ["pr"])
    b.params.append(("pr_0", (12,), "he", 4))
    b.raw("bias", "Bias", ["pr"], ["bias"], "bias_param { axis: 1 }")
    b.params.append(("bias_0", (12,), "he", 4))
    b.raw("sum", "Eltwise", ["lrelu", "bias"], ["sum"], "eltwise_param { operation: SUM coeff: 0.5 coeff: -2 }")
    b.raw("prod", "Eltwise", ["lrelu", "bias"], ["prod"], "eltwise_param { operation: PROD }")
    b.raw("mx", "Eltwise", ["lrelu", "bias", "sum"], ["mx"], "eltwise_param { operation: MAX }")
    b.raw("cat", "Concat", ["sum", "prod", "mx"], ["cat"], "concat_param { axis: 1 }")
    b.raw("cat2", "Concat", ["sum", "prod"], ["cat2"], "concat_param { axis: 2 }")
    weights = wl.init_params(b.params, seed=6, bn_identity=False)
    rng = np.random.default_rng(7)
    x = {"x": rng.standard_normal((2, 12, 7, 9)).astype(np.float32),
         "y": rng.standard_normal((2, 12, 7, 9)).astype(np.float32)}
    outs = ["lrelu", "pr", "bias", "sum", "prod", "mx", "cat", "cat2"]
    got, want = both(capi, gpu_engine, reflib, b, weights, x, outs, marks=outs)
    for name in outs:
        assert np.abs(got[name] - want[name]).max() <= 1e-5, name


def test_prelu_fused_behind_convolution(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.NetBuilder("convprelu")
    b.input([("data", (2, 16, 12, 12))])
    b.conv("c", "data", "c", 16, 40, 3, pad=1)
    b.raw("pr", "PReLU", ["c"], ["c"])
    b.params.append(("pr_0", (40,), "he", 4))
    b.raw("sh", "PReLU", ["c"], ["sh"], "prelu_param { channel_shared: true }")
    b.params.append(("sh_0", (), "he", 4))
    weights = wl.init_params(b.params, seed=8)
    x = {"data": np.random.default_rng(9).standard_normal((2, 16, 12, 12)).astype(np.float32)}
    got, want = both(capi, gpu_engine, reflib, b, weights, x, ["c", "sh"], marks=["c"])
    assert_close(got["c"], want["c"], "conv+prelu")
    assert_close(got["sh"], want["sh"], "shared prelu")


def test_normalize_permute_flatten_reshape(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.NetBuilder("misc")
    b.input([("data", (2, 20, 6, 5))])
    b.raw("norm", "Normalize", ["data"], ["norm"], "norm_param { across_spatial: false channel_shared: false }")
    b.params.append(("norm_0", (20,), "norm_scale", 0))
    b.raw("perm", "Permute", ["norm"], ["perm"], "permute_param { order: 0 order: 2 order: 3 order: 1 }")
    b.raw("perm2", "Permute", ["norm"], ["perm2"], "permute_param { order: 1 order: 0 order: 3 order: 2 }")
    b.raw("flat", "Flatten", ["perm"], ["flat"], "flatten_param { axis: 1 }")
    b.raw("resh", "Reshape", ["flat"], ["resh"], "reshape_param { shape { dim: 0 dim: -1 dim: 4 } }")
    b.raw("split", "Split", ["norm"], ["s1", "s2"])
    x = {"data": np.random.default_rng(10).standard_normal((2, 20, 6, 5)).astype(np.float32)}
    outs = ["norm", "perm", "perm2", "flat", "resh", "s1", "s2"]
    weights = wl.init_params(b.params, seed=1)
    got, want = both(capi, gpu_engine, reflib, b, weights, x, outs, marks=outs)
    for name in outs:
        assert got[name].shape == want[name].shape, name
        assert np.abs(got[name] - want[name]).max() <= 2e-5, name


def test_inner_product_variants(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.NetBuilder("ip")
    b.input([("data", (5, 8, 3, 4))])
    b.inner_product("fc1", "data", "fc1", 96, 33)                 # flattens (C, H, W) in NCHW order
    b.relu("fc1_relu", "fc1")
    b.raw("fc2", "InnerProduct", ["fc1"], ["fc2"], "inner_product_param { num_output: 7 bias_term: false transpose: true }")
    b.params.append(("fc2_0", (33, 7), "he", 33))
    b.inner_product("fc3", "fc2", "fc3", 7, 5)                     # K = 7: not a multiple of four
    weights = wl.init_params(b.params, seed=11)
    x = {"data": np.random.default_rng(12).standard_normal((5, 8, 3, 4)).astype(np.float32)}
    outs = ["fc1", "fc2", "fc3"]
    got, want = both(capi, gpu_engine, reflib, b, weights, x, outs, marks=outs)
    for name in outs:
        assert_close(got[name], want[name], name)


def test_weights_can_change_between_passes(capi, gpu_engine, reflib):
    """Folded scale/shift arrays and packed weights must follow writes through Net::params()."""
    wl = pkg("workloads")
    b = wl.NetBuilder("reload")
    b.input([("data", (1, 8, 10, 10))])
    b.conv_bn("c", "data", "c", 8, 16, 3, pad=1, bn_prefix="bn_", scale_prefix="scale_")
    x = {"data": np.random.default_rng(13).standard_normal((1, 8, 10, 10)).astype(np.float32)}
    eng = capi.Net(gpu_engine, b.text(), None, from_buffer=True)
    for seed in (1, 2):
        w = wl.init_params(b.params, seed=seed, bn_identity=False)
        eng.set_params(w)
        eng.forward(**x)
        want = run_net(capi, reflib, b, w, x, ["c"])["c"]
        assert_close(eng.blob("c").data.copy(), want, "pass %d" % seed)
    eng.close()


def test_mobilenet_v1_batch2(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.mobilenet_v1(2)
    weights = wl.init_params(b.params, seed=0)
    x = wl.normal_image_input(2, seed=0)
    outs = ["fc7", "prob"]
    marks = ["conv2_dw", "conv6_pw", "conv14_pw"]
    got, want = both(capi, gpu_engine, reflib, b, weights, x, outs + marks, marks=marks)
    for name in marks + outs:
        assert_close(got[name], want[name], name)


def test_resnet50_batch16(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.resnet50(16)
    weights = wl.init_params(b.params, seed=0)
    x = wl.image_input(16, seed=1)
    got, want = both(capi, gpu_engine, reflib, b, weights, x, ["fc1000"], marks=["res3d"])
    assert_close(got["fc1000"], want["fc1000"], "fc1000")
    # same top-1 class wherever the reference's margin between its two best logits is not tiny
    top = np.sort(want["fc1000"], axis=1)
    clear = (top[:, -1] - top[:, -2]) > 2e-2 * np.abs(top[:, -1])
    assert (np.argmax(got["fc1000"], 1)[clear] == np.argmax(want["fc1000"], 1)[clear]).all()


def test_scale_and_bias_with_the_factors_in_a_second_bottom(capi, gpu_engine, reflib):
    """Scale / Bias whose factors are data (a second bottom) or a learned blob over other axes than
    the channel axis (src/layers/scale_layer.cpp:47,72-113, bias_layer.cpp:40,45-83): per channel,
    per (image, channel), per (channel, row, column), scalar."""
    wl = pkg("workloads")
    b = wl.NetBuilder("scale2")
    b.input([("data", (2, 6, 5, 8)), ("per_channel", (6,)), ("per_image_channel", (2, 6)), ("per_pixel", (6, 5, 8))])
    b.conv("c", "data", "c", 6, 6, 3, pad=1)                                   # a tensor-core layer in front
    b.raw("s_ch", "Scale", ["c", "per_channel"], ["s_ch"], "scale_param { axis: 1 }")
    b.raw("s_nc", "Scale", ["c", "per_image_channel"], ["s_nc"], "scale_param { axis: 0 bias_term: true }")
    b.params.append(("s_nc_0", (2, 6), "uniform", 0))                          # the learned bias over (image, channel)
    b.raw("s_px", "Scale", ["s_ch", "per_pixel"], ["s_px"], "scale_param { axis: 1 }")
    b.raw("b_ch", "Bias", ["s_px", "per_channel"], ["b_ch"], "bias_param { axis: 1 }")
    b.raw("b_nc", "Bias", ["b_ch", "per_image_channel"], ["b_nc"], "bias_param { axis: 0 }")
    b.raw("s_all", "Scale", ["b_nc"], ["s_all"], "scale_param { axis: 0 num_axes: -1 bias_term: true }")
    b.params.append(("s_all_0", (2, 6, 5, 8), "uniform", 0))                   # learned, one factor per element
    b.params.append(("s_all_1", (2, 6, 5, 8), "uniform", 0))
    b.raw("s_one", "Scale", ["s_all"], ["s_one"], "scale_param { num_axes: 0 filler { value: 3 } }")
    weights = wl.init_params(b.params, seed=5)
    rng = np.random.default_rng(6)
    x = {"data": rng.standard_normal((2, 6, 5, 8)).astype(np.float32),
         "per_channel": rng.uniform(0.5, 1.5, (6,)).astype(np.float32),
         "per_image_channel": rng.uniform(-1.0, 1.0, (2, 6)).astype(np.float32),
         "per_pixel": rng.uniform(0.5, 1.5, (6, 5, 8)).astype(np.float32)}
    outs = ["s_ch", "s_nc", "s_px", "b_ch", "b_nc", "s_all", "s_one"]
    got, want = both(capi, gpu_engine, reflib, b, weights, x, outs, marks=outs)
    for name in outs:
        assert_close(got[name], want[name], name)
