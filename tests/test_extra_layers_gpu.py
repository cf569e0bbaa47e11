"""Deconvolution, Crop, Slice, BN and LRN (the layer types of the shipped SSH / WGAN / older example
nets) against the reference project's CPU code.  Deconvolution runs on the tensor cores (TF32
tolerance); with MCB200_CONV_DIRECT=1 it runs on the plain fp32 kernel, and then everything here is
fp32 on both sides and agrees to float rounding.  Copies are compared bit for bit."""
import contextlib
import os

import numpy as np
import pytest

from conftest import pkg
from parity import run_net

pytestmark = pytest.mark.gpu

COPIES = ("crop", "crop1", "s0", "s1", "s2", "e0", "e1")


@pytest.fixture(scope="module")
def gpu_engine(engine):
    engine.set_mode(True, 0)
    return engine


@contextlib.contextmanager
def plain_kernels(on):
    """With `on`, Convolution / Deconvolution layers constructed inside run on the fp32 kernels."""
    saved = os.environ.get("MCB200_CONV_DIRECT")
    if on:
        os.environ["MCB200_CONV_DIRECT"] = "1"
    else:
        os.environ.pop("MCB200_CONV_DIRECT", None)
    try:
        yield
    finally:
        if saved is None:
            os.environ.pop("MCB200_CONV_DIRECT", None)
        else:
            os.environ["MCB200_CONV_DIRECT"] = saved


def _check(got, want, fp32):
    from parity import assert_close
    for name in want:
        assert got[name].shape == want[name].shape, name
        if fp32:
            scale = max(1.0, float(np.abs(want[name]).max()))
            assert float(np.abs(got[name] - want[name]).max()) <= 2e-5 * scale, name
        else:
            assert_close(got[name], want[name], name)


@pytest.mark.parametrize("fp32", [False, True], ids=["tensor_cores", "plain_kernels"])
def test_extra_layers_against_the_reference(capi, gpu_engine, reflib, fp32):
    wl = pkg("workloads")
    for batch, seed in ((2, 1), (1, 2), (5, 3)):
        b = wl.extra_layers_net(batch)
        weights = wl.init_params(b.params, seed=5 + seed, bn_identity=False)
        x = wl.extra_layers_input(batch, seed=seed)
        outs = list(wl.EXTRA_LAYER_OUTPUTS)
        with plain_kernels(fp32):
            got = run_net(capi, gpu_engine, b, weights, x, outs, marks=outs)
        want = run_net(capi, reflib, b, weights, x, outs, marks=outs)
        _check(got, want, fp32)
        for name in COPIES:
            # same values moved around: identical wherever the source tensor is identical
            src = "up" if name in ("crop", "crop1", "e0", "e1") else "up_g"
            if np.array_equal(got[src], want[src]):
                assert np.array_equal(got[name], want[name]), name


@pytest.mark.parametrize("fp32", [False, True], ids=["tensor_cores", "plain_kernels"])
def test_extra_layers_golden_fixture(capi, gpu_engine, fp32):
    """The committed fixture (made by the reference itself) does not need the compiled reference."""
    wl = pkg("workloads")
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "extra_layers.npz"))
    b = wl.extra_layers_net(2)
    weights = {k[2:]: g[k] for k in g.files if k.startswith("w_")}
    outs = list(wl.EXTRA_LAYER_OUTPUTS)
    with plain_kernels(fp32):
        got = run_net(capi, gpu_engine, b, weights, {"data": g["in_data"], "like": np.zeros((2, 4, 13, 11), np.float32)},
                      outs, marks=outs)
    _check(got, {name: g["out_" + name] for name in outs}, fp32)


def test_ssh_style_upsampling_head(capi, gpu_engine, reflib):
    """Convolution -> Deconvolution (x2) -> Crop to the finer map -> Eltwise SUM -> Convolution + ReLU:
    the context-module pattern of the shipped SSH detector, with the tensor-core convolutions around
    the new layers (TF32 tolerance)."""
    from parity import assert_close
    wl = pkg("workloads")
    b = wl.NetBuilder("ssh_head")
    b.input([("coarse", (1, 32, 10, 13)), ("fine", (1, 32, 19, 25))])
    b.conv("reduce", "coarse", "reduce", 32, 16, 1)
    b.raw("up", "Deconvolution", ["reduce"], ["up"],
          "convolution_param { num_output: 16 kernel_size: 4 stride: 2 pad: 1 group: 16 bias_term: false }")
    b.params.append(("up_0", (16, 1, 4, 4), "he", 16))
    b.conv("lateral", "fine", "lateral", 32, 16, 1)
    b.raw("crop", "Crop", ["up", "lateral"], ["crop"], "crop_param { axis: 2 offset: 0 }")
    b.eltwise_sum("sum", ["lateral", "crop"], "sum")
    b.conv("out", "sum", "out", 16, 16, 3, pad=1)
    b.relu("relu", "out")
    weights = wl.init_params(b.params, seed=2)
    rng = np.random.default_rng(5)
    x = {"coarse": rng.standard_normal((1, 32, 10, 13)).astype(np.float32),
         "fine": rng.standard_normal((1, 32, 19, 25)).astype(np.float32)}
    got = run_net(capi, gpu_engine, b, weights, x, ["out"])
    want = run_net(capi, reflib, b, weights, x, ["out"])
    assert_close(got["out"], want["out"], "out")


def test_wgan_style_generator(capi, gpu_engine, reflib):
    """Input noise -> (Deconvolution -> BatchNorm on batch statistics -> Scale -> ReLU) x 3 -> Deconvolution
    -> TanH: the structure of the shipped WGAN generator (example/models/wgan/g.prototxt), smaller."""
    wl = pkg("workloads")
    b = wl.NetBuilder("generator")
    batch = 4
    b.input([("z", (batch, 16, 1, 1))])
    prev, cin = "z", 16
    for i, (cout, k, stride, pad) in enumerate([(32, 4, 1, 0), (16, 4, 2, 1), (8, 4, 2, 1)]):
        name = "deconv%d" % i
        b.raw(name, "Deconvolution", [prev], [name],
              "convolution_param { num_output: %d kernel_size: %d stride: %d pad: %d bias_term: false }" %
              (cout, k, stride, pad))
        b.params.append((name + "_0", (cin, cout, k, k), "he", cin))
        b.raw("bn%d" % i, "BatchNorm", [name], [name], "batch_norm_param { use_global_stats: false }")
        for j, kind in enumerate(("bn_mean", "bn_var", "one")):
            b.params.append(("bn%d_%d" % (i, j), (cout,) if j < 2 else (1,), kind, 0))
        b.scale("scale%d" % i, name, cout)
        b.relu("relu%d" % i, name)
        prev, cin = name, cout
    b.raw("out", "Deconvolution", [prev], ["out"], "convolution_param { num_output: 3 kernel_size: 4 stride: 2 pad: 1 }")
    b.params.append(("out_0", (cin, 3, 4, 4), "he", cin))
    b.params.append(("out_1", (3,), "uniform", 0))
    b.raw("tanh", "TanH", ["out"], ["image"])
    weights = wl.init_params(b.params, seed=11, bn_identity=False)
    z = {"z": np.random.default_rng(12).standard_normal((batch, 16, 1, 1)).astype(np.float32)}
    from parity import assert_close
    from test_layers_gpu import tensor_core_launches
    want = run_net(capi, reflib, b, weights, z, ["image"], marks=["deconv1"])
    assert float(np.abs(want["image"]).max()) > 0.05
    # the four Deconvolution layers on the tensor cores (each as the convolution, with a reversed
    # filter, of its input spread `stride` apart over zeros)
    got = run_net(capi, gpu_engine, b, weights, z, ["image"], marks=["deconv1"])
    assert got["image"].shape == (batch, 3, 32, 32)
    assert_close(got["image"], want["image"], "generator image")
    assert tensor_core_launches(capi, gpu_engine, b, weights, z) == 4
    # and on the plain fp32 kernel: float rounding only
    with plain_kernels(True):
        got = run_net(capi, gpu_engine, b, weights, z, ["image"], marks=["deconv1"])
    assert float(np.abs(got["image"] - want["image"]).max()) <= 5e-5


def test_sigmoid(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.NetBuilder("sig")
    b.input([("data", (3, 5, 4, 6))])
    b.raw("s", "Sigmoid", ["data"], ["s"])
    x = {"data": (np.random.default_rng(1).standard_normal((3, 5, 4, 6)) * 4).astype(np.float32)}
    got = run_net(capi, gpu_engine, b, {}, x, ["s"])
    want = run_net(capi, reflib, b, {}, x, ["s"])
    assert float(np.abs(got["s"] - want["s"]).max()) <= 1e-6
