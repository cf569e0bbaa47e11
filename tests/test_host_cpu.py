"""Host-side behaviour of libcaffe.so that needs no GPU: model-file parsing, net
construction through the C API, error reporting, exported symbols."""
import ctypes
import glob
import os
import re

import numpy as np
import pytest

from conftest import ENGINE_LIB, REFERENCE_CHECKOUT, ROOT, pkg

REFERENCE_MODELS = os.path.join(REFERENCE_CHECKOUT, "example", "models")


def test_every_declared_symbol_is_exported(kernels):
    declared = set()
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")) + [os.path.join(ROOT, "include", "caffe", "c_api.h")]:
        text = open(header).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"\b(mcb200_\w+|Caffe\w+)\s*\(", text):
            declared.add(m.group(1))
    declared -= {"mcb200_conv_shape", "mcb200_epilogue", "mcb200_conv_plan", "mcb200_proposal_params",
                 "mcb200_detout_params"}
    assert len(declared) >= 45
    missing = [name for name in sorted(declared) if not hasattr(kernels, name)]
    assert not missing, missing


def test_build_and_inspect_net_without_a_device(capi, engine):
    wl = pkg("workloads")
    b = wl.resnet50(2)
    net = capi.Net(engine, b.text(), None, from_buffer=True)
    blobs = dict(net.blobs())
    assert blobs["data"].shape == (2, 3, 224, 224)
    assert blobs["conv1"].shape == (2, 64, 112, 112)
    assert blobs["pool1"].shape == (2, 64, 56, 56)      # ceil rule: 112 -> 56
    assert blobs["res5c"].shape == (2, 2048, 7, 7)
    assert blobs["prob"].shape == (2, 1000)
    params = net.params()
    assert len(params) == len(b.params)
    assert [n for n, _ in params][:5] == ["conv1_0", "bn_conv1_0", "bn_conv1_1", "bn_conv1_2", "scale_conv1_0"]
    weights = wl.init_params(b.params, seed=0)
    net.set_params(weights)
    back = dict(net.params())["fc1000_0"].data
    assert np.array_equal(back, weights["fc1000_0"])
    # reshape an input: the C API reports the new shape immediately
    blobs["data"].reshape(1, 3, 224, 224)
    assert blobs["data"].shape == (1, 3, 224, 224)
    net.close()


def test_ssd_and_proposal_shapes(capi, engine):
    wl = pkg("workloads")
    net = capi.Net(engine, wl.ssd300_vgg16(2).text(), None, from_buffer=True)
    blobs = dict(net.blobs())
    assert blobs["pool3"].shape == (2, 256, 38, 38)     # 75 -> 38
    assert blobs["fc6"].shape == (2, 1024, 19, 19)      # dilated 3x3 keeps 19
    assert blobs["mbox_loc"].shape == (2, 8732 * 4)
    assert blobs["mbox_conf_flatten"].shape == (2, 8732 * 21)
    assert blobs["mbox_priorbox"].shape == (1, 2, 8732 * 4)
    net.close()
    net = capi.Net(engine, wl.proposal(15).text(), None, from_buffer=True)
    assert dict(net.blobs())["rois"].shape == (300, 5)
    net.close()


def test_error_path_matches_the_c_api_contract(capi, engine):
    # missing files: -1 and a non-empty message (reference: tests/run_net.c:72-74)
    with pytest.raises(capi.CaffeError) as e:
        capi.Net(engine, "/nonexistent/net.prototxt", "/nonexistent/net.caffemodel")
    assert "File not found" in str(e.value)
    with pytest.raises(capi.CaffeError) as e:
        capi.Net(engine, 'layer { name: "x" type: "NoSuchLayer" top: "x" }', None, from_buffer=True)
    assert "Unknown layer type: NoSuchLayer" in str(e.value) and "Convolution" in str(e.value)
    with pytest.raises(capi.CaffeError) as e:
        capi.Net(engine, 'layer { name: "c" type: "ReLU" bottom: "nope" top: "c" }', None, from_buffer=True)
    assert "Unknown bottom blob 'nope'" in str(e.value)
    with pytest.raises(capi.CaffeError) as e:
        capi.Net(engine, 'layer { name: "r" type: "ReLU" top: "r" }', None, from_buffer=True)
    assert "first layer should be Input" in str(e.value) or "bottom blob" in str(e.value)
    with pytest.raises(capi.CaffeError):
        capi.Net(engine, "this is not a prototxt {{{", None, from_buffer=True)
    two = ('layer { name: "in" type: "Input" top: "a" input_param { shape { dim: 1 dim: 1 } } } '
           'layer { name: "s" type: "Split" bottom: "a" top: "a2" top: "a" }')
    with pytest.raises(capi.CaffeError) as e:
        capi.Net(engine, two, None, from_buffer=True)
    assert "produced by multiple sources" in str(e.value)


def test_weight_shape_mismatch_is_reported(capi, engine, tmp_path):
    wl = pkg("workloads")
    small = wl.NetBuilder("a")
    small.input([("data", (1, 4, 8, 8))])
    small.conv("conv", "data", "conv", 4, 8, 3)
    big = wl.NetBuilder("b")
    big.input([("data", (1, 4, 8, 8))])
    big.conv("conv", "data", "conv", 4, 16, 3)
    # serialise the 16-filter net's weights with the library's own writer path: build,
    # then read its params back through a caffemodel made by python's encoder below
    model = encode_caffemodel([("conv", [np.zeros((16, 4, 3, 3), np.float32), np.zeros(16, np.float32)])])
    with pytest.raises(capi.CaffeError) as e:
        capi.Net(engine, small.text(), model, from_buffer=True)
    assert "shape mismatch" in str(e.value)
    ok = capi.Net(engine, big.text(), model, from_buffer=True)
    ok.close()


def test_forward_without_device_fails_loudly(capi, engine):
    if engine.gpu_available():
        pytest.skip("a device is present")
    wl = pkg("workloads")
    net = capi.Net(engine, wl.conv_relu(1).text(), None, from_buffer=True)
    with pytest.raises(capi.CaffeError) as e:
        net.forward()
    assert "no CUDA device" in str(e.value) or "no CPU compute path" in str(e.value)
    net.close()


def test_set_mode_cpu_refuses_forward(capi, engine):
    wl = pkg("workloads")
    engine.set_mode(False, -1)
    net = capi.Net(engine, wl.conv_relu(1).text(), None, from_buffer=True)
    with pytest.raises(capi.CaffeError) as e:
        net.forward()
    assert "no CPU compute path" in str(e.value)
    net.close()
    if engine.gpu_available():
        engine.set_mode(True, 0)


# ---------------------------------------------------------------- wire-format fixtures

def _varint(v):
    out = bytearray()
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def _field(num, wire, payload):
    return _varint((num << 3) | wire) + payload


def _len(num, payload):
    return _field(num, 2, _varint(len(payload)) + payload)


def encode_blob(arr, legacy=False, packed=True):
    body = b""
    if legacy:
        dims = (list((1,) * (4 - arr.ndim)) + list(arr.shape))
        for i, d in enumerate(dims):
            body += _field(i + 1, 0, _varint(d))
    else:
        shape = b"".join(_varint(d) for d in arr.shape)
        body += _len(7, _len(1, shape))
    flat = arr.astype("<f4").reshape(-1)
    if packed:
        body += _len(5, flat.tobytes())
    else:
        body += b"".join(_field(5, 5, flat[i:i + 1].tobytes()) for i in range(flat.size))
    return body


def encode_caffemodel(layers, legacy=False, packed=True):
    """An independent encoder of the caffemodel wire format (NetParameter.layer = 100,
    LayerParameter.name = 1, .type = 2, .blobs = 7; BlobProto.shape = 7, .data = 5)."""
    net = _len(1, b"fixture")
    for name, blobs in layers:
        body = _len(1, name.encode()) + _len(2, b"Convolution")
        for b in blobs:
            body += _len(7, encode_blob(b, legacy=legacy, packed=packed))
        body += _field(99, 0, _varint(7))      # a field the schema does not know: skipped
        net += _len(100, body)
    return net


@pytest.mark.parametrize("legacy,packed", [(False, True), (True, True), (False, False)])
def test_caffemodel_decoding(capi, engine, legacy, packed):
    wl = pkg("workloads")
    b = wl.NetBuilder("w")
    b.input([("data", (1, 4, 8, 8))])
    b.conv("conv", "data", "conv", 4, 8, 3)
    rng = np.random.default_rng(1)
    w = rng.standard_normal((8, 4, 3, 3)).astype(np.float32)
    bias = rng.standard_normal(8).astype(np.float32)
    model = encode_caffemodel([("conv", [w, bias]), ("absent_layer", [w])], legacy=legacy, packed=packed)
    net = capi.Net(engine, b.text(), model, from_buffer=True)
    got = dict(net.params())
    assert np.array_equal(got["conv_0"].data, w)
    assert np.array_equal(got["conv_1"].data, bias)
    net.close()


@pytest.mark.skipif(not os.path.isdir(REFERENCE_MODELS), reason="reference checkout not present")
def test_reference_example_prototxts_parse(capi, engine):
    built = 0
    for path in sorted(glob.glob(os.path.join(REFERENCE_MODELS, "*", "*.prototxt"))):
        try:
            net = capi.Net(engine, path, "")
        except capi.CaffeError as e:
            # nets using layer types outside this engine's scope must fail with the registry message
            assert "Unknown layer type" in str(e), path
            continue
        assert len(net.blobs()) > 0
        net.close()
        built += 1
    assert built >= 10
    # the SSH detector (Deconvolution + Crop + Proposal) and the WGAN generator (Deconvolution +
    # BatchNorm on batch statistics + TanH) are among the ones that build
    for name in ("ssh/test_ssh.prototxt", "wgan/g.prototxt", "r-fcn/test_agnostic.prototxt"):
        net = capi.Net(engine, os.path.join(REFERENCE_MODELS, name), "")
        assert len(net.blobs()) > 3
        net.close()
    net = capi.Net(engine, os.path.join(REFERENCE_MODELS, "deeplandmark", "1_F.prototxt"),
                   os.path.join(REFERENCE_MODELS, "deeplandmark", "1_F.caffemodel"))
    assert float(np.abs(dict(net.params())["conv1_0"].data).sum()) > 0
    net.close()


def test_text_format_quirks(capi, engine):
    text = """
    name: 'quirks'  # single quotes and comments
    input: "data" input_dim: 1 input_dim:3 input_dim: 8 input_dim: 8
    layer { name: "c" type: "Convolution" bottom: "data" top: "c"
            convolution_param: { num_output: 2 kernel_size: 3; pad: 1, stride: 1 } }
    layer { name: "p" type: "Pooling" bottom: "c" top: "p" pooling_param < pool: AVE kernel_size: 2 stride: 2 > }
    """
    net = capi.Net(engine, text, None, from_buffer=True)
    blobs = dict(net.blobs())
    assert blobs["data"].shape == (1, 3, 8, 8)      # legacy input fields became an Input layer
    assert blobs["p"].shape == (1, 2, 4, 4)
    net.close()


def test_cli_built_on_public_headers_fails_loudly_without_a_device(tmp_path):
    """mini-caffe_b200/cli/benchmark.cc sees include/caffe/*.hpp only (the counterpart of mini-caffe's
    tools/benchmark.cpp).  Without a GPU it must stop with the engine's error, not compute on the host."""
    import subprocess
    exe = os.path.join(ROOT, "mini-caffe_b200", "lib", "benchmark")
    if not os.path.isfile(exe):
        pytest.skip("command-line tool not built")
    wl = pkg("workloads")
    proto = tmp_path / "net.prototxt"
    proto.write_text(wl.conv_relu(1).text())
    run = subprocess.run([exe, str(proto), "1", "-1"], capture_output=True, text=True, cwd=str(tmp_path), timeout=120)
    assert run.returncode == 1
    assert "no CPU compute path" in run.stderr
    usage = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert usage.returncode == 2 and "Usage" in usage.stderr


@pytest.mark.parametrize("owner_alive", [True, False])
def test_net_destroyed_by_another_thread_than_its_creator(capi, engine, owner_alive):
    """CaffeNetCreate on a worker thread, CaffeNetDestroy on the main thread (a common pattern).
    The memory pool is per thread: the blocks must find their way back to the pool they came from
    while that thread lives, and be freed when it has ended; the main thread's pool must neither
    receive them nor hand them out."""
    import threading
    wl = pkg("workloads")
    b = wl.conv_relu(2)
    weights = wl.init_params(b.params, seed=0)
    box = {}
    created, release = threading.Event(), threading.Event()

    def worker():
        net = capi.Net(engine, b.text(), None, from_buffer=True)
        net.set_params(weights)                      # host blocks of the parameters come from this thread's pool
        net.blob("data").data[...] = 1.0             # and the input's
        box["net"] = net
        created.set()
        if owner_alive:
            release.wait(30)
            # the pool took its blocks back: a new net of the same shapes reuses them
            again = capi.Net(engine, b.text(), None, from_buffer=True)
            again.set_params(weights)
            box["again"] = float(dict(again.params())["conv_0"].data.sum())
            again.close()

    t = threading.Thread(target=worker)
    t.start()
    assert created.wait(60)
    if not owner_alive:
        t.join()
    box["net"].close()                               # destroyed here, on the main thread
    release.set()
    t.join()
    if owner_alive:
        assert box["again"] == pytest.approx(float(weights["conv_0"].sum()), rel=1e-5)
    # the main thread's own pool still works
    own = capi.Net(engine, b.text(), None, from_buffer=True)
    own.set_params(weights)
    assert np.array_equal(dict(own.params())["conv_1"].data, weights["conv_1"])
    own.close()


V1_NET = """
name: "v1_style"
input: "data" input_dim: 2 input_dim: 3 input_dim: 16 input_dim: 16
layers { name: "conv1" type: CONVOLUTION bottom: "data" top: "conv1" blobs_lr: 1 blobs_lr: 2 weight_decay: 1 weight_decay: 0
         convolution_param { num_output: 8 kernel_size: 3 pad: 1 } }
layers { name: "relu1" type: RELU bottom: "conv1" top: "conv1" }
layers { name: "pool1" type: POOLING bottom: "conv1" top: "pool1" pooling_param { pool: MAX kernel_size: 2 stride: 2 } }
layers { name: "norm1" type: LRN bottom: "pool1" top: "norm1" lrn_param { local_size: 3 alpha: 0.0001 beta: 0.75 } }
layers { name: "fc" type: INNER_PRODUCT bottom: "norm1" top: "fc" inner_product_param { num_output: 5 } }
layers { name: "prob" type: SOFTMAX bottom: "fc" top: "prob" }
"""


def test_v1_layers_definitions_are_upgraded(capi, engine):
    """`layers { type: ENUM }` files (the format before `layer { type: "String" }`) load like in the
    reference (src/util/upgrade_proto.cpp:18-44): text definitions and binary weight files."""
    rng = np.random.default_rng(2)
    w = rng.standard_normal((8, 3, 3, 3)).astype(np.float32)
    bias = rng.standard_normal(8).astype(np.float32)
    # a V1 weight file: NetParameter.layers = 2; V1LayerParameter.name = 4, .type = 5 (CONVOLUTION = 4), .blobs = 6
    v1_layer = _len(4, b"conv1") + _field(5, 0, _varint(4)) + _len(6, encode_blob(w, legacy=True)) + \
        _len(6, encode_blob(bias, legacy=True))
    model = _len(1, b"v1_weights") + _len(2, v1_layer)
    net = capi.Net(engine, V1_NET, model, from_buffer=True)
    blobs = dict(net.blobs())
    assert blobs["data"].shape == (2, 3, 16, 16)
    assert blobs["pool1"].shape == (2, 8, 8, 8) and blobs["norm1"].shape == (2, 8, 8, 8)
    assert blobs["prob"].shape == (2, 5)
    params = dict(net.params())
    assert np.array_equal(params["conv1_0"].data, w) and np.array_equal(params["conv1_1"].data, bias)
    assert params["fc_0"].shape == (5, 8 * 8 * 8)
    net.close()


def test_mixed_v1_and_current_layer_definitions_are_refused(capi, engine):
    text = V1_NET + 'layer { name: "extra" type: "ReLU" bottom: "fc" top: "fc" }\n'
    with pytest.raises(capi.CaffeError) as err:
        capi.Net(engine, text, None, from_buffer=True)
    assert "both 'layer' and 'layers'" in str(err.value)
