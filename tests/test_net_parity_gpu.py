"""End-to-end parity: generated networks run through libcaffe.so on the GPU and
through the reference project's own CPU code (oracle/_ref), same weights, same
inputs.  Tolerance for TF32 tensor-core layers: |a-b| <= 2e-2 + 1e-2*|b|."""
import numpy as np
import pytest

from conftest import pkg
from parity import assert_close, run_net

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_engine(engine):
    engine.set_mode(True, 0)
    return engine


@pytest.mark.parametrize("batch", [1, 32])
def test_conv_relu_config(capi, gpu_engine, reflib, batch):
    wl = pkg("workloads")
    b = wl.conv_relu(batch)
    weights = wl.init_params(b.params, seed=0)
    inputs = wl.conv_relu_input(batch, seed=0)
    got = run_net(capi, gpu_engine, b, weights, inputs, ["conv"])
    want = run_net(capi, reflib, b, weights, inputs, ["conv"])
    assert_close(got["conv"], want["conv"], "conv+relu b=%d" % batch)


def small_residual_net(wl, batch, bn_identity):
    b = wl.NetBuilder("mini_resnet")
    b.input([("data", (batch, 3, 32, 32))])
    b.conv_bn("stem", "data", "stem", 3, 32, 3, stride=1, pad=1, bn_prefix="bn_", scale_prefix="scale_")
    b.pool("pool1", "stem", "pool1", "MAX", k=3, stride=2)
    b.conv_bn("short", "pool1", "short", 32, 64, 1, relu=False, bn_prefix="bn_", scale_prefix="scale_")
    b.conv_bn("a", "pool1", "a", 32, 16, 1, bn_prefix="bn_", scale_prefix="scale_")
    b.conv_bn("b", "a", "b", 16, 16, 3, pad=1, bn_prefix="bn_", scale_prefix="scale_")
    b.conv_bn("c", "b", "c", 16, 64, 1, relu=False, bn_prefix="bn_", scale_prefix="scale_")
    b.eltwise_sum("res", ["short", "c"], "res")
    b.relu("res_relu", "res")
    b.pool("gap", "res", "gap", "AVE", global_pooling=True)
    b.inner_product("fc", "gap", "fc", 64, 10)
    b.softmax("prob", "fc", "prob")
    return b


@pytest.mark.parametrize("bn_identity", [True, False])
def test_small_residual_net(capi, gpu_engine, reflib, bn_identity):
    wl = pkg("workloads")
    b = small_residual_net(wl, 4, bn_identity)
    weights = wl.init_params(b.params, seed=3, bn_identity=bn_identity)
    x = {"data": np.random.default_rng(5).standard_normal((4, 3, 32, 32)).astype(np.float32)}
    outs = ["fc", "prob"]
    got = run_net(capi, gpu_engine, b, weights, x, outs)
    want = run_net(capi, reflib, b, weights, x, outs)
    for name in outs:
        assert_close(got[name], want[name], name)


def test_marked_outputs_block_fusion(capi, gpu_engine, reflib):
    """Marking an intermediate blob must keep it readable (no fusion through it)
    and must not change any result."""
    wl = pkg("workloads")
    b = small_residual_net(wl, 2, False)
    weights = wl.init_params(b.params, seed=4, bn_identity=False)
    x = {"data": np.random.default_rng(6).standard_normal((2, 3, 32, 32)).astype(np.float32)}
    marks = ["pool1", "c", "short", "res", "gap"]
    got = run_net(capi, gpu_engine, b, weights, x, marks + ["prob"], marks=marks)
    want = run_net(capi, reflib, b, weights, x, marks + ["prob"], marks=marks)
    for name in marks + ["prob"]:
        assert_close(got[name], want[name], name)


def test_resnet50_batch2(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.resnet50(2)
    weights = wl.init_params(b.params, seed=0)
    x = wl.image_input(2, seed=0)
    outs = ["fc1000", "prob"]
    marks = ["pool1", "res2c", "res3d", "res4f", "res5c"]
    got = run_net(capi, gpu_engine, b, weights, x, outs + marks, marks=marks)
    want = run_net(capi, reflib, b, weights, x, outs + marks, marks=marks)
    for name in marks + outs:
        assert_close(got[name], want[name], name)


def test_batch_invariance(capi, gpu_engine):
    """Same image at batch 1, 2, 1: identical class scores in every slot (the one
    numeric check the reference's own tests make, tests/run_net.cpp:274-321)."""
    wl = pkg("workloads")
    b = small_residual_net(wl, 1, False)
    weights = wl.init_params(b.params, seed=9, bn_identity=False)
    img = np.random.default_rng(10).standard_normal((1, 3, 32, 32)).astype(np.float32)
    net = capi.Net(gpu_engine, b.text(), None, from_buffer=True)
    net.set_params(weights)
    net.forward(data=img)
    p1 = net.blob("prob").data.copy()
    net.forward(data=np.concatenate([img, img]))
    p2 = net.blob("prob").data.copy()
    net.forward(data=img)
    p3 = net.blob("prob").data.copy()
    assert p2.shape == (2, 10)
    assert np.abs(p2[0] - p1[0]).max() < 1e-6
    assert np.abs(p2[1] - p1[0]).max() < 1e-6
    assert np.abs(p3[0] - p1[0]).max() < 1e-6


def test_cli_on_public_headers_runs_a_net(tmp_path):
    """The command-line tool written against the public C++ headers builds a net from a prototxt
    file, runs it on GPU 0 and writes the profile, like mini-caffe's tools/benchmark."""
    import json
    import os
    import subprocess
    wl = pkg("workloads")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "mini-caffe_b200", "lib", "benchmark")
    assert os.path.isfile(exe), "run __graft_entry__.build() first"
    proto = tmp_path / "resnet.prototxt"
    proto.write_text(wl.resnet50(2).text())
    run = subprocess.run([exe, str(proto), "3", "0"], capture_output=True, text=True, cwd=str(tmp_path), timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert run.stderr.count("Forward costs") == 3
    events = json.load(open(tmp_path / "profile.json"))["traceEvents"]
    assert any(e["name"] == "res2a_branch2b" for e in events)


def test_folded_model_files_run_the_same(capi, gpu_engine, tmp_path):
    """fuse_bn's output files through the engine: same function as the unfolded files (the engine
    folds the unfolded ones in memory, the tool folded the others on disk)."""
    import os
    import subprocess
    from test_fuse_bn_cpu import EXE, build_case
    if not os.path.isfile(EXE):
        pytest.skip("fuse_bn not built")
    wl = pkg("workloads")
    b, weights, proto, model = build_case(wl, tmp_path)
    subprocess.run([EXE, "--net", str(proto), "--weight", str(model)], check=True, capture_output=True, timeout=120)
    x = np.random.default_rng(8).standard_normal((2, 6, 12, 10)).astype(np.float32)
    outs = {}
    for tag, p, m in (("orig", proto, model), ("fold", tmp_path / "net_nobn.prototxt", tmp_path / "net_nobn.caffemodel")):
        net = capi.Net(gpu_engine, str(p), str(m))
        net.forward(data=x)
        outs[tag] = {name: net.blob(name).data.copy() for name in ("gap", "c3")}
        net.close()
    for name in ("gap", "c3"):
        assert_close(outs["fold"][name], outs["orig"][name], name)


def test_net_destroyed_by_another_thread_while_its_creator_keeps_working(capi, gpu_engine):
    """A net is created and run on a worker thread and destroyed on the main thread while the
    worker's stream is still busy with other nets.  Streams and memory pools are per thread: the
    destroyed net's device blocks must go back to the worker's pool only after the work that uses
    them has drained, so the worker's later results are what they were before."""
    import threading
    wl = pkg("workloads")
    b = small_residual_net(wl, 8, False)
    weights = wl.init_params(b.params, seed=21, bn_identity=False)
    x = np.random.default_rng(22).standard_normal((8, 3, 32, 32)).astype(np.float32)
    box = {"results": []}
    created, destroyed = threading.Event(), threading.Event()

    def run_once():
        net = capi.Net(gpu_engine, b.text(), None, from_buffer=True)
        net.set_params(weights)
        net.forward(data=x)
        out = net.blob("prob").data.copy()
        return net, out

    def worker():
        try:
            gpu_engine.set_mode(True, 0)
            keep, first = run_once()
            box["first"] = first
            box["net"] = keep
            created.set()
            for _ in range(6):                       # keeps the stream busy around the foreign destroy
                net, out = run_once()
                box["results"].append(out)
                net.close()
            destroyed.wait(60)
            for _ in range(3):                       # these allocations may reuse the returned blocks
                net, out = run_once()
                box["results"].append(out)
                net.close()
        except BaseException as exc:                 # noqa: BLE001
            box["error"] = exc
            created.set()

    t = threading.Thread(target=worker)
    t.start()
    assert created.wait(120)
    assert "error" not in box, box.get("error")
    box["net"].close()                               # on the main thread
    destroyed.set()
    t.join()
    assert "error" not in box, box.get("error")
    assert len(box["results"]) == 9
    for out in box["results"]:
        assert np.array_equal(out.view(np.uint32), box["first"].view(np.uint32))


def test_forward_reports_a_kernel_that_gave_up_waiting_and_recovers(capi, gpu_engine):
    """The status word a convolution kernel raises when its bounded barrier waits run out (made to
    happen here through the library's test hook, on the host's terms) turns into the API's error:
    CaffeNetForward returns -1 with a message, like every caffe::Error (src/c_api.cpp:206-223);
    the next forward pass on the same net and context succeeds with the usual results."""
    import ctypes
    wl = pkg("workloads")
    b = wl.conv_relu(1)
    weights = wl.init_params(b.params, seed=0)
    x = wl.conv_relu_input(1, seed=0)
    L = gpu_engine.lib
    L.mcb200_conv_set_wait_limit.restype = ctypes.c_longlong
    L.mcb200_conv_set_wait_limit.argtypes = [ctypes.c_longlong]
    net = capi.Net(gpu_engine, b.text(), None, from_buffer=True)
    net.set_params(weights)
    net.forward(**x)
    good = net.blob("conv").data.copy()
    previous = L.mcb200_conv_set_wait_limit(2000000)
    try:
        L.mcb200_conv_test_drop_weight_load()
        with pytest.raises(capi.CaffeError) as err:
            net.forward(**x)
        assert "gave up waiting" in str(err.value)
    finally:
        L.mcb200_conv_set_wait_limit(previous)
    net.forward(**x)
    assert np.array_equal(net.blob("conv").data.view(np.uint32), good.view(np.uint32))
    net.close()
