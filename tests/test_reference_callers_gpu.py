"""The reference project's own programs, compiled against this repository's headers and linked with
the engine's libcaffe.so (oracle/Makefile, target `callers`; built where the reference checkout is,
shipped as binaries), run on the GPU:

  * tools/benchmark.cpp (C++ API: Net(file), Forward, Profiler) on the single Convolution + ReLU
    configuration at batch 32;
  * tests/run_net.c (C API: create from files and from buffers, blob accessors, reshape, data
    pointer, forward, list blobs, error string) on generated model files;
  * tests/run_net.cpp (C++ API: ReadBinaryNetParameterFromFile, CopyTrainedLayersFrom,
    blob_by_name, three threads with a net each, nets from buffers, MemPoolGetState, and its
    reshape test, which demands equal class scores at batch 1, 2, 1 to within 1e-6).
The programs look for model/nin.*, model/googlenet.*, model/resnet.* in their working directory;
the tests write generated networks of the shapes the programs assert on under those names.
"""
import json
import os
import subprocess

import pytest

from conftest import ROOT, pkg
from parity import write_model_files

pytestmark = pytest.mark.gpu

CALLERS = os.path.join(ROOT, "oracle", "_ref", "callers")


def _program(name):
    path = os.path.join(CALLERS, name)
    if not os.path.isfile(path):
        pytest.fail("%s is not built (`make -C oracle callers` where the reference checkout is)" % path)
    return path


def _small_classifier(wl, name, width):
    """[1, 3, 224, 224] -> `prob` [1, 1000], a few layers deep."""
    b = wl.NetBuilder(name)
    b.input([("data", (1, 3, 224, 224))])
    b.conv("conv1", "data", "conv1", 3, width, 7, stride=4, pad=3)
    b.relu("relu1", "conv1")
    b.pool("pool1", "conv1", "pool1", "MAX", k=3, stride=2)
    b.conv("conv2", "pool1", "conv2", width, 2 * width, 3, pad=1)
    b.relu("relu2", "conv2")
    b.pool("gap", "conv2", "gap", "AVE", global_pooling=True)
    b.inner_product("fc", "gap", "fc", 2 * width, 1000)
    b.softmax("prob", "fc", "prob")
    return b


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    wl = pkg("workloads")
    root = tmp_path_factory.mktemp("callers")
    for stem, builder in (("nin", _small_classifier(wl, "nin", 32)), ("googlenet", _small_classifier(wl, "googlenet", 48)),
                          ("resnet", wl.resnet50(1))):
        write_model_files(builder, wl.init_params(builder.params, seed=0), root / "model", stem)
    return root


def test_reference_benchmark_tool(tmp_path):
    wl = pkg("workloads")
    proto = tmp_path / "conv_relu.prototxt"
    proto.write_text(wl.conv_relu(32).text())
    run = subprocess.run([_program("ref_benchmark"), str(proto), "3", "0"], capture_output=True, text=True,
                         cwd=str(tmp_path), timeout=600)
    assert run.returncode == 0, run.stderr[-3000:]
    assert run.stderr.count("Forward costs") == 3
    events = json.load(open(tmp_path / "profile.json"))["traceEvents"]
    assert any(e["name"] == "conv" for e in events)


def test_reference_c_program(model_dir):
    run = subprocess.run([_program("ref_run_net_c")], capture_output=True, text=True, cwd=str(model_dir), timeout=600)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    assert "Forward NIN costs" in run.stdout
    assert "data: [1, 3, 224, 224]" in run.stdout and "prob: [1, 1000, 1, 1]" in run.stdout
    assert "no-such-prototxt" in run.stdout          # the error string of the failed create


def test_reference_cpp_program(model_dir):
    run = subprocess.run([_program("ref_run_net_cpp")], capture_output=True, text=True, cwd=str(model_dir), timeout=900)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    for needle in ("Forward NIN costs", "Forward GoogLeNet costs", "Forward ResNet costs", "test 3 threads",
                   "[GPU] Hold", "Test Reshape"):
        assert needle in run.stderr, needle
    assert os.path.isfile(model_dir / "profile.json")
