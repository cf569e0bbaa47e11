"""The drop-in boundary, pinned with the reference project's own callers (no GPU needed here).

Where a checkout of the reference project is present:
  * its command-line benchmark (tools/benchmark.cpp:7-35, C++ API), its C test program
    (tests/run_net.c:19-96, C API) and its C++ test program (tests/run_net.cpp, C++ API with
    threads, buffers and reshape) are compiled from where they lie against this repository's
    include/ and linked with the engine's libcaffe.so (`make -C oracle callers`);
  * its Python package (python/minicaffe, base.py:25-47 looks for libcaffe.so beside itself) is
    imported from a scratch copy with the engine's library beside it: it builds a net, lists
    blobs and parameters, reshapes, and reports the engine's errors through its own exception.
Without a device every forward pass must fail loudly; the GPU half of this lives in
test_reference_callers_gpu.py and runs the programs built here.
"""
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest

from conftest import ENGINE_LIB, REFERENCE_CHECKOUT, ROOT, pkg
from parity import write_model_files

CALLERS = os.path.join(ROOT, "oracle", "_ref", "callers")
HAVE_REFERENCE = os.path.isfile(os.path.join(REFERENCE_CHECKOUT, "tools", "benchmark.cpp"))

pytestmark = pytest.mark.skipif(not HAVE_REFERENCE, reason="reference checkout not present")


@pytest.fixture(scope="module")
def callers():
    run = subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "callers", "REF=" + REFERENCE_CHECKOUT],
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    paths = {name: os.path.join(CALLERS, name) for name in ("ref_benchmark", "ref_run_net_c", "ref_run_net_cpp")}
    for p in paths.values():
        assert os.path.isfile(p) and os.access(p, os.X_OK), p
    return paths


def test_reference_programs_compile_and_link_against_the_engine(callers):
    # every Caffe* function the C program calls resolves to the engine's library
    out = subprocess.run(["ldd", callers["ref_run_net_c"]], capture_output=True, text=True).stdout
    line = [l for l in out.splitlines() if "libcaffe.so" in l]
    assert line and os.path.realpath(line[0].split("=>")[1].split("(")[0].strip()) == os.path.realpath(ENGINE_LIB)


def test_reference_benchmark_tool_reports_the_missing_device(callers, tmp_path):
    """tools/benchmark.cpp with gpu_id -1: the net is built by the engine, and Forward stops with
    the engine's error (there is no host compute path to fall back to)."""
    wl = pkg("workloads")
    proto = tmp_path / "net.prototxt"
    proto.write_text(wl.conv_relu(1).text())
    run = subprocess.run([callers["ref_benchmark"], str(proto), "1", "-1"], capture_output=True, text=True,
                         cwd=str(tmp_path), timeout=120)
    assert run.returncode != 0
    assert "net prototxt" in run.stderr
    assert "no CPU compute path" in run.stderr or "no CUDA device is available" in run.stderr


def test_reference_python_package_drives_the_engine(tmp_path):
    pkg_dir = tmp_path / "minicaffe"
    shutil.copytree(os.path.join(REFERENCE_CHECKOUT, "python", "minicaffe"), str(pkg_dir))
    os.symlink(ENGINE_LIB, str(pkg_dir / "libcaffe.so"))
    wl = pkg("workloads")
    b = wl.conv_relu(2)
    weights = wl.init_params(b.params, seed=0)
    proto, model = write_model_files(b, weights, tmp_path / "model", "conv_relu")
    script = tmp_path / "drive.py"
    script.write_text(
        "import sys, numpy as np\n"
        "sys.path.insert(0, %r)\n"
        "import minicaffe as mc\n"
        "net = mc.Net(%r, %r)\n"
        "blobs = net.blobs\n"
        "assert list(blobs['data'].shape) == [2, 64, 56, 56], blobs['data'].shape\n"
        "assert list(blobs['conv'].shape) == [2, 64, 56, 56]\n"
        "params = net.params\n"
        "w = params['conv'][0][1].data\n"
        "assert tuple(w.shape) == (64, 64, 3, 3) and float(np.abs(w).sum()) > 0\n"
        "blobs['data'].reshape(1, 64, 56, 56)\n"
        "assert list(net.get_blob('data').shape) == [1, 64, 56, 56]\n"
        "net.mark_output('conv')\n"
        "try:\n"
        "    mc.Net('no-such.prototxt', 'no-such.caffemodel')\n"
        "    raise SystemExit('missing file accepted')\n"
        "except Exception as e:\n"
        "    assert 'no-such.prototxt' in str(e), str(e)\n"
        "if not mc.check_gpu_available():\n"
        "    try:\n"
        "        net.forward(data=np.zeros((1, 64, 56, 56), np.float32))\n"
        "        raise SystemExit('forward without a device did not fail')\n"
        "    except Exception as e:\n"
        "        assert 'no CPU compute path' in str(e) or 'no CUDA device' in str(e), str(e)\n"
        "print('ok')\n" % (str(tmp_path), proto, model))
    run = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and "ok" in run.stdout, run.stdout[-2000:] + run.stderr[-3000:]
