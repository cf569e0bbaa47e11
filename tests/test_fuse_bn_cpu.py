"""The on-disk BatchNorm folding tool (mini-caffe_b200/cli/fuse_bn.cc, the counterpart of
mini-caffe's tools/fuse_bn.py) and, through it, the library's prototxt / caffemodel writer."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, pkg
from test_host_cpu import encode_caffemodel

EXE = os.path.join(ROOT, "mini-caffe_b200", "lib", "fuse_bn")


def build_case(wl, tmp_path):
    b = wl.NetBuilder("foldme")
    b.input([("data", (2, 6, 12, 10))])
    b.conv_bn("c1", "data", "c1", 6, 8, 3, stride=1, pad=1, bn_prefix="bn_", scale_prefix="scale_")                    # folded (no bias before)
    b.conv("c2", "c1", "c2", 8, 8, 3, pad=1, bias=True)                         # folded (bias before)
    b.batch_norm("bn_c2", "c2", 8)
    b.scale("scale_c2", "c2", 8)
    b.relu("relu_c2", "c2")
    b.conv("dw", "c2", "dw", 8, 8, 3, pad=1, group=8, bias=False)              # grouped: left alone
    b.batch_norm("bn_dw", "dw", 8)
    b.scale("scale_dw", "dw", 8)
    b.conv("c3", "dw", "c3", 8, 4, 1, bias=False)                               # BatchNorm without Scale: left alone
    b.batch_norm("bn_c3", "c3", 4)
    b.eltwise_sum("sum", ["c1", "c2"], "sum")
    b.pool("gap", "sum", "gap", "AVE", global_pooling=True)
    weights = wl.init_params(b.params, seed=3, bn_identity=False)
    by_layer = {}
    for key in sorted(weights):
        layer, idx = key.rsplit("_", 1)
        by_layer.setdefault(layer, []).append((int(idx), weights[key]))
    layers = [(name, [a for _, a in sorted(blobs)]) for name, blobs in by_layer.items()]
    proto = tmp_path / "net.prototxt"
    model = tmp_path / "net.caffemodel"
    proto.write_text(b.text())
    model.write_bytes(encode_caffemodel(layers))
    return b, weights, proto, model


@pytest.fixture(scope="module")
def tool():
    if not os.path.isfile(EXE):
        pytest.skip("fuse_bn not built")
    return EXE


def test_folds_the_reference_tools_pattern(capi, engine, tool, tmp_path):
    wl = pkg("workloads")
    no = pkg_oracle()
    b, weights, proto, model = build_case(wl, tmp_path)
    run = subprocess.run([tool, "--net", str(proto), "--weight", str(model)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stderr
    assert "fuse (c1, bn_c1, scale_c1)" in run.stdout and "fuse (c2, bn_c2, scale_c2)" in run.stdout
    assert "fuse (dw" not in run.stdout and "fuse (c3" not in run.stdout
    out_proto, out_model = tmp_path / "net_nobn.prototxt", tmp_path / "net_nobn.caffemodel"
    assert out_proto.is_file() and out_model.is_file()
    text = out_proto.read_text()
    for gone in ("bn_c1", "scale_c1", "bn_c2", "scale_c2"):
        assert '"%s"' % gone not in text
    for kept in ("bn_dw", "scale_dw", "bn_c3", "relu_c2"):
        assert '"%s"' % kept in text
    # the folded files load through the library's own reader (no device needed to build the net)
    net = capi.Net(engine, str(out_proto), str(out_model))
    got = {k: v.data.copy() for k, v in net.params()}
    net.close()
    for conv, bias in (("c1", None), ("c2", weights["c2_1"])):
        s, t = no.fold_batch_norm_scale(weights["bn_%s_0" % conv], weights["bn_%s_1" % conv],
                                        float(weights["bn_%s_2" % conv][0]), 1e-5, weights["scale_%s_0" % conv],
                                        weights["scale_%s_1" % conv], conv_bias=bias)
        want_w = weights[conv + "_0"].astype(np.float64) * s.reshape(-1, 1, 1, 1)
        assert np.allclose(got[conv + "_0"], want_w, rtol=1e-6, atol=1e-7)
        assert np.allclose(got[conv + "_1"], t, rtol=1e-6, atol=1e-6)
    assert np.array_equal(got["dw_0"], weights["dw_0"])
    assert np.array_equal(got["bn_c3_0"], weights["bn_c3_0"])


def pkg_oracle():
    import importlib
    return importlib.import_module("oracle.numpy_oracle")


def test_folded_files_compute_the_same_function_on_the_reference(capi, reflib, tool, tmp_path):
    """Original and folded files through the reference's own CPU code: same outputs to fp32 rounding."""
    wl = pkg("workloads")
    b, weights, proto, model = build_case(wl, tmp_path)
    subprocess.run([tool, "--net", str(proto), "--weight", str(model)], check=True, capture_output=True, timeout=120)
    x = np.random.default_rng(8).standard_normal((2, 6, 12, 10)).astype(np.float32)
    outs = {}
    from parity import in_fresh_thread

    def run_files(p, m):
        net = capi.Net(reflib, str(p), str(m))
        net.forward(data=x)
        res = {name: net.blob(name).data.copy() for name in ("gap", "c3")}
        net.close()
        reflib.memory_pool_clear()
        return res

    for tag, p, m in (("orig", proto, model), ("fold", tmp_path / "net_nobn.prototxt", tmp_path / "net_nobn.caffemodel")):
        outs[tag] = in_fresh_thread(lambda: run_files(p, m))
    for name in ("gap", "c3"):
        scale = max(1.0, float(np.abs(outs["orig"][name]).max()))
        assert np.abs(outs["orig"][name] - outs["fold"][name]).max() <= 2e-5 * scale
