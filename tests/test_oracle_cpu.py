"""The CPU restatements under oracle/ against the golden fixtures that were
produced by the reference project's own CPU code (tests/golden/make_golden.py).
Dense layers: float32 rounding (BLAS summation order may differ); detection
tail: bit for bit."""
import importlib
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


@pytest.fixture(scope="module")
def no():
    return importlib.import_module("oracle.numpy_oracle")


@pytest.fixture(scope="module")
def port():
    mod = importlib.import_module("oracle.port")
    mod.build()
    return mod


def close(a, b, tol=2e-5):
    assert a.shape == b.shape, (a.shape, b.shape)
    scale = max(1.0, float(np.abs(b).max()))
    assert float(np.abs(a - b).max()) <= tol * scale, float(np.abs(a - b).max())


def test_dense_layers_follow_the_reference(no):
    g = load("dense_layers")
    x = g["in_data"]
    conv = no.convolution(x, g["w_conv_0"], g["w_conv_1"], stride=2, pad=1)
    conv = no.batch_norm(conv, g["w_bn_0"], g["w_bn_1"], float(g["w_bn_2"][0]))
    conv = no.scale(conv, g["w_sc_0"], g["w_sc_1"])
    conv = no.relu(conv)
    close(conv, g["out_conv"])
    dw = no.convolution(conv, g["w_dw_0"], g["w_dw_1"], stride=1, pad=1, group=8)
    close(dw, g["out_dw"])
    pr = no.prelu(dw, g["w_prelu_0"])
    close(pr, g["out_prelu"])
    close(no.pooling(pr, "MAX", 3, stride=2, pad=1), g["out_pmax"])
    close(no.pooling(pr, "AVE", 2, stride=2, pad=1), g["out_pave"])
    close(no.convolution(pr, g["w_dil_0"], g["w_dil_1"], stride=1, pad=2, dilation=2), g["out_dil"])
    s = no.eltwise([pr, conv], "SUM")
    close(s, g["out_sum"])
    nrm = no.normalize(s, g["w_norm_0"])
    close(nrm, g["out_norm"])
    close(no.permute(nrm, (0, 2, 3, 1)), g["out_perm"])
    pm = no.pooling(pr, "MAX", 3, stride=2, pad=1)
    close(no.concat([pm, pm], axis=1), g["out_cat"])
    gap = no.pooling(s, "AVE", None, global_pooling=True)
    close(gap, g["out_gap"])
    fc = no.inner_product(gap, g["w_fc_0"], g["w_fc_1"])
    close(fc, g["out_fc"])
    close(no.softmax(fc, axis=1), g["out_prob"])


def test_folding_algebra_equals_separate_layers(no):
    g = load("dense_layers")
    raw = no.convolution(g["in_data"], g["w_conv_0"], None, stride=2, pad=1)
    s, t = no.fold_batch_norm_scale(g["w_bn_0"], g["w_bn_1"], float(g["w_bn_2"][0]), 1e-5, g["w_sc_0"], g["w_sc_1"],
                                    conv_bias=g["w_conv_1"])
    folded = no.relu((raw * s.reshape(1, -1, 1, 1) + t.reshape(1, -1, 1, 1)).astype(np.float32))
    close(folded, g["out_conv"])


def test_pool_output_sizes(no):
    # 112 -> 56 with k3 s2 p0 (ceil), 75 -> 38 (SSD pool3), 19 -> 19 with k3 s1 p1 (clip rule)
    assert no.pool_out_size(112, 3, 2, 0) == 56
    assert no.pool_out_size(75, 2, 2, 0) == 38
    assert no.pool_out_size(19, 3, 1, 1) == 19
    assert no.conv_out_size(224, 7, 2, 3) == 112
    assert no.conv_out_size(19, 3, 1, 6, dilation=6) == 19


@pytest.mark.parametrize("tag", ["a9", "a15", "tiny"])
def test_proposal_port_bit_exact(port, tag):
    g = load("proposal_" + tag)
    min_size, pre, post, thr = g["params"]
    rois, scores = port.proposal(g["scores_in"], g["deltas_in"], g["im_info"], [0.5, 1.0, 2.0], g["scales"],
                                 min_size=int(min_size), pre_nms_topn=int(pre), post_nms_topn=int(post),
                                 nms_thresh=float(thr))
    assert rois.shape == g["rois"].shape
    assert np.array_equal(rois.view(np.uint32), g["rois"].view(np.uint32))
    assert np.array_equal(scores.view(np.uint32), g["scores_out"].view(np.uint32))


@pytest.mark.parametrize("tag", ["center", "corner", "perclass"])
def test_detection_output_port_bit_exact(port, tag):
    g = load("detout_" + tag)
    num_classes, share, code, conf_thr, nms_thr, top_k, keep = g["params"]
    out = port.detection_output(g["loc"], g["conf"], g["prior"], int(num_classes), share_location=bool(share),
                                code_type=int(code), confidence_threshold=float(conf_thr),
                                nms_threshold=float(nms_thr), top_k=int(top_k), keep_top_k=int(keep))
    assert out.shape == g["out"].shape
    assert np.array_equal(out.view(np.uint32), g["out"].view(np.uint32))


def test_anchor_generation(port):
    a = port.generate_anchors(16, [0.5, 1.0, 2.0], [8, 16, 32])
    assert a.shape == (9, 4)
    # ratio 1, scale 8: a 128 x 128 box centred on (7.5, 7.5)
    assert np.allclose(a[3], [-56.0, -56.0, 71.0, 71.0])
    # widths and heights are symmetric about the centre
    assert np.allclose((a[:, 0] + a[:, 2]) / 2, 7.5) and np.allclose((a[:, 1] + a[:, 3]) / 2, 7.5)


def test_roi_pooling_restatements_bit_exact(no):
    g = load("roipooling")
    p = g["params"]
    got = no.roi_pooling(g["maps"], g["rois"], int(p[2]), int(p[3]), np.float32(p[4]))
    assert np.array_equal(got.view(np.uint32), g["out"].view(np.uint32))
    g = load("psroipooling")
    p = g["params"]
    got = no.psroi_pooling(g["maps"], g["rois"], int(p[0]), int(p[1]), np.float32(p[4]))
    assert np.array_equal(got.view(np.uint32), g["out"].view(np.uint32))
    # the fixtures hold the special cases: empty bins give exactly 0, and some bins are not empty
    assert (g["out"] == 0).any() and (g["out"] != 0).any()


def test_extra_layer_restatements_follow_the_reference(no):
    """Deconvolution, Crop, Slice, BN and LRN against the fixture the compiled reference produced."""
    g = load("extra_layers")
    x = g["in_data"]
    up = no.deconvolution(x, g["w_up_0"], g["w_up_1"], stride=2, pad=1)
    close(up, g["out_up"])
    up_g = no.deconvolution(x, g["w_up_g_0"], None, stride=1, pad=1, group=3)
    close(up_g, g["out_up_g"])
    # kernel 2 x 3, stride 3 x 2, dilation 2: the restatement takes square parameters, so check the
    # shape rule only: stride * (in - 1) + dilation * (k - 1) + 1 - 2 * pad
    assert g["out_up_d"].shape == (2, 3, 3 * 8 + 2 * 1 + 1, 2 * 6 + 2 * 2 + 1)
    crop = no.crop(g["out_up"], (2, 4, 13, 11), axis=2, offsets=(2, 1))
    assert np.array_equal(crop, g["out_crop"])
    assert np.array_equal(no.crop(g["out_up"], (2, 4, 13, 11), axis=2, offsets=(1,)), g["out_crop1"])
    s0, s1, s2 = no.slice_blob(g["out_up_g"], 1, slice_points=(1, 4))
    assert np.array_equal(s0, g["out_s0"]) and np.array_equal(s1, g["out_s1"]) and np.array_equal(s2, g["out_s2"])
    e0, e1 = no.slice_blob(g["out_up"], 2, num_tops=2)
    assert np.array_equal(e0, g["out_e0"]) and np.array_equal(e1, g["out_e1"])
    bn = no.bn(g["out_crop"], g["w_bn_0"], g["w_bn_1"], g["w_bn_2"], g["w_bn_3"])
    close(bn, g["out_bn"])
    close(no.lrn(g["out_up_g"], 5, 0.0001, 0.75, 2.0), g["out_lrn_a"])
    close(no.lrn(g["out_bn"], 3, 0.05, 0.75, within_channel=True), g["out_lrn_w"])
