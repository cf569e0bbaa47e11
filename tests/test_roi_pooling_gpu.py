"""ROIPooling and PSROIPooling (the heads behind Proposal in Faster R-CNN / R-FCN) against the
reference project's CPU code, bit for bit: the bin geometry is integer work and each bin is
reduced in the reference's order."""
import numpy as np
import pytest

from conftest import pkg
from parity import run_net

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_engine(engine):
    engine.set_mode(True, 0)
    return engine


CASES = [
    # kind, builder arguments
    ("PSROIPooling", dict(batch=1, height=63, width=38, num_rois=300, output_dim=21, group_size=7)),   # R-FCN class scores
    ("PSROIPooling", dict(batch=1, height=63, width=38, num_rois=300, output_dim=8, group_size=7)),    # R-FCN box deltas
    ("PSROIPooling", dict(batch=3, height=20, width=31, num_rois=64, output_dim=2, group_size=3)),
    ("PSROIPooling", dict(batch=1, height=5, width=4, num_rois=1, output_dim=1, group_size=1)),
    ("ROIPooling", dict(batch=1, height=63, width=38, num_rois=300, channels=256, pooled_h=7, pooled_w=7)),
    ("ROIPooling", dict(batch=2, height=14, width=14, num_rois=40, channels=33, pooled_h=6, pooled_w=3)),
    ("ROIPooling", dict(batch=1, height=3, width=2, num_rois=5, channels=1, pooled_h=7, pooled_w=7)),    # bins smaller than a cell
]


@pytest.mark.parametrize("kind,kw", CASES, ids=["%s-%d" % (k, i) for i, (k, _) in enumerate(CASES)])
def test_roi_pooling_bit_exact(capi, gpu_engine, reflib, kind, kw):
    wl = pkg("workloads")
    b = wl.roi_pooling(kind, **kw)
    channels = kw["output_dim"] * kw["group_size"] ** 2 if kind == "PSROIPooling" else kw["channels"]
    inputs = wl.roi_pooling_input(kw["batch"], channels, kw["height"], kw["width"], kw["num_rois"], seed=17)
    got = run_net(capi, gpu_engine, b, {}, inputs, ["pooled"])["pooled"]
    want = run_net(capi, reflib, b, {}, inputs, ["pooled"])["pooled"]
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert (want != 0).any()


def test_golden_fixtures_on_gpu(capi, gpu_engine):
    """The committed fixtures (made by the reference itself) do not need the compiled reference."""
    import os
    wl = pkg("workloads")
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    g = np.load(os.path.join(golden, "psroipooling.npz"))
    b = wl.roi_pooling("PSROIPooling", batch=2, height=9, width=7, num_rois=48, output_dim=3, group_size=3)
    got = run_net(capi, gpu_engine, b, {}, {"maps": g["maps"], "rois": g["rois"]}, ["pooled"])["pooled"]
    assert np.array_equal(got.view(np.uint32), g["out"].view(np.uint32))
    g = np.load(os.path.join(golden, "roipooling.npz"))
    b = wl.roi_pooling("ROIPooling", batch=2, height=9, width=7, num_rois=48, channels=5, pooled_h=3, pooled_w=2)
    got = run_net(capi, gpu_engine, b, {}, {"maps": g["maps"], "rois": g["rois"]}, ["pooled"])["pooled"]
    assert np.array_equal(got.view(np.uint32), g["out"].view(np.uint32))


def test_proposal_feeds_psroi_pooling(capi, gpu_engine, reflib):
    """Proposal -> PSROIPooling -> global average -> Softmax: the tail of an R-FCN forward pass,
    with the rois staying on the device between the two layers."""
    wl = pkg("workloads")
    anchors, h, w, classes, group = 9, 24, 18, 4, 3
    b = wl.NetBuilder("rfcn_tail")
    b.input([("rpn_cls_prob", (1, 2 * anchors, h, w)), ("rpn_bbox_pred", (1, 4 * anchors, h, w)),
             ("im_info", (1, 3)), ("rfcn_cls", (1, classes * group * group, h, w))])
    b.raw("proposal", "Proposal", ["rpn_cls_prob", "rpn_bbox_pred", "im_info"], ["rois"],
          "proposal_param { feat_stride: 16 base_size: 16 min_size: 16 pre_nms_topn: 400 post_nms_topn: 50 "
          "nms_thresh: 0.7 ratio: 0.5 ratio: 1 ratio: 2 scale: 8 scale: 16 scale: 32 }")
    b.raw("psroi", "PSROIPooling", ["rfcn_cls", "rois"], ["psroi"],
          "psroi_pooling_param { spatial_scale: 0.0625 output_dim: %d group_size: %d }" % (classes, group))
    b.pool("ave", "psroi", "cls_score", "AVE", global_pooling=True)
    b.softmax("prob", "cls_score", "cls_prob")
    inputs, _ = wl.proposal_input(num_anchors=anchors, height=h, width=w, seed=4, im_h=16.0 * h, im_w=16.0 * w)
    rng = np.random.default_rng(77)
    inputs["rfcn_cls"] = rng.standard_normal((1, classes * group * group, h, w)).astype(np.float32)
    got = run_net(capi, gpu_engine, b, {}, inputs, ["rois", "psroi", "cls_prob"], marks=["rois", "psroi"])
    want = run_net(capi, reflib, b, {}, inputs, ["rois", "psroi", "cls_prob"], marks=["rois", "psroi"])
    assert got["rois"].shape == want["rois"].shape and got["rois"].shape[0] > 0
    assert np.array_equal(got["rois"].view(np.uint32), want["rois"].view(np.uint32))
    assert np.array_equal(got["psroi"].view(np.uint32), want["psroi"].view(np.uint32))
    assert np.abs(got["cls_prob"] - want["cls_prob"]).max() < 1e-6


def test_roi_with_bad_image_index_is_an_error(capi, gpu_engine):
    """The reference stops with a CHECK failure; the engine reports it through the same error path."""
    wl = pkg("workloads")
    b = wl.roi_pooling("ROIPooling", batch=1, height=6, width=6, num_rois=2, channels=4, pooled_h=2, pooled_w=2)
    inputs = wl.roi_pooling_input(1, 4, 6, 6, 2, seed=1)
    inputs["rois"][1, 0] = 3.0
    with pytest.raises(RuntimeError):
        run_net(capi, gpu_engine, b, {}, inputs, ["pooled"])
    # the context stays usable
    inputs["rois"][1, 0] = 0.0
    out = run_net(capi, gpu_engine, b, {}, inputs, ["pooled"])["pooled"]
    assert np.isfinite(out).all()
