"""The benchmark configurations against the reference's CPU code at the sizes the configurations
state, where the other test files stop short of them:

  * DetectionOutput at the SSD300 size (8732 priors x 21 classes, confidence 0.01, NMS 0.45, top_k
    400, keep_top_k 200), bit for bit.  A TF32-level change of a score can flip an NMS decision, so
    the layer is isolated: the *reference's* own mbox_loc / mbox_conf_flatten / mbox_priorbox of an
    SSD300 pass are fed to a DetectionOutput-only net on both libraries, and the rows must be
    identical (detection_output_layer.cpp:74-226, bbox_util.cpp:681-716).
  * ResNet-50 at batch 1, and at batch 64 / 256 with the first 16 images being exactly the batch the
    oracle is run on: those 16 rows are compared with the oracle directly, all others through
    bit-exact batch invariance.
  * 16 more seeds of the Proposal stress case for both anchor counts, bit for bit.
"""
import numpy as np
import pytest

from conftest import pkg
from parity import assert_close, run_net

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_engine(engine):
    engine.set_mode(True, 0)
    return engine


SSD_HEAD = dict(num_priors=8732, num_classes=21, conf_thr=0.01, nms_thr=0.45, top_k=400, keep_top_k=200)


def _oracle_ssd_heads(capi, reflib, wl, seeds):
    """mbox_loc, mbox_conf_flatten (one row per seed) and mbox_priorbox of SSD300 passes on the oracle."""
    b = wl.ssd300_vgg16(1, with_detection_output=False)
    weights = wl.init_params(b.params, seed=0)
    names = ["mbox_loc", "mbox_conf_flatten", "mbox_priorbox"]
    rows = [run_net(capi, reflib, b, weights, wl.ssd_input(1, seed=s), names, marks=names) for s in seeds]
    return {"loc": np.concatenate([r["mbox_loc"] for r in rows], axis=0),
            "conf": np.concatenate([r["mbox_conf_flatten"] for r in rows], axis=0),
            "prior": rows[0]["mbox_priorbox"]}


@pytest.mark.parametrize("seeds", [(0,), (1, 2)])
def test_detection_output_at_ssd300_size_bit_exact(capi, gpu_engine, reflib, seeds):
    wl = pkg("workloads")
    feed = _oracle_ssd_heads(capi, reflib, wl, seeds)
    assert feed["loc"].shape == (len(seeds), 8732 * 4) and feed["conf"].shape == (len(seeds), 8732 * 21)
    head = wl.detection_head(batch=len(seeds), **SSD_HEAD)
    got = run_net(capi, gpu_engine, head, {}, feed, ["detection_out"])["detection_out"]
    want = run_net(capi, reflib, head, {}, feed, ["detection_out"])["detection_out"]
    assert got.shape == want.shape, (got.shape, want.shape)
    # random-init heads give near-uniform class scores: nearly every (prior, class) passes 0.01, so the
    # top_k = 400 cut and the keep_top_k = 200 cut both act
    assert want.shape[0] == 200 * len(seeds)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_detection_output_at_ssd300_size_trained_like_scores(capi, gpu_engine, reflib):
    """Same size with peaked class scores and spread-out priors (what a trained detector gives: few
    candidates per class, NMS decides): four images, bit for bit."""
    wl = pkg("workloads")
    head = wl.detection_head(batch=4, **SSD_HEAD)
    feed = wl.detection_head_input(4, 8732, 21, seed=77, peaked=True)
    got = run_net(capi, gpu_engine, head, {}, feed, ["detection_out"])["detection_out"]
    want = run_net(capi, reflib, head, {}, feed, ["detection_out"])["detection_out"]
    assert got.shape == want.shape and got.shape[0] > 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_resnet50_batch1(capi, gpu_engine, reflib):
    wl = pkg("workloads")
    b = wl.resnet50(1)
    weights = wl.init_params(b.params, seed=0)
    x = wl.image_input(1, seed=5)
    outs = ["fc1000", "prob"]
    marks = ["res2c", "res5c"]
    got = run_net(capi, gpu_engine, b, weights, x, outs + marks, marks=marks)
    want = run_net(capi, reflib, b, weights, x, outs + marks, marks=marks)
    for name in marks + outs:
        assert_close(got[name], want[name], "resnet50 b=1 " + name)


def _resnet_input(wl, batch):
    """The first 16 images are the batch the oracle runs; the rest is another seeded draw."""
    head = wl.image_input(16, seed=1)["data"]
    if batch == 16:
        return head
    return np.concatenate([head, wl.image_input(batch - 16, seed=2)["data"]], axis=0)


@pytest.fixture(scope="module")
def resnet_oracle_rows(capi):
    """fc1000 of the oracle for the 16 shared images (computed once for the module)."""
    import os
    from conftest import REF_LIB
    if not os.path.isfile(REF_LIB):
        pytest.fail("oracle/_ref/libcaffe_ref.so is not built")
    wl = pkg("workloads")
    ref = capi.CaffeLibrary(REF_LIB)
    b = wl.resnet50(16)
    weights = wl.init_params(b.params, seed=0)
    return run_net(capi, ref, b, weights, {"data": _resnet_input(wl, 16)}, ["fc1000"])["fc1000"]


@pytest.mark.parametrize("batch", [16, 64, 256])
def test_resnet50_stated_batches_against_the_oracle(capi, gpu_engine, resnet_oracle_rows, batch):
    wl = pkg("workloads")
    weights = wl.init_params(wl.resnet50(16).params, seed=0)
    x = _resnet_input(wl, batch)
    net = capi.Net(gpu_engine, wl.resnet50(batch).text(), None, from_buffer=True)
    net.set_params(weights)
    net.forward(data=x)
    fc = net.blob("fc1000").data.copy()
    prob = net.blob("prob").data.copy()
    net.close()
    assert fc.shape == (batch, 1000) and np.isfinite(fc).all()
    assert np.abs(prob.sum(axis=1) - 1.0).max() < 1e-4
    # the 16 shared images against the reference's CPU result, at this batch size
    assert_close(fc[:16], resnet_oracle_rows, "resnet50 b=%d fc1000[:16]" % batch)
    if batch > 16:
        # every other group of 16 images: bit for bit what a batch of those 16 alone gives
        small = capi.Net(gpu_engine, wl.resnet50(16).text(), None, from_buffer=True)
        small.set_params(weights)
        for start in sorted({0, 16, batch - 16}):
            small.forward(data=x[start:start + 16])
            alone = small.blob("fc1000").data.copy()
            assert np.array_equal(fc[start:start + 16].view(np.uint32), alone.view(np.uint32)), start
        small.close()


@pytest.mark.parametrize("anchors", [15, 9])
@pytest.mark.parametrize("seed", list(range(3, 19)))
def test_proposal_stress_case_more_seeds(capi, gpu_engine, reflib, anchors, seed):
    wl = pkg("workloads")
    b = wl.proposal(num_anchors=anchors, with_scores=True)
    inputs, _ = wl.proposal_input(num_anchors=anchors, seed=seed)
    got = run_net(capi, gpu_engine, b, {}, inputs, ["rois", "scores"])
    want = run_net(capi, reflib, b, {}, inputs, ["rois", "scores"])
    assert got["rois"].shape == want["rois"].shape and got["rois"].shape[0] > 0
    assert np.array_equal(got["rois"].view(np.uint32), want["rois"].view(np.uint32))
    assert np.array_equal(got["scores"].view(np.uint32), want["scores"].view(np.uint32))


def test_proposal_batch_compaction_with_short_first_image(capi, gpu_engine, reflib):
    """Two images in one call where the first keeps fewer rois than post_nms_topn: the second image's
    rows move up inside the output buffer (source and destination ranges overlap).  Each image's
    rows must equal the reference's single-image result."""
    wl = pkg("workloads")
    post = 300
    # pre_nms_topn 1000 keeps the cut among the positive scores: the boxes the min-size filter zeroes
    # tie at score 0, and the order of tied scores is the sort algorithm's own in the reference
    single = wl.proposal(num_anchors=9, height=20, width=30, pre_nms=1000, post_nms=post, nms_thresh=0.7,
                         min_size=16, with_scores=True)
    text = single.text().replace("dim: 1 dim: 18", "dim: 2 dim: 18").replace(
        "dim: 1 dim: 36", "dim: 2 dim: 36").replace("dim: 1 dim: 3 }", "dim: 2 dim: 3 }")
    # image 0 is a 100 x 100 picture: its boxes are clipped to that corner of the map, most of them
    # suppress each other and it keeps a few dozen rois; image 1 keeps all 300
    sizes = [(100.0, 100.0), (320.0, 480.0)]
    feeds = [wl.proposal_input(num_anchors=9, height=20, width=30, seed=50 + i, im_h=sizes[i][0], im_w=sizes[i][1])[0]
             for i in range(2)]
    want = [run_net(capi, reflib, single, {}, f, ["rois", "scores"]) for f in feeds]
    assert 0 < want[0]["rois"].shape[0] < post and want[1]["rois"].shape[0] == post
    net = capi.Net(gpu_engine, text, None, from_buffer=True)
    net.forward(**{k: np.concatenate([f[k] for f in feeds], axis=0) for k in feeds[0]})
    rois, scores = net.blob("rois").data.copy(), net.blob("scores").data.copy()
    net.close()
    n0 = want[0]["rois"].shape[0]
    assert rois.shape[0] == n0 + post
    assert (rois[:n0, 0] == 0).all() and (rois[n0:, 0] == 1).all()
    for i, (lo, hi) in enumerate(((0, n0), (n0, n0 + post))):
        assert np.array_equal(rois[lo:hi, 1:].view(np.uint32), want[i]["rois"][:, 1:].view(np.uint32)), i
        assert np.array_equal(scores[lo:hi].reshape(-1).view(np.uint32),
                              want[i]["scores"].reshape(-1).view(np.uint32)), i
