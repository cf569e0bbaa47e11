"""The benchmark configurations at their full sizes, checked through properties that do not need the
CPU oracle to run at that size: every image of a large batch must come out exactly as it does in a
small batch (the small-batch results are the ones compared with the oracle in the other test files),
probability rows sum to one, detection rows are well formed.  Each output element is accumulated
over K in the same order whatever the batch size, tile width or CTA pairing, so "exactly" is bit for
bit for the dense tensors."""
import numpy as np
import pytest

from conftest import pkg
from parity import run_net

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_engine(engine):
    engine.set_mode(True, 0)
    return engine


def _forward(capi, engine, builder, weights, feed, outs):
    net = capi.Net(engine, builder.text(), None, from_buffer=True)
    net.set_params(weights)
    net.forward(**feed)
    res = {o: net.blob(o).data.copy() for o in outs}
    net.close()
    return res


@pytest.mark.parametrize("batch", [64, 256])
def test_resnet50_full_batches(capi, gpu_engine, batch):
    wl = pkg("workloads")
    small = 16
    weights = wl.init_params(wl.resnet50(small).params, seed=0)
    x = wl.image_input(batch, seed=0)["data"]
    big = _forward(capi, gpu_engine, wl.resnet50(batch), weights, {"data": x}, ["fc1000", "prob"])
    ref = _forward(capi, gpu_engine, wl.resnet50(small), weights, {"data": x[:small]}, ["fc1000", "prob"])
    assert big["prob"].shape == (batch, 1000)
    assert np.isfinite(big["fc1000"]).all()
    assert np.abs(big["prob"].sum(axis=1) - 1.0).max() < 1e-4
    assert np.array_equal(big["fc1000"][:small].view(np.uint32), ref["fc1000"].view(np.uint32))
    # the last images of the batch, alone in a batch of their own
    tail = _forward(capi, gpu_engine, wl.resnet50(small), weights, {"data": x[-small:]}, ["fc1000"])
    assert np.array_equal(big["fc1000"][-small:].view(np.uint32), tail["fc1000"].view(np.uint32))


def test_mobilenet_v1_batch64(capi, gpu_engine):
    wl = pkg("workloads")
    weights = wl.init_params(wl.mobilenet_v1(2).params, seed=0)
    x = np.random.default_rng(3000).standard_normal((64, 3, 224, 224)).astype(np.float32)
    out = wl.mobilenet_v1(64)
    last = "prob"
    big = _forward(capi, gpu_engine, out, weights, {"data": x}, [last])
    ref = _forward(capi, gpu_engine, wl.mobilenet_v1(2), weights, {"data": x[10:12]}, [last])
    assert big[last].shape[0] == 64 and np.isfinite(big[last]).all()
    assert np.abs(big[last].reshape(64, -1).sum(axis=1) - 1.0).max() < 1e-4
    assert np.array_equal(big[last][10:12].view(np.uint32), ref[last].view(np.uint32))


def test_ssd300_batch32(capi, gpu_engine):
    wl = pkg("workloads")
    weights = wl.init_params(wl.ssd300_vgg16(2).params, seed=0)
    x = wl.ssd_input(32, seed=0)["data"]
    outs = ["mbox_loc", "mbox_conf_flatten", "detection_out"]
    net = capi.Net(gpu_engine, wl.ssd300_vgg16(32).text(), None, from_buffer=True)
    for m in outs[:2]:
        net.mark_output(m)
    net.set_params(weights)
    net.forward(data=x)
    big = {o: net.blob(o).data.copy() for o in outs}
    net.close()
    net = capi.Net(gpu_engine, wl.ssd300_vgg16(2).text(), None, from_buffer=True)
    for m in outs[:2]:
        net.mark_output(m)
    net.set_params(weights)
    net.forward(data=x[30:32])
    ref = {o: net.blob(o).data.copy() for o in outs}
    net.close()
    assert big["mbox_loc"].shape == (32, 34928) and big["mbox_conf_flatten"].shape == (32, 183372)
    assert np.array_equal(big["mbox_loc"][30:32].view(np.uint32), ref["mbox_loc"].view(np.uint32))
    assert np.array_equal(big["mbox_conf_flatten"][30:32].view(np.uint32), ref["mbox_conf_flatten"].view(np.uint32))
    det = big["detection_out"]
    assert det.shape[1] == 7 and 0 < det.shape[0] <= 32 * 200
    ids = det[:, 0].astype(int)
    assert (np.diff(ids) >= 0).all() and ids.min() >= 0 and ids.max() <= 31      # grouped by image, in order
    assert ((det[:, 1] >= 1) & (det[:, 1] <= 20)).all()                          # background never reported
    assert (det[:, 2] > 0.01).all()
    assert np.bincount(ids, minlength=32).max() <= 200                           # keep_top_k per image
    # identical inputs give identical detections: rows of images 30, 31 against the batch of two
    mine = det[ids >= 30].copy()
    mine[:, 0] -= 30
    assert np.array_equal(mine.view(np.uint32), ref["detection_out"].view(np.uint32))


def test_proposal_32_images_per_call(capi, gpu_engine):
    """The stress configuration as one replica runs it (256 images over 8 GPUs = 32 per call): every
    image's rois equal those of a call with that image alone (which the detection tests compare with
    the reference bit for bit)."""
    wl = pkg("workloads")
    images = 32
    single = wl.proposal(num_anchors=15, with_scores=True)
    text = single.text().replace("dim: 1 dim: 30", "dim: %d dim: 30" % images).replace(
        "dim: 1 dim: 60", "dim: %d dim: 60" % images).replace("dim: 1 dim: 3 }", "dim: %d dim: 3 }" % images)
    feeds = [wl.proposal_input(num_anchors=15, seed=100 + i)[0] for i in range(images)]
    feed = {k: np.concatenate([f[k] for f in feeds], axis=0) for k in feeds[0]}
    net = capi.Net(gpu_engine, text, None, from_buffer=True)
    net.forward(**feed)
    rois, scores = net.blob("rois").data.copy(), net.blob("scores").data.copy()
    net.close()
    assert rois.shape[1] == 5 and rois.shape[0] == scores.shape[0]
    one = capi.Net(gpu_engine, single.text(), None, from_buffer=True)
    offset = 0
    for i in (0, 7, 31):
        start = int(np.searchsorted(rois[:, 0], i, side="left"))
        stop = int(np.searchsorted(rois[:, 0], i, side="right"))
        one.forward(**feeds[i])
        r1, s1 = one.blob("rois").data.copy(), one.blob("scores").data.copy()
        assert stop - start == r1.shape[0] > 0
        assert np.array_equal(rois[start:stop, 1:].view(np.uint32), r1[:, 1:].view(np.uint32))
        assert np.array_equal(scores[start:stop].view(np.uint32), s1.view(np.uint32))
    one.close()
