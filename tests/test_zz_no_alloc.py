"""mcb200_proposal_forward_static: the proposal pipeline with its scratch in a
fixed array inside the library, for callers that cannot allocate device memory
(their process has given all of it to another pool, or they cannot afford the
synchronisation an allocation implies).

Checked through the C ABI against mcb200_proposal_forward (caller-provided
workspace): identical rois, scores and counts, bit for bit, on two calls in a
row with different inputs -- the second call sees the first call's leftovers in
the shared scratch and must not be affected by them.  This file sorts last on
purpose, so a run that stops at the first failure has already run everything
else; it also passes on its own in a fresh process."""
import ctypes

import numpy as np
import pytest

from conftest import pkg

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


class ProposalParams(ctypes.Structure):
    _fields_ = [("num_anchors", ctypes.c_int), ("height", ctypes.c_int), ("width", ctypes.c_int),
                ("feat_stride", ctypes.c_int), ("min_size", ctypes.c_int), ("pre_nms_topn", ctypes.c_int),
                ("post_nms_topn", ctypes.c_int), ("nms_thresh", ctypes.c_float)]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _anchors(scales):
    port = __import__("importlib").import_module("oracle.port")
    return port.generate_anchors(16, [0.5, 1.0, 2.0], scales)


def _run(lib, static, params, inputs, anchors):
    post = params.post_nms_topn
    scores = torch.from_numpy(inputs["rpn_cls_prob"]).cuda()
    deltas = torch.from_numpy(inputs["rpn_bbox_pred"]).cuda()
    info = torch.from_numpy(inputs["im_info"]).cuda()
    anc = torch.from_numpy(anchors).cuda()
    rois = torch.full((post, 5), -7.0, device="cuda")
    roi_scores = torch.full((post,), -7.0, device="cuda")
    counts = torch.zeros(1, dtype=torch.int32, device="cuda")
    if static:
        rc = lib.mcb200_proposal_forward_static(ctypes.byref(params), 1, _ptr(scores), _ptr(deltas), _ptr(info),
                                                _ptr(anc), _ptr(rois), _ptr(roi_scores), _ptr(counts), None)
    else:
        lib.mcb200_proposal_workspace_bytes.restype = ctypes.c_size_t
        need = lib.mcb200_proposal_workspace_bytes(ctypes.byref(params), 1)
        assert need > 0
        ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
        base = (ws.data_ptr() + 255) & ~255
        rc = lib.mcb200_proposal_forward(ctypes.byref(params), 1, _ptr(scores), _ptr(deltas), _ptr(info), _ptr(anc),
                                         ctypes.c_void_p(base), _ptr(rois), _ptr(roi_scores), _ptr(counts), None)
    assert rc == 0, rc
    torch.cuda.synchronize()
    n = int(counts.item())
    return n, rois[:n].cpu().numpy(), roi_scores[:n].cpu().numpy()


def test_static_scratch_warmup_is_repeatable(kernels):
    """The warm-up entry point does the one-time work of the first call (device code loaded, array
    address looked up, kernels opted into their shared-memory size) and launches nothing; hosts call
    it before they take the device memory for their own pool.  Calling it again changes nothing."""
    kernels.mcb200_launch_count.restype = ctypes.c_longlong
    before = kernels.mcb200_launch_count()
    assert kernels.mcb200_proposal_static_warmup() == 0
    assert kernels.mcb200_proposal_static_warmup() == 0
    assert kernels.mcb200_launch_count() == before


def test_static_scratch_variant_matches_workspace_variant(kernels):
    wl = pkg("workloads")
    calls = [
        # a large case first, then a small one that reuses a fraction of the dirty scratch
        (dict(num_anchors=15, height=63, width=38, pre=6000, post=300, thr=0.7), wl.PROPOSAL_SCALES_15, 3),
        (dict(num_anchors=9, height=20, width=30, pre=500, post=50, thr=0.5), wl.PROPOSAL_SCALES_9, 4),
    ]
    for shape, scales, seed in calls:
        params = ProposalParams(shape["num_anchors"], shape["height"], shape["width"], 16, 16, shape["pre"],
                                shape["post"], shape["thr"])
        inputs, _ = wl.proposal_input(num_anchors=shape["num_anchors"], height=shape["height"], width=shape["width"],
                                      seed=seed, im_h=16.0 * shape["height"], im_w=16.0 * shape["width"])
        anchors = _anchors(scales)
        n_ws, rois_ws, scores_ws = _run(kernels, False, params, inputs, anchors)
        n_st, rois_st, scores_st = _run(kernels, True, params, inputs, anchors)
        assert n_ws > 0 and n_st == n_ws
        assert np.array_equal(rois_st.view(np.uint32), rois_ws.view(np.uint32))
        assert np.array_equal(scores_st.view(np.uint32), scores_ws.view(np.uint32))


def test_static_scratch_variant_rejects_oversized_requests(kernels):
    # 64 images of the stock configuration need far more than the built-in 8 MiB
    params = ProposalParams(15, 63, 38, 16, 16, 6000, 300, 0.7)
    dummy = torch.zeros(16, device="cuda")
    rc = kernels.mcb200_proposal_forward_static(ctypes.byref(params), 64, _ptr(dummy), _ptr(dummy), _ptr(dummy),
                                                _ptr(dummy), _ptr(dummy), _ptr(dummy), _ptr(dummy), None)
    assert rc == -20
