#!/usr/bin/env python3
"""Generates the golden fixtures in this directory by running the reference
project's own, unmodified CPU sources (oracle/_ref/libcaffe_ref.so, built from a
reference checkout by oracle/Makefile) on small seeded inputs.

    python tests/golden/make_golden.py

It can only run where the reference checkout was available at build time; the
resulting .npz files are committed so that every other machine can check the
CPU restatements under oracle/ (and, through them, the CUDA kernels) against
what the reference really computes.
"""
import importlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

capi = importlib.import_module("mini-caffe_b200.capi")
wl = importlib.import_module("mini-caffe_b200.workloads")
REF = capi.CaffeLibrary(os.path.join(ROOT, "oracle", "_ref", "libcaffe_ref.so"))


def run(builder, weights, inputs, outputs, marks=()):
    """One network through the reference, in a thread of its own (see tests/parity.py)."""
    from parity import run_net
    return run_net(capi, REF, builder, weights, inputs, outputs, marks=marks)


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    print("wrote", name, {k: v.shape for k, v in arrays.items()})


def dense_layers():
    rng = np.random.default_rng(100)
    b = wl.NetBuilder("dense")
    b.input([("data", (2, 6, 11, 9))])
    b.conv("conv", "data", "conv", 6, 8, 3, stride=2, pad=1)
    b.batch_norm("bn", "conv", 8)
    b.scale("sc", "conv", 8)
    b.relu("relu", "conv")
    b.conv("dw", "conv", "dw", 8, 8, 3, stride=1, pad=1, group=8)
    b.raw("prelu", "PReLU", ["dw"], ["prelu"])
    b.params.append(("prelu_0", (8,), "he", 8))
    b.pool("pmax", "prelu", "pmax", "MAX", k=3, stride=2, pad=1)
    b.pool("pave", "prelu", "pave", "AVE", k=2, stride=2, pad=1)
    b.conv("dil", "prelu", "dil", 8, 4, 3, stride=1, pad=2, dilation=2)
    b.eltwise_sum("sum", ["prelu", "conv"], "sum")
    b.raw("norm", "Normalize", ["sum"], ["norm"], "norm_param { across_spatial: false channel_shared: false }")
    b.params.append(("norm_0", (8,), "norm_scale", 0))
    b.raw("perm", "Permute", ["norm"], ["perm"], "permute_param { order: 0 order: 2 order: 3 order: 1 }")
    b.raw("cat", "Concat", ["pmax", "pmax"], ["cat"], "concat_param { axis: 1 }")
    b.pool("gap", "sum", "gap", "AVE", global_pooling=True)
    b.inner_product("fc", "gap", "fc", 8, 5)
    b.softmax("prob", "fc", "prob")
    weights = wl.init_params(b.params, seed=7, bn_identity=False)
    x = {"data": rng.standard_normal((2, 6, 11, 9)).astype(np.float32)}
    outs = ["conv", "dw", "prelu", "pmax", "pave", "dil", "sum", "norm", "perm", "cat", "gap", "fc", "prob"]
    marks = outs
    res = run(b, weights, x, outs, marks=marks)
    arrays = {"in_data": x["data"]}
    arrays.update({"w_" + k: v for k, v in weights.items()})
    arrays.update({"out_" + k: v for k, v in res.items()})
    save("dense_layers", **arrays)


def proposal_cases():
    for tag, anchors, h, w, pre, post, thr, min_size, seed in [
            ("a9", 9, 12, 10, 300, 40, 0.7, 16, 1), ("a15", 15, 9, 7, 200, 30, 0.5, 8, 2),
            ("tiny", 3, 2, 2, 6000, 300, 0.7, 16, 3)]:
        scales = {9: (8, 16, 32), 15: (2, 4, 8, 16, 32), 3: (8,)}[anchors]
        b = wl.NetBuilder("proposal")
        b.input([("rpn_cls_prob", (1, 2 * anchors, h, w)), ("rpn_bbox_pred", (1, 4 * anchors, h, w)),
                 ("im_info", (1, 3))])
        b.raw("proposal", "Proposal", ["rpn_cls_prob", "rpn_bbox_pred", "im_info"], ["rois", "scores"],
              "proposal_param { feat_stride: 16 base_size: 16 min_size: %d pre_nms_topn: %d post_nms_topn: %d "
              "nms_thresh: %g ratio: 0.5 ratio: 1 ratio: 2 %s }" % (min_size, pre, post, thr,
                                                                     " ".join("scale: %d" % s for s in scales)))
        inputs, _ = wl.proposal_input(num_anchors=anchors, height=h, width=w, seed=seed, im_h=16.0 * h,
                                      im_w=16.0 * w)
        res = run(b, {}, inputs, ["rois", "scores"])
        save("proposal_" + tag, scores_in=inputs["rpn_cls_prob"], deltas_in=inputs["rpn_bbox_pred"],
             im_info=inputs["im_info"], scales=np.array(scales, np.float32),
             params=np.array([min_size, pre, post, thr], np.float64), rois=res["rois"], scores_out=res["scores"])


def detection_cases():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_detection_gpu import detection_head_net, detection_inputs
    for tag, case in [
            ("center", dict(batch=2, num_priors=300, num_classes=5, conf_thr=0.01, nms_thr=0.45, top_k=60,
                            keep_top_k=40)),
            ("corner", dict(batch=1, num_priors=200, num_classes=4, conf_thr=0.05, nms_thr=0.45, top_k=50,
                            keep_top_k=-1, code_type="CORNER")),
            ("perclass", dict(batch=2, num_priors=150, num_classes=3, conf_thr=0.05, nms_thr=0.5, top_k=40,
                              keep_top_k=25, share_location=False))]:
        b = detection_head_net(wl, **case)
        inputs = detection_inputs(case["batch"], case["num_priors"], case["num_classes"], seed=31,
                                  share_location=case.get("share_location", True), peaked=True)
        res = run(b, {}, inputs, ["detection_out"])
        code = {"CORNER": 1, "CENTER_SIZE": 2, "CORNER_SIZE": 3}[case.get("code_type", "CENTER_SIZE")]
        save("detout_" + tag, loc=inputs["loc"], conf=inputs["conf"], prior=inputs["prior"],
             params=np.array([case["num_classes"], 1 if case.get("share_location", True) else 0, code,
                              case["conf_thr"], case["nms_thr"], case["top_k"], case["keep_top_k"]], np.float64),
             out=res["detection_out"])


def prior_box_case():
    b = wl.NetBuilder("priors")
    b.input([("feat", (1, 8, 5, 7)), ("data", (1, 3, 300, 300))])
    b.raw("pb", "PriorBox", ["feat", "data"], ["pb"],
          "prior_box_param { min_size: 60 max_size: 111 aspect_ratio: 2 aspect_ratio: 3 flip: true clip: true "
          "variance: 0.1 variance: 0.1 variance: 0.2 variance: 0.2 step: 16 offset: 0.5 }")
    x = {"feat": np.zeros((1, 8, 5, 7), np.float32), "data": np.zeros((1, 3, 300, 300), np.float32)}
    save("prior_box", out=run(b, {}, x, ["pb"])["pb"])


def roi_pooling_cases():
    for kind, kw in [("PSROIPooling", dict(batch=2, height=9, width=7, num_rois=48, output_dim=3, group_size=3)),
                     ("ROIPooling", dict(batch=2, height=9, width=7, num_rois=48, channels=5, pooled_h=3,
                                         pooled_w=2))]:
        b = wl.roi_pooling(kind, spatial_scale=1.0 / 16, **kw)
        channels = kw["output_dim"] * kw["group_size"] ** 2 if kind == "PSROIPooling" else kw["channels"]
        inputs = wl.roi_pooling_input(kw["batch"], channels, kw["height"], kw["width"], kw["num_rois"], seed=3)
        res = run(b, {}, inputs, ["pooled"])
        save(kind.lower(), maps=inputs["maps"], rois=inputs["rois"], out=res["pooled"],
             params=np.array([kw.get("output_dim", 0), kw.get("group_size", 0), kw.get("pooled_h", 0),
                              kw.get("pooled_w", 0), 1.0 / 16], np.float64))


def extra_layers_case():
    b = wl.extra_layers_net(2)
    weights = wl.init_params(b.params, seed=5, bn_identity=False)
    x = wl.extra_layers_input(2, seed=1)
    res = run(b, weights, x, list(wl.EXTRA_LAYER_OUTPUTS), marks=list(wl.EXTRA_LAYER_OUTPUTS))
    arrays = {"in_data": x["data"]}
    arrays.update({"w_" + k: v for k, v in weights.items()})
    arrays.update({"out_" + k: v for k, v in res.items()})
    save("extra_layers", **arrays)


if __name__ == "__main__":
    dense_layers()
    extra_layers_case()
    roi_pooling_cases()
    proposal_cases()
    detection_cases()
    prior_box_case()
