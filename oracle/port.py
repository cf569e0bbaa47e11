"""ctypes wrapper over the C restatement of the detection tail (detection_oracle.c).

TEST INFRASTRUCTURE ONLY -- see the header of detection_oracle.c.  build() compiles
the C file with gcc into oracle/liboracle_port.so (no -march, -ffp-contract=off).
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "detection_oracle.c")
LIBRARY = os.path.join(HERE, "liboracle_port.so")
_f = ctypes.POINTER(ctypes.c_float)


def build():
    if os.path.isfile(LIBRARY) and os.path.getmtime(LIBRARY) >= os.path.getmtime(SOURCE):
        return LIBRARY
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    subprocess.check_call([cc, "-O2", "-ffp-contract=off", "-shared", "-fPIC", "-o", LIBRARY, SOURCE, "-lm"])
    return LIBRARY


def _lib():
    lib = ctypes.CDLL(build())
    lib.oracle_proposal.restype = ctypes.c_int
    lib.oracle_detection_output.restype = ctypes.c_int
    return lib


def _p(a):
    return a.ctypes.data_as(_f)


def generate_anchors(base_size, ratios, scales):
    ratios = np.ascontiguousarray(ratios, dtype=np.float32)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    out = np.empty((len(ratios) * len(scales), 4), dtype=np.float32)
    _lib().oracle_generate_anchors(ctypes.c_int(base_size), _p(ratios), ctypes.c_int(len(ratios)), _p(scales),
                                   ctypes.c_int(len(scales)), _p(out))
    return out


def proposal(scores, deltas, im_info, ratios, scales, feat_stride=16, base_size=16, min_size=16, pre_nms_topn=6000,
             post_nms_topn=300, nms_thresh=0.7):
    """One image: scores [1, 2A, H, W], deltas [1, 4A, H, W], im_info [1, 3] -> (rois [R, 5], scores [R])."""
    anchors = generate_anchors(base_size, ratios, scales)
    a = anchors.shape[0]
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    deltas = np.ascontiguousarray(deltas, dtype=np.float32)
    im_info = np.ascontiguousarray(im_info, dtype=np.float32)
    h, w = scores.shape[2], scores.shape[3]
    rois = np.zeros((post_nms_topn, 5), dtype=np.float32)
    roi_scores = np.zeros((post_nms_topn,), dtype=np.float32)
    n = _lib().oracle_proposal(_p(scores), _p(deltas), _p(im_info), _p(anchors), ctypes.c_int(a), ctypes.c_int(h),
                               ctypes.c_int(w), ctypes.c_int(feat_stride), ctypes.c_int(min_size),
                               ctypes.c_int(pre_nms_topn), ctypes.c_int(post_nms_topn), ctypes.c_float(nms_thresh),
                               _p(rois), _p(roi_scores))
    return rois[:n].copy(), roi_scores[:n].copy()


def detection_output(loc, conf, prior, num_classes, share_location=True, background_label_id=0, code_type=2,
                     variance_encoded_in_target=False, confidence_threshold=-3.4028234663852886e38,
                     nms_threshold=0.3, eta=1.0, top_k=-1, keep_top_k=-1):
    loc = np.ascontiguousarray(loc, dtype=np.float32)
    conf = np.ascontiguousarray(conf, dtype=np.float32)
    prior = np.ascontiguousarray(prior, dtype=np.float32)
    batch = loc.shape[0]
    num_priors = prior.shape[-1] // 4
    out = np.zeros((batch * num_priors * num_classes + batch, 7), dtype=np.float32)
    rows = _lib().oracle_detection_output(
        _p(loc), _p(conf), _p(prior), ctypes.c_int(batch), ctypes.c_int(num_priors), ctypes.c_int(num_classes),
        ctypes.c_int(1 if share_location else 0), ctypes.c_int(background_label_id), ctypes.c_int(code_type),
        ctypes.c_int(1 if variance_encoded_in_target else 0), ctypes.c_float(confidence_threshold),
        ctypes.c_float(nms_threshold), ctypes.c_float(eta), ctypes.c_int(top_k), ctypes.c_int(keep_top_k), _p(out))
    if rows == 0:
        out = np.full((batch, 7), -1.0, dtype=np.float32)
        out[:, 0] = np.arange(batch)
        return out
    return out[:rows].copy()
