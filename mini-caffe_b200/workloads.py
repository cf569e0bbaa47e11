"""Seeded synthetic workloads: the benchmark / parity configurations as generated
prototxt text plus random-init weights and inputs.

No dataset, published prototxt or pretrained caffemodel is used anywhere: every
network here is emitted layer by layer by the small builder below, in the layer
layout Caffe model zoos use (Convolution + BatchNorm + Scale + ReLU, Eltwise
residual sums, ...), and all tensors come from numpy's default_rng with a fixed
seed.  The same (prototxt, weights, inputs) triple is fed to the engine and to
the CPU oracle.

Configurations (shapes and distributions as the benchmark definition states):
  conv_relu      one Convolution(64, 3x3, pad 1) + ReLU over [N, 64, 56, 56]
  resnet50       ResNet-50, bottleneck blocks [3, 4, 6, 3], 224 x 224 input
  mobilenet_v1   MobileNet-v1 1.0 / 224 with depthwise 3x3 + pointwise 1x1
  ssd300_vgg16   SSD300 on VGG16: L2Norm, six multibox heads, PriorBox,
                 DetectionOutput (21 classes, 8732 priors)
  proposal       RPN ProposalLayer over a 63 x 38 score map
"""
import numpy as np


class NetBuilder(object):
    """Accumulates prototxt text and remembers how to initialise each parameter."""

    def __init__(self, name):
        self.lines = ['name: "%s"' % name]
        # (param display name, shape, init kind, fan_in)
        self.params = []

    def text(self):
        return "\n".join(self.lines) + "\n"

    def _layer(self, name, ltype, bottoms, tops, body=""):
        parts = ['layer { name: "%s" type: "%s"' % (name, ltype)]
        parts += ['bottom: "%s"' % b for b in bottoms]
        parts += ['top: "%s"' % t for t in tops]
        if body:
            parts.append(body)
        parts.append("}")
        self.lines.append(" ".join(parts))

    def input(self, tops_shapes):
        shapes = " ".join("shape { %s }" % " ".join("dim: %d" % d for d in s) for _, s in tops_shapes)
        self._layer("input", "Input", [], [t for t, _ in tops_shapes], "input_param { %s }" % shapes)

    def conv(self, name, bottom, top, cin, cout, k, stride=1, pad=0, dilation=1, group=1, bias=True,
             weight_init="he", bias_init="zero"):
        body = "convolution_param { num_output: %d kernel_size: %d stride: %d pad: %d" % (cout, k, stride, pad)
        if dilation != 1:
            body += " dilation: %d" % dilation
        if group != 1:
            body += " group: %d" % group
        if not bias:
            body += " bias_term: false"
        body += " }"
        self._layer(name, "Convolution", [bottom], [top], body)
        fan_in = (cin // group) * k * k
        self.params.append((name + "_0", (cout, cin // group, k, k), weight_init, fan_in))
        if bias:
            self.params.append((name + "_1", (cout,), bias_init, fan_in))

    def batch_norm(self, name, blob, channels):
        self._layer(name, "BatchNorm", [blob], [blob], "batch_norm_param { use_global_stats: true }")
        self.params.append((name + "_0", (channels,), "bn_mean", 0))
        self.params.append((name + "_1", (channels,), "bn_var", 0))
        self.params.append((name + "_2", (1,), "one", 0))

    def scale(self, name, blob, channels):
        self._layer(name, "Scale", [blob], [blob], "scale_param { bias_term: true }")
        self.params.append((name + "_0", (channels,), "gamma", 0))
        self.params.append((name + "_1", (channels,), "beta", 0))

    def relu(self, name, blob):
        self._layer(name, "ReLU", [blob], [blob])

    def pool(self, name, bottom, top, method, k=None, stride=1, pad=0, global_pooling=False):
        if global_pooling:
            body = "pooling_param { pool: %s global_pooling: true }" % method
        else:
            body = "pooling_param { pool: %s kernel_size: %d stride: %d pad: %d }" % (method, k, stride, pad)
        self._layer(name, "Pooling", [bottom], [top], body)

    def eltwise_sum(self, name, bottoms, top):
        self._layer(name, "Eltwise", bottoms, [top], "eltwise_param { operation: SUM }")

    def inner_product(self, name, bottom, top, k, n, weight_init="he"):
        self._layer(name, "InnerProduct", [bottom], [top], "inner_product_param { num_output: %d }" % n)
        self.params.append((name + "_0", (n, k), weight_init, k))
        self.params.append((name + "_1", (n,), "zero", k))

    def softmax(self, name, bottom, top, axis=1):
        self._layer(name, "Softmax", [bottom], [top], "softmax_param { axis: %d }" % axis)

    def raw(self, name, ltype, bottoms, tops, body=""):
        self._layer(name, ltype, bottoms, tops, body)

    # -- conv + BatchNorm + Scale (+ ReLU), the unit ResNet / MobileNet repeat --
    def conv_bn(self, name, bottom, top, cin, cout, k, stride=1, pad=0, group=1, relu=True, bn_prefix="bn",
                scale_prefix="scale"):
        self.conv(name, bottom, top, cin, cout, k, stride=stride, pad=pad, group=group, bias=False)
        self.batch_norm(bn_prefix + name, top, cout)
        self.scale(scale_prefix + name, top, cout)
        if relu:
            self.relu(name + "_relu", top)


def init_params(params, seed, bn_identity=True):
    """{display name: ndarray} for a NetBuilder.params list.

    he      N(0, 2 / fan_in)           (weights)
    small   N(0, 0.01^2)               uniform   U(-0.1, 0.1)
    zero / one / gamma (=1) / beta (=0) / bn_mean (=0) / bn_var (=1)
    With bn_identity=False the BatchNorm statistics and Scale parameters are
    drawn at random instead (exercises the folding algebra).
    """
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape, kind, fan_in in params:
        if kind == "he":
            v = rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)
        elif kind == "small":
            v = rng.standard_normal(shape) * 0.01
        elif kind == "head":
            v = rng.standard_normal(shape) * np.sqrt(1.0 / fan_in)
        elif kind == "uniform":
            v = rng.uniform(-0.1, 0.1, shape)
        elif kind in ("zero", "beta", "bn_mean"):
            v = np.zeros(shape) if (bn_identity or kind == "zero") else rng.standard_normal(shape) * 0.1
        elif kind in ("one", ):
            v = np.ones(shape)
        elif kind in ("gamma", "bn_var"):
            v = np.ones(shape) if bn_identity else rng.uniform(0.5, 1.5, shape)
        elif kind == "norm_scale":
            v = np.full(shape, 20.0)
        else:
            raise ValueError(kind)
        out[name] = v.astype(np.float32)
    return out


# --------------------------------------------------------------------------- config 1

def conv_relu(batch):
    b = NetBuilder("conv_relu")
    b.input([("data", (batch, 64, 56, 56))])
    b.conv("conv", "data", "conv", 64, 64, 3, stride=1, pad=1, weight_init="small", bias_init="uniform")
    b.relu("relu", "conv")
    return b


def conv_relu_input(batch, seed=0):
    return {"data": np.random.default_rng(seed + 1000).standard_normal((batch, 64, 56, 56)).astype(np.float32)}


# --------------------------------------------------------------------------- config 2

def resnet50(batch, num_classes=1000):
    b = NetBuilder("resnet50")
    b.input([("data", (batch, 3, 224, 224))])
    b.conv("conv1", "data", "conv1", 3, 64, 7, stride=2, pad=3, bias=False)
    b.batch_norm("bn_conv1", "conv1", 64)
    b.scale("scale_conv1", "conv1", 64)
    b.relu("conv1_relu", "conv1")
    b.pool("pool1", "conv1", "pool1", "MAX", k=3, stride=2)
    prev, cin = "pool1", 64
    stages = [(2, 3, 64), (3, 4, 128), (4, 6, 256), (5, 3, 512)]
    for stage, blocks, width in stages:
        for i in range(blocks):
            tag = "%d%s" % (stage, "abcdefgh"[i])
            stride = 2 if (i == 0 and stage > 2) else 1
            cout = width * 4
            if i == 0:
                shortcut = "res%s_branch1" % tag
                b.conv_bn(shortcut, prev, shortcut, cin, cout, 1, stride=stride, relu=False, bn_prefix="bn_",
                          scale_prefix="scale_")
            else:
                shortcut = prev
            x = "res%s_branch2a" % tag
            b.conv_bn(x, prev, x, cin, width, 1, stride=stride, bn_prefix="bn_", scale_prefix="scale_")
            y = "res%s_branch2b" % tag
            b.conv_bn(y, x, y, width, width, 3, pad=1, bn_prefix="bn_", scale_prefix="scale_")
            z = "res%s_branch2c" % tag
            b.conv_bn(z, y, z, width, cout, 1, relu=False, bn_prefix="bn_", scale_prefix="scale_")
            out = "res%s" % tag
            b.eltwise_sum(out, [shortcut, z], out)
            b.relu(out + "_relu", out)
            prev, cin = out, cout
    b.pool("pool5", prev, "pool5", "AVE", global_pooling=True)
    b.inner_product("fc1000", "pool5", "fc1000", cin, num_classes)
    b.softmax("prob", "fc1000", "prob")
    return b


IMAGE_MEANS = (104.0, 117.0, 123.0)   # per-channel means subtracted from the U(0, 255) input


def image_input(batch, size=224, seed=0):
    rng = np.random.default_rng(seed + 2000)
    x = rng.uniform(0.0, 255.0, (batch, 3, size, size))
    x -= np.asarray(IMAGE_MEANS).reshape(1, 3, 1, 1)
    return {"data": x.astype(np.float32)}


def resnet50_conv_table():
    """One row per Convolution / InnerProduct of resnet50():
    (name, cin, cout, kernel, stride, in_size, out_size, fused_residual)."""
    rows = [("conv1", 3, 64, 7, 2, 224, 112, False)]
    h, cin = 56, 64
    for stage, blocks, width in [(2, 3, 64), (3, 4, 128), (4, 6, 256), (5, 3, 512)]:
        for i in range(blocks):
            tag = "%d%s" % (stage, "abcdefgh"[i])
            stride = 2 if (i == 0 and stage > 2) else 1
            ho = h // stride
            cout = width * 4
            if i == 0:
                rows.append(("res%s_branch1" % tag, cin, cout, 1, stride, h, ho, False))
            rows.append(("res%s_branch2a" % tag, cin, width, 1, stride, h, ho, False))
            rows.append(("res%s_branch2b" % tag, width, width, 3, 1, ho, ho, False))
            rows.append(("res%s_branch2c" % tag, width, cout, 1, 1, ho, ho, True))
            h, cin = ho, cout
    rows.append(("fc1000", cin, 1000, 1, 1, 1, 1, False))
    return rows


def resnet50_flops_per_image():
    """2 * MACs of every Convolution and the InnerProduct of resnet50()."""
    return sum(2 * cout * ho * ho * cin * k * k for _, cin, cout, k, _, _, ho, _ in resnet50_conv_table())


def resnet50_conv_bytes(batch, bf16_storage=False):
    """Algorithmic bytes of the convolution / inner-product kernels of one forward pass:
    element size * (input + output + weights [+ residual input when fused]) + 4 * per-channel
    terms, each tensor counted once per layer.  Elements are 4 bytes; with the engine's bfloat16
    storage the 48 convolutions between pool1 and pool5 read 2-byte activations, weights and
    residuals and write 2-byte results, except the last one, which writes fp32 for the average
    pool (conv1 and fc1000 stay fp32)."""
    total = 0
    table = resnet50_conv_table()
    for i, (name, cin, cout, k, _, hi, ho, res) in enumerate(table):
        narrow = bf16_storage and name not in ("conv1", "fc1000")
        es_in = 2 if narrow else 4
        es_out = 2 if (narrow and table[i + 1][0] != "fc1000") else 4
        total += es_in * (batch * cin * hi * hi + cout * cin * k * k) + es_out * batch * cout * ho * ho + 4 * cout
        if res:
            total += es_in * batch * cout * ho * ho
    return total


# --------------------------------------------------------------------------- config 3

def mobilenet_v1(batch, num_classes=1000):
    b = NetBuilder("mobilenet_v1")
    b.input([("data", (batch, 3, 224, 224))])
    b.conv_bn("conv1", "data", "conv1", 3, 32, 3, stride=2, pad=1, bn_prefix="bn_", scale_prefix="scale_")
    cfg = [(64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2), (512, 1), (512, 1), (512, 1), (512, 1),
           (512, 1), (1024, 2), (1024, 1)]
    prev, cin = "conv1", 32
    for i, (cout, stride) in enumerate(cfg):
        dw = "conv%d_dw" % (i + 2)
        b.conv_bn(dw, prev, dw, cin, cin, 3, stride=stride, pad=1, group=cin, bn_prefix="bn_", scale_prefix="scale_")
        pw = "conv%d_pw" % (i + 2)
        b.conv_bn(pw, dw, pw, cin, cout, 1, bn_prefix="bn_", scale_prefix="scale_")
        prev, cin = pw, cout
    b.pool("pool6", prev, "pool6", "AVE", global_pooling=True)
    b.conv("fc7", "pool6", "fc7", cin, num_classes, 1)
    b.softmax("prob", "fc7", "prob")
    return b


def wgan_generator(batch, noise=100, widths=(512, 256, 128, 64)):
    """The structure of mini-caffe's shipped WGAN generator (example/models/wgan/g.prototxt): noise
    [batch, 100, 1, 1] -> Deconvolution 4x4 to 4 x 4 x 512 -> three Deconvolutions 4x4 stride 2 pad 1
    (each followed by BatchNorm on batch statistics, Scale, ReLU) -> Deconvolution to 3 x 64 x 64 -> TanH."""
    b = NetBuilder("wgan_g")
    b.input([("z", (batch, noise, 1, 1))])
    prev, cin = "z", noise
    for i, cout in enumerate(widths):
        name = "deconv%d" % i
        geometry = "kernel_size: 4" if i == 0 else "kernel_size: 4 stride: 2 pad: 1"
        b.raw(name, "Deconvolution", [prev], [name], "convolution_param { num_output: %d %s bias_term: false }" % (cout, geometry))
        b.params.append((name + "_0", (cin, cout, 4, 4), "he", cin))
        b.raw("bn%d" % i, "BatchNorm", [name], [name], "batch_norm_param { use_global_stats: false }")
        for j, kind in enumerate(("bn_mean", "bn_var", "one")):
            b.params.append(("bn%d_%d" % (i, j), (cout,) if j < 2 else (1,), kind, 0))
        b.scale("scale%d" % i, name, cout)
        b.relu("relu%d" % i, name)
        prev, cin = name, cout
    b.raw("out", "Deconvolution", [prev], ["out"], "convolution_param { num_output: 3 kernel_size: 4 stride: 2 pad: 1 }")
    b.params.append(("out_0", (cin, 3, 4, 4), "he", cin))
    b.params.append(("out_1", (3,), "uniform", 0))
    b.raw("tanh", "TanH", ["out"], ["image"])
    return b


def wgan_noise(batch, noise=100, seed=0):
    return {"z": np.random.default_rng(seed + 5000).standard_normal((batch, noise, 1, 1)).astype(np.float32)}


def normal_image_input(batch, size=224, seed=0):
    return {"data": np.random.default_rng(seed + 3000).standard_normal((batch, 3, size, size)).astype(np.float32)}


# --------------------------------------------------------------------------- config 4

SSD_MIN_SIZES = (30.0, 60.0, 111.0, 162.0, 213.0, 264.0)
SSD_MAX_SIZES = (60.0, 111.0, 162.0, 213.0, 264.0, 315.0)
SSD_ASPECTS = ((2.0,), (2.0, 3.0), (2.0, 3.0), (2.0, 3.0), (2.0,), (2.0,))
SSD_STEPS = (8, 16, 32, 64, 100, 300)
SSD_NUM_CLASSES = 21


def ssd300_vgg16(batch, with_detection_output=True):
    b = NetBuilder("ssd300_vgg16")
    b.input([("data", (batch, 3, 300, 300))])
    prev, cin = "data", 3

    def block(idx, convs, cout):
        nonlocal prev, cin
        for j in range(convs):
            name = "conv%d_%d" % (idx, j + 1)
            b.conv(name, prev, name, cin, cout, 3, pad=1)
            b.relu("relu%d_%d" % (idx, j + 1), name)
            prev, cin = name, cout

    block(1, 2, 64)
    b.pool("pool1", prev, "pool1", "MAX", k=2, stride=2); prev = "pool1"
    block(2, 2, 128)
    b.pool("pool2", prev, "pool2", "MAX", k=2, stride=2); prev = "pool2"
    block(3, 3, 256)
    b.pool("pool3", prev, "pool3", "MAX", k=2, stride=2); prev = "pool3"      # 75 -> 38 (ceil)
    block(4, 3, 512)
    conv4_3 = prev
    b.pool("pool4", prev, "pool4", "MAX", k=2, stride=2); prev = "pool4"
    block(5, 3, 512)
    b.pool("pool5", prev, "pool5", "MAX", k=3, stride=1, pad=1); prev = "pool5"
    b.conv("fc6", prev, "fc6", 512, 1024, 3, pad=6, dilation=6); b.relu("relu6", "fc6")
    b.conv("fc7", "fc6", "fc7", 1024, 1024, 1); b.relu("relu7", "fc7")
    extras = [("conv6_1", 1024, 256, 1, 1, 0), ("conv6_2", 256, 512, 3, 2, 1),
              ("conv7_1", 512, 128, 1, 1, 0), ("conv7_2", 128, 256, 3, 2, 1),
              ("conv8_1", 256, 128, 1, 1, 0), ("conv8_2", 128, 256, 3, 1, 0),
              ("conv9_1", 256, 128, 1, 1, 0), ("conv9_2", 128, 256, 3, 1, 0)]
    prev = "fc7"
    for name, ci, co, k, s, p in extras:
        b.conv(name, prev, name, ci, co, k, stride=s, pad=p)
        b.relu(name + "_relu", name)
        prev = name
    b.raw("conv4_3_norm", "Normalize", [conv4_3], ["conv4_3_norm"],
          "norm_param { across_spatial: false channel_shared: false scale_filler { type: \"constant\" value: 20 } }")
    b.params.append(("conv4_3_norm_0", (512,), "norm_scale", 0))
    sources = [("conv4_3_norm", 512), ("fc7", 1024), ("conv6_2", 512), ("conv7_2", 256), ("conv8_2", 256),
               ("conv9_2", 256)]
    locs, confs, priors = [], [], []
    for i, (src, ci) in enumerate(sources):
        num_priors = 2 + 2 * len(SSD_ASPECTS[i])
        for kind, cout, store in (("loc", num_priors * 4, locs), ("conf", num_priors * SSD_NUM_CLASSES, confs)):
            name = "%s_mbox_%s" % (src, kind)
            b.conv(name, src, name, ci, cout, 3, pad=1, weight_init="head")
            b.raw(name + "_perm", "Permute", [name], [name + "_perm"],
                  "permute_param { order: 0 order: 2 order: 3 order: 1 }")
            b.raw(name + "_flat", "Flatten", [name + "_perm"], [name + "_flat"], "flatten_param { axis: 1 }")
            store.append(name + "_flat")
        pname = "%s_mbox_priorbox" % src
        ars = " ".join("aspect_ratio: %g" % a for a in SSD_ASPECTS[i])
        b.raw(pname, "PriorBox", [src, "data"], [pname],
              "prior_box_param { min_size: %g max_size: %g %s flip: true clip: false variance: 0.1 variance: 0.1 "
              "variance: 0.2 variance: 0.2 step: %d offset: 0.5 }" % (SSD_MIN_SIZES[i], SSD_MAX_SIZES[i], ars,
                                                                       SSD_STEPS[i]))
        priors.append(pname)
    b.raw("mbox_loc", "Concat", locs, ["mbox_loc"], "concat_param { axis: 1 }")
    b.raw("mbox_conf", "Concat", confs, ["mbox_conf"], "concat_param { axis: 1 }")
    b.raw("mbox_priorbox", "Concat", priors, ["mbox_priorbox"], "concat_param { axis: 2 }")
    b.raw("mbox_conf_reshape", "Reshape", ["mbox_conf"], ["mbox_conf_reshape"],
          "reshape_param { shape { dim: 0 dim: -1 dim: %d } }" % SSD_NUM_CLASSES)
    b.softmax("mbox_conf_softmax", "mbox_conf_reshape", "mbox_conf_softmax", axis=2)
    b.raw("mbox_conf_flatten", "Flatten", ["mbox_conf_softmax"], ["mbox_conf_flatten"], "flatten_param { axis: 1 }")
    if with_detection_output:
        b.raw("detection_out", "DetectionOutput", ["mbox_loc", "mbox_conf_flatten", "mbox_priorbox"],
              ["detection_out"],
              "detection_output_param { num_classes: %d share_location: true background_label_id: 0 "
              "nms_param { nms_threshold: 0.45 top_k: 400 } code_type: CENTER_SIZE keep_top_k: 200 "
              "confidence_threshold: 0.01 }" % SSD_NUM_CLASSES)
    return b


def ssd_input(batch, seed=0):
    return {"data": np.random.default_rng(seed + 4000).uniform(-1.0, 1.0, (batch, 3, 300, 300)).astype(np.float32)}


# --------------------------------------------------------------------------- config 5

PROPOSAL_SCALES_15 = (2, 4, 8, 16, 32)   # 5 scales x 3 ratios = the stated 15 anchors
PROPOSAL_SCALES_9 = (8, 16, 32)          # the literal 3 x 3 = 9-anchor variant
PROPOSAL_RATIOS = (0.5, 1.0, 2.0)


def proposal(num_anchors=15, height=63, width=38, pre_nms=6000, post_nms=300, nms_thresh=0.7, min_size=16,
             feat_stride=16, with_scores=False):
    scales = PROPOSAL_SCALES_15 if num_anchors == 15 else PROPOSAL_SCALES_9
    assert len(scales) * len(PROPOSAL_RATIOS) == num_anchors
    b = NetBuilder("proposal")
    b.input([("rpn_cls_prob", (1, 2 * num_anchors, height, width)),
             ("rpn_bbox_pred", (1, 4 * num_anchors, height, width)), ("im_info", (1, 3))])
    body = ("proposal_param { feat_stride: %d base_size: 16 min_size: %d pre_nms_topn: %d post_nms_topn: %d "
            "nms_thresh: %g %s %s }" % (feat_stride, min_size, pre_nms, post_nms, nms_thresh,
                                        " ".join("ratio: %g" % r for r in PROPOSAL_RATIOS),
                                        " ".join("scale: %g" % s for s in scales)))
    tops = ["rois", "scores"] if with_scores else ["rois"]
    b.raw("proposal", "Proposal", ["rpn_cls_prob", "rpn_bbox_pred", "im_info"], tops, body)
    return b


def proposal_input(num_anchors=15, height=63, width=38, seed=0, im_h=1000.0, im_w=600.0):
    """Scores ~ N(0, 1), deltas ~ N(0, 0.1^2).  Exact float ties among the scores would make
    the kept set depend on the sort algorithm's tie order, so tied foreground scores are
    re-drawn until all are distinct (the number of re-draws is returned)."""
    rng = np.random.default_rng(seed + 5000)
    scores = rng.standard_normal((1, 2 * num_anchors, height, width)).astype(np.float32)
    deltas = (rng.standard_normal((1, 4 * num_anchors, height, width)) * 0.1).astype(np.float32)
    fg = scores[0, num_anchors:].reshape(-1)
    redraws = 0
    while True:
        _, first, counts = np.unique(fg, return_index=True, return_counts=True)
        if (counts == 1).all():
            break
        dup = np.setdiff1d(np.arange(fg.size), first)
        fg[dup] = rng.standard_normal(dup.size).astype(np.float32)
        redraws += dup.size
    scores[0, num_anchors:] = fg.reshape(num_anchors, height, width)
    return {"rpn_cls_prob": scores, "rpn_bbox_pred": deltas,
            "im_info": np.array([[im_h, im_w, 1.0]], dtype=np.float32)}, redraws


# ----------------------------------------------------------------- region-of-interest pooling (R-FCN / Faster R-CNN heads)

def roi_pooling(kind="PSROIPooling", batch=1, height=63, width=38, num_rois=300, output_dim=21, group_size=7,
                channels=64, pooled_h=7, pooled_w=7, spatial_scale=1.0 / 16):
    """Input maps + Input rois -> one pooling layer.  PSROIPooling takes output_dim * group_size^2 score
    maps (R-FCN: 21 classes x 7 x 7 = 1029 maps); ROIPooling takes `channels` feature maps."""
    b = NetBuilder(kind.lower())
    c = output_dim * group_size * group_size if kind == "PSROIPooling" else channels
    b.input([("maps", (batch, c, height, width)), ("rois", (num_rois, 5))])
    if kind == "PSROIPooling":
        body = "psroi_pooling_param { spatial_scale: %.10g output_dim: %d group_size: %d }" % (
            spatial_scale, output_dim, group_size)
    else:
        body = "roi_pooling_param { pooled_h: %d pooled_w: %d spatial_scale: %.10g }" % (
            pooled_h, pooled_w, spatial_scale)
    b.raw("pool", kind, ["maps", "rois"], ["pooled"], body)
    return b


def roi_pooling_input(batch, channels, height, width, num_rois, seed=0, feat_stride=16.0):
    """Maps ~ N(0, 1).  Rois in image coordinates (the map times feat_stride): mostly boxes inside the image,
    plus the shapes the layers special-case: boxes hanging over every border, boxes smaller than a bin,
    degenerate boxes (x2 < x1), boxes entirely outside, and half-integer corners (round() half away from
    zero).  Column 0 is the image index."""
    rng = np.random.default_rng(seed + 9000)
    maps = rng.standard_normal((batch, channels, height, width)).astype(np.float32)
    im_w, im_h = width * feat_stride, height * feat_stride
    rois = np.zeros((num_rois, 5), dtype=np.float32)
    for r in range(num_rois):
        kind = r % 8
        x1, y1 = rng.uniform(0, im_w - 32), rng.uniform(0, im_h - 32)
        w, h = rng.uniform(8, im_w / 2), rng.uniform(8, im_h / 2)
        if kind == 1:      # over the right / bottom border
            x1, y1 = im_w - w / 2, im_h - h / 2
        elif kind == 2:    # over the left / top border
            x1, y1 = -w / 2, -h / 2
        elif kind == 3:    # smaller than one bin
            w, h = rng.uniform(0, 6), rng.uniform(0, 6)
        elif kind == 4:    # degenerate
            w, h = -rng.uniform(1, 40), rng.uniform(8, 100)
        elif kind == 5:    # outside the image
            x1, y1 = im_w + 50, im_h + 50
        elif kind == 6:    # corners on half integers
            x1, y1, w, h = np.floor(x1) + 0.5, np.floor(y1) + 0.5, np.floor(w) + 0.5, np.floor(h)
        rois[r] = (rng.integers(0, batch), x1, y1, x1 + w, y1 + h)
    return {"maps": maps, "rois": rois}


# ----------------------------------------------------------------- DetectionOutput alone (the SSD post-processing step)

def detection_head(batch, num_priors, num_classes, conf_thr, nms_thr, top_k, keep_top_k, code_type="CENTER_SIZE",
                   share_location=True):
    """Input loc / conf / prior -> DetectionOutput, with the layer's parameters spelled out."""
    loc_classes = 1 if share_location else num_classes
    b = NetBuilder("detout")
    b.input([("loc", (batch, num_priors * loc_classes * 4)), ("conf", (batch, num_priors * num_classes)),
             ("prior", (1, 2, num_priors * 4))])
    b.raw("detection_out", "DetectionOutput", ["loc", "conf", "prior"], ["detection_out"],
          "detection_output_param { num_classes: %d share_location: %s background_label_id: 0 "
          "nms_param { nms_threshold: %g top_k: %d } code_type: %s keep_top_k: %d confidence_threshold: %g }" %
          (num_classes, "true" if share_location else "false", nms_thr, top_k, code_type, keep_top_k, conf_thr))
    return b


def detection_head_input(batch, num_priors, num_classes, seed, share_location=True, peaked=False):
    """loc ~ N(0, 0.5^2); conf = softmax of N(0, s^2) logits (s = 3 "peaked": a few classes pass the
    threshold per prior; s = 0.3: near-uniform scores, every class passes, the top_k cut does the work);
    priors uniform in the unit square with SSD's variances (0.1, 0.1, 0.2, 0.2)."""
    rng = np.random.default_rng(seed)
    loc_classes = 1 if share_location else num_classes
    loc = (rng.standard_normal((batch, num_priors * loc_classes * 4)) * 0.5).astype(np.float32)
    logits = rng.standard_normal((batch, num_priors, num_classes)) * (3.0 if peaked else 0.3)
    e = np.exp(logits - logits.max(axis=2, keepdims=True))
    conf = (e / e.sum(axis=2, keepdims=True)).astype(np.float32).reshape(batch, -1)
    cx = rng.uniform(0.1, 0.9, num_priors)
    cy = rng.uniform(0.1, 0.9, num_priors)
    w = rng.uniform(0.05, 0.4, num_priors)
    h = rng.uniform(0.05, 0.4, num_priors)
    boxes = np.stack([cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2], axis=1).astype(np.float32)
    var = np.tile(np.array([0.1, 0.1, 0.2, 0.2], dtype=np.float32), (num_priors, 1))
    prior = np.stack([boxes.reshape(-1), var.reshape(-1)])[None].astype(np.float32)
    return {"loc": loc, "conf": conf, "prior": prior}


# ----------------------------------------------------------------- layer types of the shipped example nets

def extra_layers_net(batch=2):
    """A small network through Deconvolution (plain, strided + padded, grouped, dilated), Crop, Slice,
    BN and both LRN variants, shaped like their uses in the SSH detector and the WGAN generator."""
    b = NetBuilder("extra_layers")
    b.input([("data", (batch, 6, 9, 7)), ("like", (batch, 4, 13, 11))])
    b.raw("up", "Deconvolution", ["data"], ["up"],
          "convolution_param { num_output: 4 kernel_size: 4 stride: 2 pad: 1 }")
    b.params.append(("up_0", (6, 4, 4, 4), "he", 6 * 16))
    b.params.append(("up_1", (4,), "uniform", 0))
    b.raw("up_g", "Deconvolution", ["data"], ["up_g"],
          "convolution_param { num_output: 6 kernel_size: 3 stride: 1 pad: 1 group: 3 bias_term: false }")
    b.params.append(("up_g_0", (6, 2, 3, 3), "he", 18))
    b.raw("up_d", "Deconvolution", ["data"], ["up_d"],
          "convolution_param { num_output: 3 kernel_h: 2 kernel_w: 3 stride_h: 3 stride_w: 2 dilation: 2 }")
    b.params.append(("up_d_0", (6, 3, 2, 3), "he", 36))
    b.params.append(("up_d_1", (3,), "uniform", 0))
    b.raw("crop", "Crop", ["up", "like"], ["crop"], "crop_param { axis: 2 offset: 2 offset: 1 }")
    b.raw("crop1", "Crop", ["up", "like"], ["crop1"], "crop_param { axis: 2 offset: 1 }")
    b.raw("slice", "Slice", ["up_g"], ["s0", "s1", "s2"], "slice_param { axis: 1 slice_point: 1 slice_point: 4 }")
    b.raw("slice_even", "Slice", ["up"], ["e0", "e1"], "slice_param { axis: 2 }")
    b.raw("bn", "BN", ["crop"], ["bn"], "bn_param { frozen: true }")
    for i, kind in enumerate(("gamma", "beta", "bn_mean", "bn_var")):
        b.params.append(("bn_%d" % i, (1, 4), kind, 0))
    b.raw("lrn_a", "LRN", ["up_g"], ["lrn_a"], "lrn_param { local_size: 5 alpha: 0.0001 beta: 0.75 k: 2 }")
    b.raw("lrn_w", "LRN", ["bn"], ["lrn_w"],
          "lrn_param { local_size: 3 alpha: 0.05 beta: 0.75 norm_region: WITHIN_CHANNEL }")
    return b


EXTRA_LAYER_OUTPUTS = ("up", "up_g", "up_d", "crop", "crop1", "s0", "s1", "s2", "e0", "e1", "bn", "lrn_a", "lrn_w")


def extra_layers_input(batch=2, seed=0):
    rng = np.random.default_rng(seed + 7000)
    return {"data": rng.standard_normal((batch, 6, 9, 7)).astype(np.float32),
            "like": np.zeros((batch, 4, 13, 11), dtype=np.float32)}


# ----------------------------------------------------------------- algorithmic work of a generated network

def conv_work(builder, blob_shapes):
    """FLOPs and algorithmic bytes of the Convolution / InnerProduct layers of a generated network.

    blob_shapes: {blob name: shape} as the library reports them for this prototxt (Net construction
    needs no device).  Per layer, with fp32 elements:
        flops = 2 * N * Cout * Ho * Wo * (Cin / group) * Kh * Kw            (InnerProduct: 2 * M * N * K)
        bytes = 4 * (input elements + output elements + weight elements + Cout)
    every tensor counted once per layer (an activation written by one layer and read by the next is
    counted by both: each kernel has to move it once).  Fused residual inputs are not known at this
    level and are left out.  Returns {"flops", "bytes", "layers"}."""
    import re
    weights = {name: shape for name, shape, _, _ in builder.params}
    flops = 0
    nbytes = 0
    layers = 0
    for line in builder.lines:
        m = re.match(r'layer \{ name: "([^"]+)" type: "(Convolution|InnerProduct)"', line)
        if not m:
            continue
        name = m.group(1)
        bottom = re.search(r'bottom: "([^"]+)"', line).group(1)
        top = re.search(r'top: "([^"]+)"', line).group(1)
        w = weights[name + "_0"]
        n_in = int(np.prod(blob_shapes[bottom]))
        n_out = int(np.prod(blob_shapes[top]))
        n_w = int(np.prod(w))
        cout = w[0]
        # every output element takes (weight elements / Cout) multiply-adds
        flops += 2 * n_out * (n_w // cout)
        nbytes += 4 * (n_in + n_out + n_w + cout)
        layers += 1
    return {"flops": flops, "bytes": nbytes, "layers": layers}
