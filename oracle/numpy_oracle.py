"""CPU restatement (numpy) of mini-caffe's forward arithmetic for the dense
layers on the engine's hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under oracle/ is part of the product: the
engine never imports, links or calls it.  It exists so that tests can check the
CUDA kernels against an independent statement of what the reference computes,
also on machines where the compiled reference (oracle/_ref) is absent.

Pinning: the reference project ships no golden vectors or known-answer tests
for these layers, so this restatement is pinned against outputs of the
reference itself: tests/golden/*.npz were produced by running the reference's
unmodified CPU sources (oracle/_ref, built by oracle/Makefile) through
tests/golden/make_golden.py, and tests/test_oracle_cpu.py checks every
function here against them.

Each function cites the reference code it follows (paths relative to the
mini-caffe project).  All arithmetic is float32 like the reference; matrix
products go through numpy (whose BLAS may sum in a different order than
OpenBLAS does for the reference: agreement is to float32 rounding, about 1e-6
relative).
"""
import numpy as np

F = np.float32


def conv_out_size(size, kernel, stride, pad, dilation=1):
    """floor((in + 2p - (d(k-1)+1)) / s) + 1 -- src/layers/conv_layer.cpp:12-25."""
    ext = dilation * (kernel - 1) + 1
    return (size + 2 * pad - ext) // stride + 1


def im2col(x, kh, kw, stride, pad, dilation=1):
    """One image [C, H, W] -> [C*kh*kw, Ho*Wo]; zero padding.  src/util/im2col.cpp:19-55."""
    c, h, w = x.shape
    ho = conv_out_size(h, kh, stride, pad, dilation)
    wo = conv_out_size(w, kw, stride, pad, dilation)
    padded = np.zeros((c, h + 2 * pad, w + 2 * pad), dtype=F)
    padded[:, pad:pad + h, pad:pad + w] = x
    col = np.empty((c, kh, kw, ho, wo), dtype=F)
    for r in range(kh):
        for s in range(kw):
            y0, x0 = r * dilation, s * dilation
            col[:, r, s] = padded[:, y0:y0 + stride * (ho - 1) + 1:stride, x0:x0 + stride * (wo - 1) + 1:stride]
    return col.reshape(c * kh * kw, ho * wo), ho, wo


def convolution(x, weight, bias=None, stride=1, pad=0, dilation=1, group=1):
    """Per image: im2col, then per group W[Cout/g, K] x col[K, HoWo], then bias added as a
    rank-1 product.  src/layers/base_conv_layer.cpp:254-278."""
    n, c, h, w = x.shape
    cout, cin_g, kh, kw = weight.shape
    assert cin_g * group == c and cout % group == 0
    out = None
    for i in range(n):
        col, ho, wo = im2col(x[i], kh, kw, stride, pad, dilation)
        if out is None:
            out = np.empty((n, cout, ho, wo), dtype=F)
        kg = cin_g * kh * kw
        og = cout // group
        y = np.empty((cout, ho * wo), dtype=F)
        for g in range(group):
            y[g * og:(g + 1) * og] = weight[g * og:(g + 1) * og].reshape(og, kg) @ col[g * kg:(g + 1) * kg]
        if bias is not None:
            y += bias.astype(F)[:, None]
        out[i] = y.reshape(cout, ho, wo)
    return out


def inner_product(x, weight, bias=None, axis=1, transpose=False):
    """Y = X W^T (+ 1 b^T) over the dims from `axis` flattened.  src/layers/inner_product_layer.cpp:80-93."""
    m = int(np.prod(x.shape[:axis]))
    xm = x.reshape(m, -1).astype(F)
    y = xm @ (weight if transpose else weight.T)
    if bias is not None:
        y = y + bias.astype(F)[None, :]
    return y.astype(F).reshape(x.shape[:axis] + (y.shape[1],))


def batch_norm(x, mean, var, factor, eps=1e-5):
    """mean = b0/f, var = b1/f (f = b2[0], 0 -> 0); y = (x - mean) / (var + eps)^0.5, all float.
    src/layers/batch_norm_layer.cpp:83-135."""
    f = F(0) if factor == 0 else F(1) / F(factor)
    m = (mean.astype(F) * f).reshape(1, -1, *([1] * (x.ndim - 2)))
    v = (var.astype(F) * f + F(eps)).reshape(1, -1, *([1] * (x.ndim - 2)))
    return ((x - m) / np.power(v, F(0.5))).astype(F)


def scale(x, gamma, beta=None):
    """y = x * gamma[c] (+ beta[c]).  src/layers/scale_layer.cpp:96-113, bias_layer.cpp:68-83."""
    shape = (1, -1) + (1,) * (x.ndim - 2)
    y = x * gamma.astype(F).reshape(shape)
    if beta is not None:
        y = y + beta.astype(F).reshape(shape)
    return y.astype(F)


def relu(x, negative_slope=0.0):
    """max(x, 0) + slope * min(x, 0).  src/layers/relu_layer.cpp:12-29."""
    return (np.maximum(x, 0) + F(negative_slope) * np.minimum(x, 0)).astype(F)


def prelu(x, slopes, channel_shared=False):
    """max(x, 0) + slope[c] * min(x, 0).  src/layers/prelu_layer.cpp:52-84."""
    s = slopes.astype(F).reshape(-1)
    shape = (1, -1) + (1,) * (x.ndim - 2)
    sl = s[0] if channel_shared else s.reshape(shape)
    return (np.maximum(x, 0) + sl * np.minimum(x, 0)).astype(F)


def eltwise(inputs, op="SUM", coeffs=None):
    """SUM: 0 + sum coeff_i x_i in bottom order; PROD; MAX.  src/layers/eltwise_layer.cpp:37-78."""
    if op == "SUM":
        coeffs = coeffs or [1.0] * len(inputs)
        y = np.zeros_like(inputs[0], dtype=F)
        for c, x in zip(coeffs, inputs):
            y = y + F(c) * x
        return y.astype(F)
    if op == "PROD":
        y = inputs[0].astype(F)
        for x in inputs[1:]:
            y = y * x
        return y.astype(F)
    y = inputs[0]
    for x in inputs[1:]:
        y = np.maximum(y, x)
    return y.astype(F)


def pool_out_size(size, kernel, stride, pad):
    """ceil((in + 2p - k) / s) + 1, minus one if the last window would start in the padding.
    src/layers/pooling_layer.cpp:92-107."""
    out = int(np.ceil(F(size + 2 * pad - kernel) / F(stride))) + 1
    if pad and (out - 1) * stride >= size + pad:
        out -= 1
    return out


def pooling(x, method, kernel, stride=1, pad=0, global_pooling=False):
    """MAX over the window clipped to the image (start -FLT_MAX); AVE = sum over the clipped
    window / area of the window clipped to the padded image.  src/layers/pooling_layer.cpp:124-181."""
    n, c, h, w = x.shape
    kh, kw = (h, w) if global_pooling else (kernel, kernel)
    ho, wo = pool_out_size(h, kh, stride, pad), pool_out_size(w, kw, stride, pad)
    out = np.empty((n, c, ho, wo), dtype=F)
    for py in range(ho):
        for px in range(wo):
            y0, x0 = py * stride - pad, px * stride - pad
            if method == "MAX":
                y1, x1 = min(y0 + kh, h), min(x0 + kw, w)
                out[:, :, py, px] = x[:, :, max(y0, 0):y1, max(x0, 0):x1].max(axis=(2, 3))
            else:
                y1, x1 = min(y0 + kh, h + pad), min(x0 + kw, w + pad)
                area = F((y1 - y0) * (x1 - x0))
                win = x[:, :, max(y0, 0):min(y1, h), max(x0, 0):min(x1, w)]
                out[:, :, py, px] = win.sum(axis=(2, 3), dtype=F) / area
    return out


def softmax(x, axis=1):
    """Subtract the max over `axis`, exp (float), divide by the sum.  src/layers/softmax_layer.cpp:29-63."""
    m = x.max(axis=axis, keepdims=True)
    e = np.exp((x - m).astype(F)).astype(F)
    return (e / e.sum(axis=axis, keepdims=True, dtype=F)).astype(F)


def concat(inputs, axis=1):
    """src/layers/concat_layer.cpp:53-70."""
    return np.concatenate(inputs, axis=axis).astype(F)


def normalize(x, scale_values, eps=1e-10, channel_shared=False):
    """across_spatial = false: y = x / (sum_c x^2 + eps)^0.5 * scale[c].  src/layers/normalize_layer.cpp:86-135."""
    norm = np.power((x.astype(F) ** 2).sum(axis=1, keepdims=True, dtype=F) + F(eps), F(0.5))
    s = scale_values.astype(F).reshape(-1)
    sc = s[0] if channel_shared else s.reshape(1, -1, 1, 1)
    return (x / norm * sc).astype(F)


def permute(x, order):
    """src/layers/permute_layer.cpp:8-22."""
    return np.ascontiguousarray(np.transpose(x, order)).astype(F)


def conv_relu(x, weight, bias, pad=1):
    """The single Convolution + ReLU network of the first benchmark configuration."""
    return relu(convolution(x, weight, bias, stride=1, pad=pad))


def fold_batch_norm_scale(mean, var, factor, eps, gamma, beta, conv_bias=None):
    """Per-channel (scale, shift) such that scale * conv + shift == Scale(BatchNorm(conv + bias)).
    The folding algebra of tools/fuse_bn.py:34-38 with BatchNorm's scale factor blob
    (src/layers/batch_norm_layer.cpp:85-90)."""
    f = 0.0 if factor == 0 else 1.0 / float(factor)
    inv_std = 1.0 / np.sqrt(var.astype(np.float64) * f + eps)
    s = gamma.astype(np.float64) * inv_std
    b0 = conv_bias.astype(np.float64) if conv_bias is not None else 0.0
    t = (b0 - mean.astype(np.float64) * f) * s + beta.astype(np.float64)
    return s, t


def _round_half_away(x):
    """C round(): halves go away from zero (numpy's rint goes to even)."""
    x = F(x)
    return F(np.floor(np.abs(x) + F(0.5)) * np.sign(x)) if np.isfinite(x) else x


def roi_pooling(maps, rois, pooled_h, pooled_w, spatial_scale):
    """Max over an adaptive grid per roi; corners scaled then rounded; an empty bin gives 0.
    src/layers/roi_pooling_layer.cpp:37-109.  Loops in Python: small cases only."""
    n, c, h, w = maps.shape
    out = np.zeros((rois.shape[0], c, pooled_h, pooled_w), dtype=F)
    s = F(spatial_scale)
    for r, roi in enumerate(rois.astype(F)):
        b = int(roi[0])
        assert 0 <= b < n
        sw, sh, ew, eh = (int(_round_half_away(F(roi[i]) * s)) for i in (1, 2, 3, 4))
        rh, rw = max(eh - sh + 1, 1), max(ew - sw + 1, 1)
        bh, bw = F(rh) / F(pooled_h), F(rw) / F(pooled_w)
        for ph in range(pooled_h):
            hs = min(max(int(np.floor(F(ph) * bh)) + sh, 0), h)
            he = min(max(int(np.ceil(F(ph + 1) * bh)) + sh, 0), h)
            for pw in range(pooled_w):
                ws = min(max(int(np.floor(F(pw) * bw)) + sw, 0), w)
                we = min(max(int(np.ceil(F(pw + 1) * bw)) + sw, 0), w)
                if he > hs and we > ws:
                    out[r, :, ph, pw] = maps[b, :, hs:he, ws:we].max(axis=(1, 2))
    return out


def psroi_pooling(maps, rois, output_dim, group_size, spatial_scale):
    """Position-sensitive average: bin (ph, pw) of channel c averages score map (c*G + ph)*G + pw over
    the bin, summed row by row in float; corners rounded then scaled, far corner + 1; an empty bin gives 0.
    src/layers/psroi_pooling_layer.cpp:45-106.  Loops in Python: small cases only."""
    n, c, h, w = maps.shape
    g = group_size
    assert c == output_dim * g * g
    out = np.zeros((rois.shape[0], output_dim, g, g), dtype=F)
    s = F(spatial_scale)
    for r, roi in enumerate(rois.astype(F)):
        b = int(roi[0])
        assert 0 <= b < n
        sw, sh = F(_round_half_away(roi[1]) * s), F(_round_half_away(roi[2]) * s)
        ew, eh = F(_round_half_away(F(roi[3] + F(1))) * s), F(_round_half_away(F(roi[4] + F(1))) * s)
        rh, rw = max(F(eh - sh), F(0.1)), max(F(ew - sw), F(0.1))
        bh, bw = F(rh / F(g)), F(rw / F(g))
        for ph in range(g):
            hs = min(max(int(np.floor(F(F(ph) * bh) + sh)), 0), h)
            he = min(max(int(np.ceil(F(F(ph + 1) * bh) + sh)), 0), h)
            for pw in range(g):
                ws = min(max(int(np.floor(F(F(pw) * bw) + sw)), 0), w)
                we = min(max(int(np.ceil(F(F(pw + 1) * bw) + sw)), 0), w)
                if he <= hs or we <= ws:
                    continue
                for ch in range(output_dim):
                    plane = maps[b, (ch * g + ph) * g + pw]
                    acc = F(0)
                    for y in range(hs, he):
                        for x in range(ws, we):
                            acc = F(acc + plane[y, x])
                    out[r, ch, ph, pw] = F(acc / F((he - hs) * (we - ws)))
    return out


def deconvolution(x, weight, bias=None, stride=1, pad=0, dilation=1, group=1):
    """Transposed convolution: every input pixel scatters weight[ci, co] * x into the output at
    (iy * stride - pad + r * dilation, ...); weight is [C_in, C_out / group, kh, kw]; out = stride * (in - 1)
    + dilation * (k - 1) + 1 - 2 * pad.  src/layers/deconv_layer.cpp:7-44 (GEMM with the transposed
    weights, then col2im), src/layers/base_conv_layer.cpp:280-296."""
    n, c, h, w = x.shape
    _, cout_g, kh, kw = weight.shape
    cin_g = c // group
    ho = stride * (h - 1) + dilation * (kh - 1) + 1 - 2 * pad
    wo = stride * (w - 1) + dilation * (kw - 1) + 1 - 2 * pad
    full = np.zeros((n, cout_g * group, ho + 2 * pad, wo + 2 * pad), dtype=np.float64)
    for g in range(group):
        xg = x[:, g * cin_g:(g + 1) * cin_g].astype(np.float64)
        wg = weight[g * cin_g:(g + 1) * cin_g].astype(np.float64)
        for r in range(kh):
            for q in range(kw):
                contrib = np.einsum("nchw,co->nohw", xg, wg[:, :, r, q])
                y0, x0 = r * dilation, q * dilation
                full[:, g * cout_g:(g + 1) * cout_g, y0:y0 + stride * (h - 1) + 1:stride,
                     x0:x0 + stride * (w - 1) + 1:stride] += contrib
    out = full[:, :, pad:pad + ho, pad:pad + wo]
    if bias is not None:
        out = out + bias.astype(np.float64).reshape(1, -1, 1, 1)
    return out.astype(F)


def lrn(x, local_size=5, alpha=1.0, beta=0.75, k=1.0, within_channel=False):
    """ACROSS_CHANNELS: y = x * (k + alpha/size * sum of x^2 over `size` neighbouring channels)^-beta
    (src/layers/lrn_layer.cpp:107-150).  WITHIN_CHANNEL: y = x * (1 + alpha * AVE-pool(x^2, size, pad
    (size-1)/2))^-beta, the pooling being the reference's (divides by the window clipped to the padded
    plane) (src/layers/lrn_layer.cpp:19-66,152-159)."""
    if within_channel:
        pooled = pooling((x.astype(F) ** 2).astype(F), "AVE", local_size, stride=1, pad=(local_size - 1) // 2)
        return (x * np.power(F(1) + F(alpha) * pooled, F(-beta))).astype(F)
    n, c, h, w = x.shape
    pre = (local_size - 1) // 2
    sq = np.zeros((n, c + local_size - 1, h, w), dtype=F)
    sq[:, pre:pre + c] = x.astype(F) ** 2
    scale = np.full(x.shape, F(k), dtype=F)
    for j in range(local_size):
        scale += F(alpha / local_size) * sq[:, j:j + c]
    return (x * np.power(scale, F(-beta))).astype(F)


def bn(x, slope, bias, mean, factor):
    """Inference path of the fused-parameter BN layer: y = ((x - mean) * factor) * slope + bias, `factor`
    being what the layer's fourth blob holds (src/layers/bn_layer.cpp:66-133)."""
    shape = (1, -1) + (1,) * (x.ndim - 2)
    y = (x - mean.astype(F).reshape(shape)) * factor.astype(F).reshape(shape)
    return (y * slope.astype(F).reshape(shape) + bias.astype(F).reshape(shape)).astype(F)


def slice_blob(x, axis, slice_points=None, num_tops=None):
    """src/layers/slice_layer.cpp:18-96."""
    if slice_points:
        return [a.astype(F) for a in np.split(x, list(slice_points), axis=axis)]
    return [a.astype(F) for a in np.split(x, num_tops, axis=axis)]


def crop(x, like_shape, axis=2, offsets=(0,)):
    """Cut x to like_shape from `axis` on, starting at the offsets (one for all axes, or one per
    cropped axis).  src/layers/crop_layer.cpp:28-100."""
    idx = [slice(None)] * x.ndim
    for i in range(axis, x.ndim):
        off = offsets[0] if len(offsets) == 1 else offsets[i - axis]
        idx[i] = slice(off, off + like_shape[i])
    return np.ascontiguousarray(x[tuple(idx)]).astype(F)
