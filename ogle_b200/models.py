"""Builders of dlx models in the form the reference's ONNX converter emits.

What the converter produces, restated (converter/converter/onnx/onnx_converter.cc:43-193,
onnx/ops/*.cc, optimizers/remapper.cc:97-204 in kl456123/OGLE):
  - one Input node per graph input carrying the ONNX (NCHW) dims;
  - one Const node per initializer, emitted just before its first consumer: conv
    filters data_format ANY -> target HWN4C4, everything else ANY -> ANY4; int64
    initializers stored as floats;
  - Conv -> BatchNormalization [-> Relu|Clip] folded into the Conv: W' = W*scale,
    b' = b*scale + (beta - scale*mean), scale = gamma/sqrt(var+eps), all in fp32;
    the activation becomes conv2d_attr.activation_type; a zero bias Const named
    "<conv>:2" is created when the conv had none; the node takes the name of the
    last fused node's output;
  - node name == name of its first output tensor; producer_name "ONNX".
Weights are seeded random: there is no trained checkpoint in this repository.
"""
import math

import numpy as np

from . import dlx


def fold_batchnorm(w, b, gamma, beta, mean, var, eps):
    """remapper.cc:142-149, evaluated in fp32 like the converter does."""
    w = np.array(w, dtype=np.float32, copy=True)
    K = w.shape[0]
    b = np.zeros(K, np.float32) if b is None else np.array(b, dtype=np.float32, copy=True)
    eps = np.float32(eps)
    for i in range(K):
        scale = np.float32(gamma[i]) / np.float32(np.sqrt(np.float32(var[i]) + eps))
        bias = np.float32(-scale * np.float32(mean[i]) + np.float32(beta[i]))
        w[i] = w[i] * scale
        b[i] = np.float32(b[i] * scale + bias)
    return w, b


class _Builder:
    def __init__(self, seed, weight_std):
        self.s = dlx.Scope()
        self.rng = np.random.default_rng(seed)
        self.he = weight_std == "he"
        self.std = np.float32(0.0 if self.he else weight_std)
        self.counter = 0
        self.flops = 0          # 2*MACs of every conv/gemm, per image
        self.conv_nodes = 0

    def name(self):
        self.counter += 1
        return str(self.counter + 100)

    def weights(self, shape):
        """N(0, weight_std); weight_std "he" scales by sqrt(2/fan_in) so that activations
        keep unit scale through the network (used by parity tests)."""
        if self.he:
            fan_in = int(np.prod(shape[1:])) if len(shape) > 1 else 1
            std = np.float32(math.sqrt(2.0 / fan_in)) if len(shape) > 1 else np.float32(0.1)
        else:
            std = self.std
        return (self.rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float32)

    def conv(self, x, cin, cout, k, stride=1, pad=0, group=1, bn=True, act="Relu", bias=False, hw=None, name=None):
        """Conv [+ identity-statistics BN folded] [+ fused activation]. Returns tensor id."""
        w = self.weights((cout, cin // group, k, k))
        b = self.weights((cout,)) if bias else None
        if bn:
            ones, zeros = np.ones(cout, np.float32), np.zeros(cout, np.float32)
            w, b = fold_batchnorm(w, b, ones, zeros, zeros, ones, 1e-5)
        name = name or self.name()
        wid = self.s.add_const(name + ".weight", w, dlx.ANY, dlx.HWN4C4)
        bid = None
        if b is not None:
            # remapper.cc:66-68 names the bias it creates "<node>:<input index>"
            bid = self.s.add_const(name + (":2" if (bn and not bias) else ".bias"), b, dlx.ANY, dlx.ANY4)
        out = self.s.add_conv(name, x, wid, bid, k, stride, pad, 1, group, act if bn or act else "", 0.0, 0.0)
        self.conv_nodes += 1
        if hw is not None:
            ho = (hw - k + 2 * pad) // stride + 1
            self.flops += 2 * ho * ho * cout * (cin // group) * k * k
            return out, ho
        return out


def ssd_prior_boxes(image_size=300, maps=(19, 10, 5, 3, 2, 1), min_sizes=(60, 105, 150, 195, 240, 285),
                    max_sizes=(105, 150, 195, 240, 285, 330), anchors_per_cell=(3, 6, 6, 6, 6, 6)):
    """Centre-size priors (cx, cy, w, h) in [0,1] for an SSD-300 head: per cell a
    square of min_size, then (6-anchor maps) a square of sqrt(min*max), then aspect
    ratios 2, 1/2 and (6-anchor maps) 3, 1/3 of the min_size box. Clipped to [0,1]."""
    out = []
    for f, smin, smax, n in zip(maps, min_sizes, max_sizes, anchors_per_cell):
        s = smin / image_size
        sp = math.sqrt(s * smax / image_size)
        for i in range(f):
            for j in range(f):
                cx, cy = (j + 0.5) / f, (i + 0.5) / f
                boxes = [(s, s)]
                if n == 6:
                    boxes.append((sp, sp))
                ratios = (2.0,) if n == 3 else (2.0, 3.0)
                for r in ratios:
                    q = math.sqrt(r)
                    boxes += [(s * q, s / q), (s / q, s * q)]
                assert len(boxes) == n
                out += [(cx, cy, w, h) for w, h in boxes]
    return np.clip(np.array(out, dtype=np.float32), 0.0, 1.0)


MOBILENET_V1 = [  # (out_channels, stride) of the 13 depthwise-separable blocks
    (64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2), (512, 1), (512, 1), (512, 1), (512, 1), (512, 1),
    (1024, 2), (1024, 1)]
SSD_EXTRAS = [(256, 512), (128, 256), (128, 256), (64, 128)]   # (1x1 width, 3x3-s2 width)


def mobilenet_v1_ssd(batch=1, num_classes=2, image_size=300, seed=0, weight_std=0.02, exported_shape_ops=False):
    """MobileNet-v1-SSD 300x300: stem 3x3 s2 32ch; 13 depthwise-separable blocks
    (depthwise 3x3 + 1x1 pointwise, BN+ReLU folded) up to 1024ch at 10x10; 4 extra
    1x1 / 3x3-s2 blocks giving 5x5, 3x3, 2x2, 1x1 maps; 3x3 loc/conf heads with
    3/6/6/6/6/6 anchors on the six maps (1917 anchors). Outputs "box_preds"
    [N,1917,4], "cls_logits" [N,1917,C] and the constant "anchors" [1917,4].
    exported_shape_ops: build every head's Reshape target the way an ONNX export of
    `y.view(y.size(0), -1, width)` does - Shape -> Gather(index 0) -> Unsqueeze(axes [0]) ->
    Concat with the constants [-1] and [width] - instead of one constant
    (converter/converter/onnx/ops/shape.cc, gather.cc, unsqueeze.cc emit those nodes as they are).
    Same weights either way. Returns (dlx.Model, info dict)."""
    b = _Builder(seed, weight_std)
    s = b.s
    x = s.add_input("input", [batch, 3, image_size, image_size])
    x, hw = b.conv(x, 3, 32, 3, 2, 1, hw=image_size)
    cin = 32
    sources = []
    for i, (cout, stride) in enumerate(MOBILENET_V1):
        x, hw = b.conv(x, cin, cin, 3, stride, 1, group=cin, hw=hw)
        x, hw = b.conv(x, cin, cout, 1, hw=hw)
        cin = cout
        if i in (10, 12):
            sources.append((x, cin, hw))
    for mid, cout in SSD_EXTRAS:
        x, hw = b.conv(x, cin, mid, 1, hw=hw)
        x, hw = b.conv(x, mid, cout, 3, 2, 1, hw=hw)
        cin = cout
        sources.append((x, cin, hw))
    anchors_per_cell = (3, 6, 6, 6, 6, 6)
    locs, confs = [], []
    total = 0
    for (src, c, fhw), a in zip(sources, anchors_per_cell):
        total += fhw * fhw * a
        for width, bucket in ((4, locs), (num_classes, confs)):
            y, _ = b.conv(src, c, a * width, 3, 1, 1, bn=False, act="", bias=True, hw=fhw)
            t = s.add_node(b.name(), "Transpose", [y], {"transpose_attr": {"perm": [0, 2, 3, 1]}})
            if exported_shape_ops:
                dims = s.add_node(b.name(), "Shape", [y], {"shape_attr": {}})
                index = s.add_const(b.name(), np.array(0, np.float32), dlx.ANY, dlx.ANY4)      # scalar: x.size(0)
                n = s.add_node(b.name(), "Gather", [dims, index], {"gather_attr": {"axis": 0}})
                n = s.add_node(b.name(), "Unsqueeze", [n], {"unsqueeze_attr": {"axes": [0]}})
                rest = [s.add_const(b.name(), np.array([v], np.float32), dlx.ANY, dlx.ANY4) for v in (-1, width)]
                shape = s.add_node(b.name(), "Concat", [n] + rest, {"concat_attr": {"axis": 0}})
            else:
                shape = s.add_const(b.name(), np.array([batch, -1, width], np.float32), dlx.ANY, dlx.ANY4)
            bucket.append(s.add_node(b.name(), "Reshape", [t, shape], {"reshape_attr": {}}))
    s.add_node("box_preds", "Concat", locs, {"concat_attr": {"axis": 1}})
    s.add_node("cls_logits", "Concat", confs, {"concat_attr": {"axis": 1}})
    priors = ssd_prior_boxes(image_size, [h for _, _, h in sources], anchors_per_cell=anchors_per_cell)
    assert priors.shape[0] == total
    s.add_const("anchors", priors, dlx.ANY, dlx.ANY4)
    for n in ("cls_logits", "box_preds", "anchors"):
        s.add_output_name(n)
    info = dict(flops_per_image=b.flops, conv_nodes=b.conv_nodes, num_anchors=total, num_classes=num_classes,
                image_size=image_size, batch=batch, extras=SSD_EXTRAS)
    return s.model, info


def resnet18(batch=1, num_classes=1000, image_size=224, seed=0, weight_std=0.02):
    """ResNet-18-style classifier: 7x7 s2 conv 64ch + BN/ReLU + 3x3 s2 maxpool, four
    stages of two basic blocks (64/128/256/512ch, stride-2 3x3 downsampling with a
    1x1 projection), global average pool, Flatten, Gemm 512 -> num_classes. Output "logits"."""
    b = _Builder(seed, weight_std)
    s = b.s
    x = s.add_input("input", [batch, 3, image_size, image_size])
    x, hw = b.conv(x, 3, 64, 7, 2, 3, hw=image_size)
    x = s.add_node(b.name(), "MaxPool", [x], {"maxpool_attr": {"kernel_shape": [3, 3], "strides": [2, 2], "pads": [1] * 4}})
    hw = (hw - 3 + 2) // 2 + 1
    cin = 64
    for stage, cout in enumerate((64, 128, 256, 512)):
        for blk in range(2):
            stride = 2 if (stage > 0 and blk == 0) else 1
            y, hw2 = b.conv(x, cin, cout, 3, stride, 1, hw=hw)
            y, _ = b.conv(y, cout, cout, 3, 1, 1, act="", hw=hw2)
            sc = x
            if stride != 1 or cin != cout:
                sc, _ = b.conv(x, cin, cout, 1, stride, 0, act="", hw=hw)
            y = s.add_node(b.name(), "Add", [y, sc], {"binary_attr": {"binary_op_type": "Add"}})
            x = s.add_node(b.name(), "Relu", [y], {"relu_attr": {}})
            cin, hw = cout, hw2
    x = s.add_node(b.name(), "GlobalAveragePool", [x])
    x = s.add_node(b.name(), "Flatten", [x], {"flatten_attr": {"axis": 1}})
    w = s.add_const("fc.weight", b.weights((num_classes, cin)), dlx.ANY, dlx.ANY4)
    bias = s.add_const("fc.bias", b.weights((num_classes,)), dlx.ANY, dlx.ANY4)
    b.flops += 2 * cin * num_classes
    s.add_node("logits", "Gemm", [x, w, bias], {"gemm_attr": {"alpha": 1.0, "beta": 1.0, "transB": 1}})
    s.add_output_name("logits")
    return s.model, dict(flops_per_image=b.flops, conv_nodes=b.conv_nodes, batch=batch, image_size=image_size)


def box_decoder_graph(map_h, map_w, seed=0):
    """The Decoder operator as a graph node (nn/kernels/decoder.cc:12-92): an input of box deltas
    [1, 4, map_h, map_w] (stored NHWC), reshaped to [1, map_h*map_w, 4], decoded against a constant
    anchor tensor [1, map_h, map_w, 4] (cx, cy, w, h) with the kernel's fixed variances. Output "boxes".
    Returns (dlx.Model, anchors array [map_h*map_w, 4])."""
    s = dlx.Scope()
    rng = np.random.default_rng(seed)
    anchors = np.concatenate([rng.random((map_h * map_w, 2), dtype=np.float32),
                              rng.random((map_h * map_w, 2), dtype=np.float32) * np.float32(0.4) + np.float32(0.05)], axis=1)
    x = s.add_input("input", [1, 4, map_h, map_w])
    shape = s.add_const("deltas.shape", np.array([1, -1, 4], np.float32), dlx.ANY, dlx.ANY4)
    pred = s.add_node("deltas", "Reshape", [x, shape], {"reshape_attr": {}})
    a = s.add_const("anchors", anchors.reshape(1, map_h, map_w, 4), dlx.ANY, dlx.ANY4)
    s.add_node("boxes", "Decoder", [pred, a], {})
    s.add_output_name("boxes")
    return s.model, anchors


def concat_of_convs(x_shape, widths, seed=0, kernels=(1,), consumer=True):
    """input -> len(widths) convolutions (branch i: kernels[i % len(kernels)] x same, pad to keep the size, ReLU on the
    first half of the branches) -> Concat on the channel axis (ONNX axis 1) [-> 1x1 conv "output"]: the graph shape
    where producers can write a concat in place. Output "cat" (and "output"). Returns dlx.Model."""
    s = dlx.Scope()
    rng = np.random.default_rng(seed)
    N, H, W, C = x_shape
    x = s.add_input("input", [N, C, H, W])
    parts = []
    for i, k_out in enumerate(widths):
        kernel = kernels[i % len(kernels)]
        w = (rng.standard_normal((k_out, C, kernel, kernel), dtype=np.float32) * np.float32(0.2)).astype(np.float32)
        b = rng.standard_normal(k_out, dtype=np.float32)
        wid = s.add_const(f"branch{i}.weight", w, dlx.ANY, dlx.HWN4C4)
        bid = s.add_const(f"branch{i}.bias", b, dlx.ANY, dlx.ANY4)
        parts.append(s.add_conv(f"branch{i}", x, wid, bid, kernel, 1, kernel // 2, 1, 1, "Relu" if 2 * i < len(widths) else "", 0.0, 0.0))
    cat = s.add_node("cat", "Concat", parts, {"concat_attr": {"axis": 1}})
    s.add_output_name("cat")
    if consumer:
        total = sum(widths)
        w = (rng.standard_normal((8, total, 1, 1), dtype=np.float32) * np.float32(0.1)).astype(np.float32)
        wid = s.add_const("output.weight", w, dlx.ANY, dlx.HWN4C4)
        s.add_conv("output", cat, wid, None, 1, 1, 0, 1, 1, "", 0.0, 0.0)
        s.add_output_name("output")
    return s.model


def single_conv(x_shape, w, bias=None, stride=1, pad=0, dilation=1, group=1, activation="", min_=0.0, max_=0.0):
    """One-op graph of the shape the reference's conv2d_test.cc:111-137 builds."""
    s = dlx.Scope()
    N, H, W, C = x_shape
    x = s.add_input("input", [N, C, H, W])
    wid = s.add_const("conv2d1.weight", w, dlx.NCHW, dlx.HWN4C4)
    bid = s.add_const("conv2d1.bias", bias, dlx.ANY, dlx.ANY4) if bias is not None else None
    s.add_conv("output", x, wid, bid, w.shape[2], stride, pad, dilation, group, activation, min_, max_)
    s.add_output_name("output")
    return s.model
