"""Thin Python front end over the C ABI (include/ogle_cuda.h), one function per
entry point, working on torch CUDA tensors. torch is used for device memory and
the current stream only; every computation is a call into libogle_cuda.so.

Activations are "padded" tensors: shape [..., round_up(C,4)] fp32 contiguous,
the reference's NHWC4/ANY4 byte layout. `upload`/`download` convert from and to
dense host arrays with the library's own pad/unpad kernels, the way the
reference's Context copies do (ogl_runtime/opengl/core/context.cc:123-185).
"""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import (ACT_CLIP, ACT_NONE, ACT_RELU, MATH_FP32, MATH_TF32, MATH_TF32X3,  # noqa: F401
                   ConcatParams, ConvParams, DetectParams, GemmParams, PoolParams, check)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def up4(v):
    return (v + 3) // 4 * 4


def _require_cuda(*ts):
    for t in ts:
        if t is not None and (not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous()):
            raise ValueError("expected contiguous fp32 CUDA tensors")


def upload(x, stride=0):
    """Dense host array [..., last] -> padded device tensor [..., round_up(last,4)]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    last = x.shape[-1]
    rows = x.size // last
    d = torch.from_numpy(x).cuda()
    s = stride or up4(last)
    out = torch.empty(x.shape[:-1] + (s,), dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_pad4(_p(d), _p(out), rows, last, s, _stream()), "pad4")
    return out


def download(t, last):
    """Padded device tensor -> dense host array [..., last]."""
    _require_cuda(t)
    stride = t.shape[-1]
    rows = t.numel() // stride
    out = torch.empty(t.shape[:-1] + (last,), dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_unpad4(_p(t), _p(out), rows, last, stride, _stream()), "unpad4")
    return out.cpu().numpy()


def dense_to_device(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def conv_params(N, H, W, Cin, K, kernel, stride=1, pad=0, dilation=1, group=1, has_bias=True, act=ACT_NONE,
                lo=0.0, hi=0.0, math_mode=MATH_FP32, in_stride=0, out_stride=0, out_offset=0):
    p = ConvParams()
    p.N = N
    p.in_hwc[:] = [H, W, Cin]
    p.out_hwc[:] = [0, 0, K]
    p.kernel, p.stride, p.pad, p.dilation, p.group = kernel, stride, pad, dilation, group
    p.has_bias, p.act, p.min_value, p.max_value = int(has_bias), act, lo, hi
    p.in_channel_stride, p.out_channel_stride, p.out_channel_offset = in_stride, out_stride, out_offset
    p.math_mode = math_mode
    check(_lib.cuda_lib().ogle_cuda_conv2d_infer(C.byref(p)), "conv2d_infer")
    return p


def conv2d_prepack(p, w_oihw):
    """w_oihw: dense device tensor [K, C/group, k, k] -> opaque packed filter (device bytes)."""
    _require_cuda(w_oihw)
    lib = _lib.cuda_lib()
    nbytes = lib.ogle_cuda_conv2d_filter_bytes(C.byref(p))
    if nbytes == 0:
        raise _lib.OgleError("conv2d_filter_bytes: invalid parameters")
    packed = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    check(lib.ogle_cuda_conv2d_prepack(C.byref(p), _p(w_oihw), _p(packed), _stream()), "conv2d_prepack")
    return packed


def conv_workspace(p):
    """Scratch tensor of the size ogle_cuda_conv2d_workspace_bytes asks for (None when the layer wants none)."""
    n = int(_lib.cuda_lib().ogle_cuda_conv2d_workspace_bytes(C.byref(p)))
    return torch.empty(n // 4, dtype=torch.float32, device="cuda") if n else None


def conv2d(p, x4, packed, bias=None, out=None, workspace="auto"):
    """workspace: "auto" lends the scratch the layer asks for (what the session does), None lends none,
    or a float32 device tensor."""
    _require_cuda(x4, packed, bias)
    Ho, Wo, K = p.out_hwc
    ks = p.out_channel_stride or up4(K)
    if out is None:
        out = torch.zeros((p.N, Ho, Wo, ks), dtype=torch.float32, device="cuda") if ks != up4(K) else \
            torch.empty((p.N, Ho, Wo, ks), dtype=torch.float32, device="cuda")
    if isinstance(workspace, str):
        workspace = conv_workspace(p)
    check(_lib.cuda_lib().ogle_cuda_conv2d_ws(C.byref(p), _p(x4), _p(packed), _p(bias), _p(out), _p(workspace),
                                               workspace.numel() * 4 if workspace is not None else 0, _stream()), "conv2d")
    return out


def conv2d_residual(p, x4, packed, bias, residual4, out=None):
    """act(conv(x) + bias + residual) in one pass (ogle_cuda_conv2d_residual); residual4 has the output's shape."""
    _require_cuda(x4, packed, bias, residual4)
    Ho, Wo, K = p.out_hwc
    if out is None:
        out = torch.empty((p.N, Ho, Wo, up4(K)), dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_conv2d_residual(C.byref(p), _p(x4), _p(packed), _p(bias), _p(residual4),
                                                    residual4.shape[-1], _p(out), _stream()), "conv2d_residual")
    return out


def conv2d_pair(x4, w1, b1, w2, b2, N, H, W, Cin, kernel, stride=1, pad=0, dilation=1, act=ACT_NONE, lo=0.0, hi=0.0,
                math_mode=MATH_TF32X3, use_workspace=True):
    """Two convolutions over the same input in one pass (w1/w2 dense OIHW device tensors, b1/b2 device
    vectors or None). Returns (y1, y2) as padded NHWC4 device tensors."""
    _require_cuda(x4, w1, w2, b1, b2)
    K1, K2 = w1.shape[0], w2.shape[0]
    split = (K1 + 31) // 32 * 32
    w = torch.zeros((split + K2,) + tuple(w1.shape[1:]), dtype=torch.float32, device="cuda")
    w[:K1] = w1
    w[split:] = w2
    bias = None
    if b1 is not None:
        bias = torch.zeros(split + K2, dtype=torch.float32, device="cuda")
        bias[:K1] = b1[:K1]
        bias[split:] = b2[:K2]
    p = conv_params(N, H, W, Cin, split + K2, kernel, stride, pad, dilation, 1, bias is not None, act, lo, hi, math_mode)
    lib = _lib.cuda_lib()
    if not lib.ogle_cuda_conv2d_pair_supported(C.byref(p)):
        raise _lib.OgleError("conv2d_pair: these parameters are not served by the tensor-core path")
    packed = conv2d_prepack(p, w)
    Ho, Wo, _ = p.out_hwc
    y1 = torch.full((N, Ho, Wo, up4(K1)), float("nan"), dtype=torch.float32, device="cuda")
    y2 = torch.full((N, Ho, Wo, up4(K2)), float("nan"), dtype=torch.float32, device="cuda")
    n_ws = int(lib.ogle_cuda_conv2d_pair_workspace_bytes(C.byref(p), K1, split)) if use_workspace else 0
    ws = torch.empty(n_ws // 4, dtype=torch.float32, device="cuda") if n_ws else None
    check(lib.ogle_cuda_conv2d_pair_ws(C.byref(p), _p(x4), _p(packed), _p(bias), K1, split, _p(y1), _p(y2), _p(ws), n_ws,
                                       _stream()), "conv2d_pair")
    return y1, y2


def pool_params(N, H, W, Cc, kernel, stride, pad, type_):
    p = PoolParams()
    p.N = N
    p.in_hwc[:] = [H, W, Cc]
    p.kernel, p.stride, p.pad, p.type = kernel, stride, pad, type_
    check(_lib.cuda_lib().ogle_cuda_pool_infer(C.byref(p)), "pool_infer")
    return p


def pool(p, x4):
    _require_cuda(x4)
    Ho, Wo, Cc = p.out_hwc
    out = torch.empty((p.N, Ho, Wo, up4(Cc)), dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_pool(C.byref(p), _p(x4), _p(out), _stream()), "pool")
    return out


def batchnorm(x4, gamma, beta, mean, var, Cc, eps):
    _require_cuda(x4, gamma, beta, mean, var)
    out = torch.empty_like(x4)
    pixels = x4.numel() // x4.shape[-1]
    check(_lib.cuda_lib().ogle_cuda_batchnorm(_p(x4), _p(gamma), _p(beta), _p(mean), _p(var), _p(out),
                                              pixels, Cc, x4.shape[-1], eps, _stream()), "batchnorm")
    return out


def relu(x4):
    out = torch.empty_like(x4)
    check(_lib.cuda_lib().ogle_cuda_relu(_p(x4), _p(out), x4.numel(), _stream()), "relu")
    return out


def clip(x4, lo, hi):
    out = torch.empty_like(x4)
    check(_lib.cuda_lib().ogle_cuda_clip(_p(x4), _p(out), x4.numel(), lo, hi, _stream()), "clip")
    return out


def add(a4, b4):
    out = torch.empty_like(a4)
    check(_lib.cuda_lib().ogle_cuda_add(_p(a4), _p(b4), _p(out), a4.numel(), _stream()), "add")
    return out


def add_act(a4, b4, act=ACT_RELU, lo=0.0, hi=0.0):
    """act(a + b) in one pass (a residual block's Add -> Relu / Clip)."""
    out = torch.empty_like(a4)
    check(_lib.cuda_lib().ogle_cuda_add_act(_p(a4), _p(b4), _p(out), a4.numel(), act, lo, hi, _stream()), "add_act")
    return out


def gemm(A4, B4, C4, M, K, N, transB=0, alpha=1.0, beta=1.0, bias_mode=0, math_mode=MATH_FP32):
    """A4 [M, up4(K)], B4 [K, up4(N)] or [N, up4(K)] when transB; C4 [M, up4(N)] or [up4(N)]."""
    _require_cuda(A4, B4, C4)
    p = GemmParams()
    p.M, p.K, p.N, p.transB, p.alpha, p.beta, p.bias_mode = M, K, N, transB, alpha, beta, bias_mode
    p.lda, p.ldb = A4.shape[-1], B4.shape[-1]
    p.ldc = C4.shape[-1] if (C4 is not None and bias_mode == 1) else 0
    p.ldy = up4(N)
    p.math_mode = math_mode
    out = torch.empty((M, up4(N)), dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_gemm(C.byref(p), _p(A4), _p(B4), _p(C4), _p(out), _stream()), "gemm")
    return out


def _gemm_params(A4, B4, C4, M, K, N, transB, alpha, beta, bias_mode, math_mode):
    p = GemmParams()
    p.M, p.K, p.N, p.transB, p.alpha, p.beta, p.bias_mode = M, K, N, transB, alpha, beta, bias_mode
    p.lda, p.ldb = A4.shape[-1], B4.shape[-1]
    p.ldc = C4.shape[-1] if (C4 is not None and bias_mode == 1) else 0
    p.ldy = up4(N)
    p.math_mode = math_mode
    return p


def gemm_pack_b(B4, M, K, N, transB=0, math_mode=MATH_TF32X3):
    """Packs a constant B once for the tensor-core modes; returns the opaque device blob."""
    _require_cuda(B4)
    p = _gemm_params(B4, B4, None, M, K, N, transB, 1.0, 1.0, 0, math_mode)
    p.lda = up4(K)
    lib = _lib.cuda_lib()
    nbytes = lib.ogle_cuda_gemm_packed_b_bytes(C.byref(p))
    packed = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    check(lib.ogle_cuda_gemm_pack_b(C.byref(p), _p(B4), _p(packed), _stream()), "gemm_pack_b")
    return packed


def gemm_packed(A4, packed_b, C4, M, K, N, transB=0, alpha=1.0, beta=1.0, bias_mode=0, math_mode=MATH_TF32X3):
    _require_cuda(A4, packed_b, C4)
    p = _gemm_params(A4, A4, C4, M, K, N, transB, alpha, beta, bias_mode, math_mode)
    p.ldb = 0
    out = torch.empty((M, up4(N)), dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_gemm_packed(C.byref(p), _p(A4), _p(packed_b), _p(C4), _p(out), _stream()), "gemm_packed")
    return out


def gemm_ws(A4, B4, C4, M, K, N, transB=0, alpha=1.0, beta=1.0, bias_mode=0, math_mode=MATH_TF32X3, workspace=None):
    """gemm with a run-time B: the caller lends the packing workspace."""
    _require_cuda(A4, B4, C4)
    p = _gemm_params(A4, B4, C4, M, K, N, transB, alpha, beta, bias_mode, math_mode)
    lib = _lib.cuda_lib()
    need = lib.ogle_cuda_gemm_packed_b_bytes(C.byref(p))
    if workspace is None:
        workspace = torch.empty(need // 4, dtype=torch.float32, device="cuda")
    out = torch.empty((M, up4(N)), dtype=torch.float32, device="cuda")
    check(lib.ogle_cuda_gemm_ws(C.byref(p), _p(A4), _p(B4), _p(C4), _p(out), _p(workspace), workspace.numel() * 4,
                                _stream()), "gemm_ws")
    return out


def gemm_static(A4, B4, C4, out, M, K, N, transB=0, alpha=1.0, beta=1.0, bias_mode=0, math_mode=MATH_TF32X3):
    """gemm with a run-time B, packing scratch inside the library; writes into the caller's `out`
    ([M, up4(N)] floats on the device). Neither this wrapper nor the call allocates."""
    _require_cuda(A4, B4, C4, out)
    p = _gemm_params(A4, B4, C4, M, K, N, transB, alpha, beta, bias_mode, math_mode)
    check(_lib.cuda_lib().ogle_cuda_gemm_static(C.byref(p), _p(A4), _p(B4), _p(C4), _p(out), _stream()), "gemm_static")
    return out


def concat(xs4, shapes, axis):
    """xs4: padded device tensors; shapes: their logical shapes (rank <= 4); axis in that rank."""
    rank = len(shapes[0])
    if axis < 0:
        axis += rank
    p = ConcatParams()
    p.n_inputs = len(xs4)
    p.axis = axis + 4 - rank
    out_shape = list(shapes[0])
    out_shape[axis] = sum(s[axis] for s in shapes)
    for i, s in enumerate(shapes):
        p.in_shapes[i][:] = [1] * (4 - rank) + list(s)
    out = torch.empty(out_shape[:-1] + [up4(out_shape[-1])], dtype=torch.float32, device="cuda")
    ptrs = (C.c_void_p * len(xs4))(*[x.data_ptr() for x in xs4])
    check(_lib.cuda_lib().ogle_cuda_concat(C.byref(p), ptrs, _p(out), _stream()), "concat")
    return out, out_shape


def transpose(x4, shape, perm):
    rank = len(shape)
    s4 = (C.c_int * 4)(*([1] * (4 - rank) + list(shape)))
    p4 = (C.c_int * 4)(*(list(range(4 - rank)) + [q + 4 - rank for q in perm]))
    out_shape = [shape[q] for q in perm]
    out = torch.empty(out_shape[:-1] + [up4(out_shape[-1])], dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_transpose(_p(x4), _p(out), s4, p4, _stream()), "transpose")
    return out, out_shape


def reshape(x4, in_shape, out_shape):
    n = int(np.prod(in_shape))
    out = torch.empty(list(out_shape[:-1]) + [up4(out_shape[-1])], dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_reshape(_p(x4), _p(out), n, in_shape[-1], out_shape[-1], _stream()), "reshape")
    return out


def nchw_to_nhwc4(x_nchw):
    _require_cuda(x_nchw)
    N, Cc, H, W = x_nchw.shape
    out = torch.empty((N, H, W, up4(Cc)), dtype=torch.float32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_nchw_to_nhwc4(_p(x_nchw), _p(out), N, Cc, H, W, _stream()), "nchw_to_nhwc4")
    return out


def preprocess_bgr8(image_u8, dst_h, dst_w, mean_rgb=(123.0, 117.0, 104.0), out=None):
    """image_u8: uint8 CUDA tensor [H, W, 3] (BGR) -> float32 [dst_h, dst_w, 4] RGB, resized, mean-subtracted."""
    if not image_u8.is_cuda or image_u8.dtype != torch.uint8 or not image_u8.is_contiguous():
        raise ValueError("expected a contiguous uint8 CUDA tensor")
    H, W, _ = image_u8.shape
    if out is None:
        out = torch.empty((dst_h, dst_w, 4), dtype=torch.float32, device="cuda")
    mean = (C.c_float * 3)(*mean_rgb)
    check(_lib.cuda_lib().ogle_cuda_preprocess_bgr8(C.c_void_p(image_u8.data_ptr()), H, W, W * 3, _p(out), dst_h, dst_w,
                                                    mean, _stream()), "preprocess_bgr8")
    return out


IMAGE_DESC = np.dtype([("offset", "<i8"), ("height", "<i4"), ("width", "<i4"), ("row_bytes", "<i4"), ("reserved", "<i4")])


def preprocess_bgr8_batch(images_u8, dst_h, dst_w, mean_rgb=(123.0, 117.0, 104.0)):
    """images_u8: list of uint8 numpy arrays [h_i, w_i, 3] (BGR) -> float32 CUDA [n, dst_h, dst_w, 4], one launch."""
    n = len(images_u8)
    table = np.zeros(n, dtype=IMAGE_DESC)
    total = 0
    for i, im in enumerate(images_u8):
        table[i] = (total, im.shape[0], im.shape[1], im.shape[1] * 3, 0)
        total += im.size
    packed = np.concatenate([np.ascontiguousarray(im).reshape(-1) for im in images_u8]) if n else np.zeros(1, np.uint8)
    buf = torch.from_numpy(packed).cuda()
    descs = torch.from_numpy(table.view(np.uint8)).cuda()
    out = torch.empty((n, dst_h, dst_w, 4), dtype=torch.float32, device="cuda")
    mean = (C.c_float * 3)(*mean_rgb)
    check(_lib.cuda_lib().ogle_cuda_preprocess_bgr8_batch(C.c_void_p(buf.data_ptr()), C.c_void_p(descs.data_ptr()), n,
                                                          _p(out), dst_h, dst_w, mean, _stream()), "preprocess_bgr8_batch")
    return out


def ssd_decode(pred, anchors, variances=(0.1, 0.1, 0.2, 0.2)):
    """pred [N,A,4], anchors [A,4] device tensors -> [N,A,4] corner boxes."""
    _require_cuda(pred, anchors)
    N, A, _ = pred.shape
    out = torch.empty_like(pred)
    v = (C.c_float * 4)(*variances)
    check(_lib.cuda_lib().ogle_cuda_ssd_decode(_p(pred), _p(anchors), _p(out), N, A, v, _stream()), "ssd_decode")
    return out


def ssd_detect(logits, boxes, num_classes, mode, score_thr, top_k, nms_thr=0.0, image_w=1, image_h=1):
    """logits [N,A,stride>=C], boxes [N,A,4]. Returns (score, anchor, cls, box, count) device tensors."""
    _require_cuda(logits, boxes)
    N, A, ls = logits.shape
    p = DetectParams()
    p.N, p.A, p.C, p.logit_stride, p.mode = N, A, num_classes, ls, mode
    p.score_thr, p.top_k, p.nms_thr, p.image_w, p.image_h = score_thr, top_k, nms_thr, image_w, image_h
    rows = top_k if mode == 0 else (num_classes - 1) * top_k
    score = torch.empty((N, rows), dtype=torch.float32, device="cuda")
    anchor = torch.empty((N, rows), dtype=torch.int32, device="cuda")
    cls = torch.empty((N, rows), dtype=torch.int32, device="cuda")
    box = torch.empty((N, rows, 4), dtype=torch.float32, device="cuda")
    count = torch.empty((N,) if mode == 0 else (N, num_classes - 1), dtype=torch.int32, device="cuda")
    check(_lib.cuda_lib().ogle_cuda_ssd_detect(C.byref(p), _p(logits), _p(boxes), _p(score),
                                               C.c_void_p(anchor.data_ptr()), C.c_void_p(cls.data_ptr()),
                                               _p(box), C.c_void_p(count.data_ptr()), _stream()), "ssd_detect")
    return score, anchor, cls, box, count


def launch_count():
    return int(_lib.cuda_lib().ogle_cuda_launch_count())
