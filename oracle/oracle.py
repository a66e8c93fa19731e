"""Test infrastructure only: numpy front end to the CPU oracle libraries.

`load("port")` opens oracle/liboracle.so (the restatement); `load("reference")`
opens oracle/_ref/libogle_ref.so (the reference's own shader and functor source
compiled for the CPU). Both export the interface declared in oracle/oracle.h.
Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; nothing in the ogle_b200 package does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATHS = {
    "port": os.path.join(_HERE, "liboracle.so"),
    "reference": os.path.join(_HERE, "_ref", "libogle_ref.so"),
}

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def _f(a):
    return a.ctypes.data_as(_fp)


def _i(a):
    return a.ctypes.data_as(_ip)


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def build(kind="port"):
    """Compile the library with oracle/Makefile (gcc only; no GPU needed)."""
    target = "all" if kind == "port" else "ref"
    subprocess.run(["make", "-s", "-C", _HERE, target], check=True)


def available(kind):
    return os.path.exists(_PATHS[kind])


class Oracle:
    def __init__(self, kind):
        self.kind = kind
        self.lib = C.CDLL(_PATHS[kind])
        L = self.lib
        L.ogle_oracle_threads.restype = C.c_int
        L.ogle_oracle_conv2d.argtypes = [_fp, _fp, _fp, _fp] + [C.c_int] * 11 + [C.c_float, C.c_float]
        L.ogle_oracle_pool.argtypes = [_fp, _fp] + [C.c_int] * 8
        L.ogle_oracle_batchnorm.argtypes = [_fp] * 6 + [C.c_int] * 4 + [C.c_float]
        L.ogle_oracle_relu.argtypes = [_fp, _fp, C.c_long]
        L.ogle_oracle_clip.argtypes = [_fp, _fp, C.c_long, C.c_float, C.c_float]
        L.ogle_oracle_add.argtypes = [_fp, _fp, _fp, C.c_long]
        L.ogle_oracle_gemm.argtypes = [_fp] * 4 + [C.c_int] * 4 + [C.c_float, C.c_float, C.c_int]
        L.ogle_oracle_concat.argtypes = [C.c_int, C.POINTER(_fp), _ip, C.c_int, _fp]
        L.ogle_oracle_transpose.argtypes = [_fp, _ip, _ip, _fp]
        L.ogle_oracle_decode.argtypes = [_fp, _fp, _fp, C.c_int, C.c_int, _fp]
        L.ogle_oracle_pad4.argtypes = [_fp, _fp, C.c_long, C.c_int]
        L.ogle_oracle_unpad4.argtypes = [_fp, _fp, C.c_long, C.c_int]
        L.ogle_oracle_prepack_filter.argtypes = [_fp, _fp] + [C.c_int] * 4
        L.ogle_oracle_unpack_filter.argtypes = [_fp, _fp] + [C.c_int] * 4
        L.ogle_oracle_detect.argtypes = [_fp, _fp] + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_float, _ip, _fp, _ip, _ip]
        L.ogle_oracle_topk_per_class.argtypes = [_fp, C.c_int, C.c_int, C.c_float, C.c_int, _fp, _ip, _ip]
        L.ogle_oracle_preprocess_bgr8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _fp, C.c_int, C.c_int, _fp]
        if kind == "reference":
            # the reference's own examples/ssd/detector.cc + common.cc (oracle/ref_detector.cc)
            L.ogle_ref_detect.argtypes = [_fp, _fp] + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_float, _ip, _fp, _ip]
            L.ogle_ref_softmax.argtypes = [_fp, _fp, C.c_int]

    def threads(self):
        return self.lib.ogle_oracle_threads()

    def set_threads(self, n):
        self.lib.ogle_oracle_set_threads(int(n))

    @staticmethod
    def _check(rc, what):
        if rc < 0:
            raise ValueError(f"oracle {what} rejected the request (code {rc})")

    def conv2d(self, x, w, bias=None, stride=1, pad=0, dilation=1, group=1, act=0, lo=0.0, hi=0.0):
        """x NHWC, w OIHW, bias [K] or None -> y NHWC."""
        x, w = _c(x), _c(w)
        N, H, W, Cin = x.shape
        K, _, k, _ = w.shape
        eff = k * dilation - dilation + 1
        Ho = (H - eff + 2 * pad) // stride + 1
        Wo = (W - eff + 2 * pad) // stride + 1
        y = np.empty((N, Ho, Wo, K), np.float32)
        b = _c(bias) if bias is not None else None
        rc = self.lib.ogle_oracle_conv2d(_f(x), _f(w), _f(b) if b is not None else None, _f(y),
                                         N, H, W, Cin, K, k, stride, pad, dilation, group, act, lo, hi)
        self._check(rc, "conv2d")
        return y

    def pool(self, x, kernel, stride, pad, type_):
        x = _c(x)
        N, H, W, Cc = x.shape
        Ho = (H - kernel + 2 * pad) // stride + 1
        Wo = (W - kernel + 2 * pad) // stride + 1
        y = np.empty((N, Ho, Wo, Cc), np.float32)
        self._check(self.lib.ogle_oracle_pool(_f(x), _f(y), N, H, W, Cc, kernel, stride, pad, type_), "pool")
        return y

    def batchnorm(self, x, gamma, beta, mean, var, eps):
        x = _c(x)
        N, H, W, Cc = x.shape
        y = np.empty_like(x)
        self._check(self.lib.ogle_oracle_batchnorm(_f(x), _f(_c(gamma)), _f(_c(beta)), _f(_c(mean)), _f(_c(var)),
                                                   _f(y), N, H, W, Cc, eps), "batchnorm")
        return y

    def relu(self, x):
        x = _c(x)
        y = np.empty_like(x)
        self.lib.ogle_oracle_relu(_f(x), _f(y), x.size)
        return y

    def clip(self, x, lo, hi):
        x = _c(x)
        y = np.empty_like(x)
        self.lib.ogle_oracle_clip(_f(x), _f(y), x.size, lo, hi)
        return y

    def add(self, a, b):
        a, b = _c(a), _c(b)
        y = np.empty_like(a)
        self.lib.ogle_oracle_add(_f(a), _f(b), _f(y), a.size)
        return y

    def gemm(self, A, B, Cm=None, transB=0, alpha=1.0, beta=1.0):
        A, B = _c(A), _c(B)
        M, K = A.shape
        N = B.shape[0] if transB else B.shape[1]
        mode = 0
        cm = None
        if Cm is not None:
            cm = _c(Cm)
            mode = 1 if cm.ndim == 2 else 2
        Y = np.empty((M, N), np.float32)
        rc = self.lib.ogle_oracle_gemm(_f(A), _f(B), _f(cm) if cm is not None else None, _f(Y),
                                       M, K, N, transB, alpha, beta, mode)
        self._check(rc, "gemm")
        return Y

    def concat(self, xs, axis):
        """xs: arrays of equal rank <= 4; axis in that rank (may be negative)."""
        xs = [_c(x) for x in xs]
        rank = xs[0].ndim
        if axis < 0:
            axis += rank
        shapes4 = np.array([[1] * (4 - rank) + list(x.shape) for x in xs], np.int32)
        ax4 = axis + 4 - rank
        out_shape = list(xs[0].shape)
        out_shape[axis] = sum(x.shape[axis] for x in xs)
        y = np.empty(out_shape, np.float32)
        ptrs = (_fp * len(xs))(*[_f(x) for x in xs])
        self._check(self.lib.ogle_oracle_concat(len(xs), ptrs, _i(shapes4), ax4, _f(y)), "concat")
        return y

    def transpose(self, x, perm):
        x = _c(x)
        rank = x.ndim
        s4 = np.array([1] * (4 - rank) + list(x.shape), np.int32)
        p4 = np.array(list(range(4 - rank)) + [p + 4 - rank for p in perm], np.int32)
        y = np.empty([x.shape[p] for p in perm], np.float32)
        self._check(self.lib.ogle_oracle_transpose(_f(x), _i(s4), _i(p4), _f(y)), "transpose")
        return y

    def decode(self, pred, anchors, variances=(0.1, 0.1, 0.2, 0.2)):
        pred, anchors = _c(pred), _c(anchors)
        N, A, _ = pred.shape
        out = np.empty_like(pred)
        v = np.array(variances, np.float32)
        self._check(self.lib.ogle_oracle_decode(_f(pred), _f(anchors), _f(out), N, A, _f(v)), "decode")
        return out

    def pad4(self, x):
        x = _c(x)
        last = x.shape[-1]
        rows = x.size // last
        y = np.empty(x.shape[:-1] + ((last + 3) // 4 * 4,), np.float32)
        self.lib.ogle_oracle_pad4(_f(x), _f(y), rows, last)
        return y

    def unpad4(self, x4, last):
        x4 = _c(x4)
        rows = x4.size // x4.shape[-1]
        y = np.empty(x4.shape[:-1] + (last,), np.float32)
        self.lib.ogle_oracle_unpad4(_f(x4), _f(y), rows, last)
        return y

    def prepack_filter(self, w):
        w = _c(w)
        O, I, kh, kw = w.shape
        p = np.empty((kh * kw * ((O + 3) // 4), (I + 3) // 4 * 4, 4), np.float32)
        self.lib.ogle_oracle_prepack_filter(_f(w), _f(p), O, I, kh, kw)
        return p

    def unpack_filter(self, p, O, I, kh, kw):
        p = _c(p)
        w = np.empty((O, I, kh, kw), np.float32)
        self.lib.ogle_oracle_unpack_filter(_f(p), _f(w), O, I, kh, kw)
        return w

    def detect(self, boxes, logits, image_w, image_h, score_thr=0.3, top_k=100, nms_thr=0.45):
        """One image. Returns dict of rect [n,4] int, score [n], cls [n], anchor [n]."""
        boxes, logits = _c(boxes), _c(logits)
        A, Cc = logits.shape
        rect = np.zeros((top_k, 4), np.int32)
        score = np.zeros(top_k, np.float32)
        cls = np.zeros(top_k, np.int32)
        anchor = np.zeros(top_k, np.int32)
        n = self.lib.ogle_oracle_detect(_f(boxes), _f(logits), A, Cc, image_w, image_h, score_thr, top_k, nms_thr,
                                        _i(rect), _f(score), _i(cls), _i(anchor))
        self._check(n, "detect")
        return {"rect": rect[:n], "score": score[:n], "cls": cls[:n], "anchor": anchor[:n]}

    def ref_detect(self, boxes, logits, image_w, image_h, score_thr=0.3, top_k=100, nms_thr=0.45):
        """kind "reference" only: Detector::GenerateBoxInfo -> GetTopK -> NMS as the reference compiled them.
        Returns dict of rect [n,4] int, score [n], cls [n] (the reference records no anchor index)."""
        boxes, logits = _c(boxes), _c(logits)
        A, Cc = logits.shape
        rect = np.zeros((max(top_k, 1), 4), np.int32)
        score = np.zeros(max(top_k, 1), np.float32)
        cls = np.zeros(max(top_k, 1), np.int32)
        n = self.lib.ogle_ref_detect(_f(boxes), _f(logits), A, Cc, image_w, image_h, score_thr, top_k, nms_thr,
                                     _i(rect), _f(score), _i(cls))
        self._check(n, "ref_detect")
        return {"rect": rect[:n], "score": score[:n], "cls": cls[:n]}

    def ref_softmax(self, row):
        """kind "reference" only: softmax of examples/ssd/common.cc:86-97 on one row."""
        row = _c(row).reshape(-1)
        out = np.empty_like(row)
        self.lib.ogle_ref_softmax(_f(row), _f(out), row.size)
        return out

    def preprocess_bgr8(self, image_bgr, dst_h, dst_w, mean_rgb=(123.0, 117.0, 104.0)):
        """image_bgr: uint8 [H, W, 3] -> float32 [dst_h, dst_w, 3] RGB, resized, mean-subtracted."""
        img = np.ascontiguousarray(image_bgr, dtype=np.uint8)
        H, W, _ = img.shape
        out = np.empty((dst_h, dst_w, 3), np.float32)
        mean = np.asarray(mean_rgb, np.float32)
        self._check(self.lib.ogle_oracle_preprocess_bgr8(img.ctypes.data, H, W, W * 3, _f(out), dst_h, dst_w, _f(mean)),
                    "preprocess_bgr8")
        return out

    def topk_per_class(self, logits, score_thr=0.01, top_k=200):
        """One image, logits [A,C]. Returns score [C-1,top_k], anchor [C-1,top_k], count [C-1]."""
        logits = _c(logits)
        A, Cc = logits.shape
        score = np.zeros((Cc - 1, top_k), np.float32)
        anchor = np.zeros((Cc - 1, top_k), np.int32)
        count = np.zeros(Cc - 1, np.int32)
        self._check(self.lib.ogle_oracle_topk_per_class(_f(logits), A, Cc, score_thr, top_k,
                                                        _f(score), _i(anchor), _i(count)), "topk_per_class")
        return score, anchor, count


_cache = {}


def load(kind="port"):
    if kind not in _cache:
        if not available(kind):
            build(kind)
        if not available(kind):
            raise FileNotFoundError(_PATHS[kind])
        _cache[kind] = Oracle(kind)
    return _cache[kind]
