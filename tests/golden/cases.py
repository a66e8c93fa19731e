"""Seeded case definitions shared by the golden-vector generator and the tests.

Each case names an oracle operation, its seeded inputs and its scalar
parameters. Inputs are regenerated from the seed wherever they are needed, so
the committed fixture file holds only the reference's OUTPUTS.
"""
import numpy as np


def _rng(seed):
    return np.random.default_rng(seed)


def _f(r, shape, scale=1.0):
    return (r.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def conv_case(seed, N, H, W, C, K, k, s, p, d, g, act, bias, lo=-0.5, hi=1.5):
    r = _rng(seed)
    x = _f(r, (N, H, W, C))
    w = _f(r, (K, C // g, k, k), 0.3)
    b = _f(r, (K,)) if bias else None
    return dict(op="conv2d", x=x, w=w, bias=b, stride=s, pad=p, dilation=d, group=g, act=act, lo=lo, hi=hi)


CASES = {
    # general 3x3 with bias + relu; odd sizes, C and K not multiples of 4
    "conv_general_relu": lambda: conv_case(101, 2, 9, 7, 5, 6, 3, 1, 1, 1, 1, 2, True),
    # pointwise with clip: lower bound is 0 whatever min says (conv2d_pw.glsl:85)
    "conv_pointwise_clip": lambda: conv_case(102, 1, 8, 8, 8, 12, 1, 1, 0, 1, 1, 1, True),
    "conv_depthwise_s2_relu": lambda: conv_case(103, 2, 9, 9, 6, 6, 3, 2, 1, 1, 6, 2, True),
    "conv_depthwise_s1": lambda: conv_case(104, 1, 6, 6, 8, 8, 3, 1, 1, 1, 8, 0, False),
    "conv_grouped": lambda: conv_case(105, 1, 7, 7, 4, 8, 3, 1, 1, 1, 2, 0, False),
    "conv_grouped_relu_min": lambda: conv_case(106, 1, 5, 5, 8, 4, 3, 1, 1, 1, 2, 2, True),
    "conv_dilated_s2_clip": lambda: conv_case(107, 1, 10, 10, 3, 7, 3, 2, 1, 2, 1, 1, True),
    # the stem shape of the reference's own conv test (320x320x3 -> 32, stride 2), cut down
    "conv_stem_s2": lambda: conv_case(108, 1, 32, 32, 3, 32, 3, 2, 1, 1, 1, 2, True),
    "conv_7x7_s2": lambda: conv_case(109, 1, 20, 20, 3, 8, 7, 2, 3, 1, 1, 2, True),
    "conv_1x1_s2": lambda: conv_case(110, 1, 9, 9, 8, 16, 1, 2, 0, 1, 1, 0, False),
    "pool_max_3s2p1": lambda: dict(op="pool", x=_f(_rng(201), (2, 9, 9, 5)), kernel=3, stride=2, pad=1, type_=0),
    "pool_avg_3s2p1": lambda: dict(op="pool", x=_f(_rng(202), (2, 9, 9, 5)), kernel=3, stride=2, pad=1, type_=1),
    "pool_max_2s2": lambda: dict(op="pool", x=_f(_rng(203), (1, 8, 8, 4)), kernel=2, stride=2, pad=0, type_=0),
    "pool_global": lambda: dict(op="pool", x=_f(_rng(204), (2, 7, 7, 6)), kernel=7, stride=1, pad=0, type_=1),
    "batchnorm": lambda: (lambda r: dict(op="batchnorm", x=_f(r, (2, 5, 5, 6)), gamma=_f(r, (6,)), beta=_f(r, (6,)),
                                         mean=_f(r, (6,)), var=np.abs(_f(r, (6,))), eps=1e-5))(_rng(301)),
    "relu": lambda: dict(op="relu", x=_f(_rng(302), (2, 3, 4, 8))),
    "clip": lambda: dict(op="clip", x=_f(_rng(303), (2, 3, 4, 8)), lo=-0.2, hi=0.3),
    "add": lambda: (lambda r: dict(op="add", a=_f(r, (2, 3, 4, 8)), b=_f(r, (2, 3, 4, 8))))(_rng(304)),
    # shapes of the reference's gemm tests (gemm_test.cc:116-134), reduced in K
    "gemm_full_bias": lambda: (lambda r: dict(op="gemm", A=_f(r, (10, 64)), B=_f(r, (64, 50)), Cm=_f(r, (10, 50)),
                                              transB=0, alpha=0.7, beta=1.3))(_rng(401)),
    "gemm_transb_row_bias": lambda: (lambda r: dict(op="gemm", A=_f(r, (1, 96)), B=_f(r, (30, 96)), Cm=_f(r, (30,)),
                                                    transB=1, alpha=1.0, beta=1.0))(_rng(402)),
    "concat_channels": lambda: (lambda r: dict(op="concat", xs=[_f(r, (2, 3, 4, c)) for c in (4, 8, 4)], axis=3))(_rng(501)),
    "concat_rows": lambda: (lambda r: dict(op="concat", xs=[_f(r, (2, h, 5)) for h in (1, 3, 2)], axis=1))(_rng(502)),
    "transpose_nchw_to_nhwc": lambda: dict(op="transpose", x=_f(_rng(601), (2, 3, 4, 5)), perm=(0, 2, 3, 1)),
    "transpose_swap": lambda: dict(op="transpose", x=_f(_rng(602), (2, 3, 4, 5)), perm=(1, 0, 3, 2)),
    # shape {1,100,4} of the reference's decoder test (functor_test.cc:298-334)
    "decode": lambda: (lambda r: dict(op="decode", pred=_f(r, (1, 100, 4), 0.5), anchors=np.abs(_f(r, (100, 4))) + 0.05))(_rng(701)),
    "prepack_filter": lambda: dict(op="prepack_filter", w=_f(_rng(801), (6, 5, 3, 3))),
    "pad4": lambda: dict(op="pad4", x=_f(_rng(802), (2, 3, 4, 5))),
}


def run_case(lib, case):
    """Runs one case on an oracle library (port or reference) and returns the output array."""
    c = dict(case)
    op = c.pop("op")
    if op == "concat":
        return lib.concat(c["xs"], c["axis"])
    return getattr(lib, op)(**c)
