"""GPU parity of every operator behind include/ogle_cuda.h against the oracle.

Tolerances (fp32 CUDA-core mode, OGLE_MATH_FP32):
  - data movement (pad, concat, transpose, reshape, pool max, relu, clip, add): bit-exact;
  - batchnorm: bit-exact (IEEE divide/sqrt, no contraction);
  - conv / gemm / average pool: |diff| <= 1e-5 + 1e-5*|ref| on the reference's
    own test shapes (its tests use 1e-5 absolute), the kernels differ from the
    oracle only in summation order and fused multiply-add;
  - decode: 1e-5 absolute (the reference's own decoder test tolerance).
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
sys.path.insert(0, os.path.dirname(__file__))
import cases  # noqa: E402
from ctypes import byref as C_byref  # noqa: E402

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))
EXACT = {"pool_max_3s2p1", "pool_max_2s2", "batchnorm", "relu", "clip", "add", "concat_channels", "concat_rows",
         "transpose_nchw_to_nhwc", "transpose_swap", "pad4"}


def close(a, b, atol=1e-5, rtol=1e-5):
    assert a.shape == b.shape
    err = np.abs(a - b) - (atol + rtol * np.abs(b))
    assert err.max() <= 0, f"max abs diff {np.abs(a - b).max():.3e}"


@pytest.mark.parametrize("name", sorted(n for n in cases.CASES if n != "prepack_filter"))
def test_cuda_matches_committed_reference_outputs(name):
    from gpu_ops import run_case_cuda
    got = run_case_cuda(cases.CASES[name]())
    if name in EXACT:
        assert np.array_equal(got, GOLDEN[name])
    else:
        close(got, GOLDEN[name])


def test_conv_reference_shape_sweep(oracle_port):
    """conv2d_test.cc:206-354: sizes 1..256 (powers of two) x channels 1..20, 3x3 pad 1,
    uniform [0,1) inputs; general, depthwise (K = C and K = 2C -> grouped) and dilated."""
    from gpu_ops import run_case_cuda
    rng = np.random.default_rng(11)
    for size in (1, 2, 4, 8, 16, 32, 64):
        for ch in (1, 2, 3, 4, 5, 8, 13, 20):
            x = rng.random((1, size, size, ch), dtype=np.float32)
            w = rng.random((ch + 3, ch, 3, 3), dtype=np.float32)
            b = rng.random(ch + 3, dtype=np.float32)
            case = dict(op="conv2d", x=x, w=w, bias=b, stride=1, pad=1, dilation=1, group=1, act=0, lo=0.0, hi=0.0)
            close(run_case_cuda(case), oracle_port.conv2d(x, w, b, 1, 1), atol=2e-5)
            wd = rng.random((ch, 1, 3, 3), dtype=np.float32)
            case = dict(op="conv2d", x=x, w=wd, bias=None, stride=1, pad=1, dilation=1, group=ch, act=0, lo=0.0, hi=0.0)
            close(run_case_cuda(case), oracle_port.conv2d(x, wd, None, 1, 1, 1, ch))
            if ch > 1:
                wg = rng.random((2 * ch, 1, 3, 3), dtype=np.float32)
                case = dict(op="conv2d", x=x, w=wg, bias=None, stride=1, pad=1, dilation=1, group=ch, act=0, lo=0.0, hi=0.0)
                close(run_case_cuda(case), oracle_port.conv2d(x, wg, None, 1, 1, 1, ch))
    x = rng.random((2, 33, 31, 6), dtype=np.float32)
    w = rng.random((9, 6, 3, 3), dtype=np.float32)
    case = dict(op="conv2d", x=x, w=w, bias=None, stride=2, pad=2, dilation=2, group=1, act=0, lo=0.0, hi=0.0)
    close(run_case_cuda(case), oracle_port.conv2d(x, w, None, 2, 2, 2), atol=2e-5)


def test_conv_mobilenet_layer_shapes(oracle_port):
    """Layer shapes of the MobileNet-v1-SSD graph at batch 2 (N(0,1) activations,
    N(0,0.05) weights): north-star tolerance max-abs 1e-3 / rel 1e-3, and the
    stricter 1e-4 that fp32 FMA actually reaches."""
    from gpu_ops import run_case_cuda
    rng = np.random.default_rng(12)
    shapes = [  # H, C, K, k, s, p, group
        (38, 256, 256, 3, 1, 1, 1), (19, 512, 1024, 1, 1, 0, 1), (38, 512, 512, 3, 2, 1, 512),
        (19, 512, 126, 3, 1, 1, 1), (10, 1024, 24, 3, 1, 1, 1), (10, 256, 512, 3, 2, 1, 1), (75, 64, 128, 1, 1, 0, 1),
        (3, 256, 126, 3, 1, 1, 1), (1, 128, 24, 3, 1, 1, 1),
    ]
    for H, C, K, k, s, p, g in shapes:
        x = rng.standard_normal((2, H, H, C), dtype=np.float32)
        w = rng.standard_normal((K, C // g, k, k), dtype=np.float32) * np.float32(0.05)
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        case = dict(op="conv2d", x=x, w=w, bias=b, stride=s, pad=p, dilation=1, group=g, act=2, lo=0.0, hi=0.0)
        got, ref = run_case_cuda(case), oracle_port.conv2d(x, w, b, s, p, 1, g, 2)
        close(got, ref, atol=1e-4, rtol=1e-4)


TC_SHAPES = [  # N, H, C, K, k, s, p, act
    (2, 38, 256, 256, 3, 1, 1, 2), (2, 19, 512, 1024, 1, 1, 0, 2), (2, 19, 512, 126, 3, 1, 1, 0),
    (2, 10, 1024, 24, 3, 1, 1, 0), (2, 10, 256, 512, 3, 2, 1, 2), (3, 75, 64, 128, 1, 1, 0, 1),
    (2, 3, 256, 126, 3, 1, 1, 0), (5, 1, 128, 24, 3, 1, 1, 0), (2, 19, 512, 63, 3, 1, 1, 0),
    (2, 19, 512, 12, 3, 1, 1, 0), (1, 150, 32, 64, 1, 1, 0, 1), (2, 20, 40, 300, 1, 1, 0, 2),
    (2, 17, 24, 70, 5, 2, 2, 2),
]


def test_conv_tensor_core_modes(oracle_port):
    """The tcgen05 path per layer shape, outputs of magnitude ~1-4. 3xTF32 (hi/lo operand split):
    the tensor core truncates its fp32 accumulator at every step instead of rounding, so the
    error grows with the reduction length (up to 9216 here); bound 3e-4 absolute, inside the 1e-3
    target. One-pass TF32 (10-bit operands) is held to 2e-3 of the output's largest magnitude."""
    from gpu_ops import run_case_cuda
    from ogle_b200 import _lib, ops
    rng = np.random.default_rng(31)
    for N, H, C, K, k, s, p, act in TC_SHAPES:
        x = rng.standard_normal((N, H, H, C), dtype=np.float32)
        w = rng.standard_normal((K, C, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(C * k * k))
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        case = dict(op="conv2d", x=x, w=w, bias=b, stride=s, pad=p, dilation=1, group=1, act=act, lo=0.0, hi=6.0)
        ref = oracle_port.conv2d(x, w, b, s, p, 1, 1, act, 0.0, 6.0)
        scale = np.abs(ref).max()
        got = run_case_cuda(case, ops.MATH_TF32X3)
        assert np.abs(got - ref).max() <= 3e-4, (N, H, C, K, k, float(np.abs(got - ref).max()))
        got = run_case_cuda(case, ops.MATH_TF32)
        assert np.abs(got - ref).max() / scale <= 2e-3, (N, H, C, K, k)
    assert _lib.cuda_lib().ogle_cuda_device_status() == 0


def test_conv_with_residual_operand_equals_the_separate_passes(oracle_port):
    """ogle_cuda_conv2d_residual: act(conv(x) + bias + residual) in the convolution's pass performs the same fp32
    operations in the same order as ogle_cuda_conv2d followed by ogle_cuda_add_act, so the two must agree bit for
    bit; also checked against the oracle's conv + add + relu. Pointwise and 3x3 (tiles of whole rows), a ragged
    last tile, a channel count that is no multiple of 4 (padded lanes stay zero), Relu and no activation."""
    import torch
    from ogle_b200 import _lib, ops
    rng = np.random.default_rng(91)
    shapes = [  # N, H, C, K, k, s, p, act
        (3, 19, 64, 64, 1, 1, 0, 2), (2, 28, 128, 128, 3, 1, 1, 2), (5, 7, 512, 510, 3, 1, 1, 0), (1, 56, 64, 64, 3, 1, 1, 2),
        (2, 14, 256, 30, 1, 1, 0, 2)]
    for N, H, Cc, K, k, st, pd, act in shapes:
        x = rng.standard_normal((N, H, H, Cc), dtype=np.float32)
        w = rng.standard_normal((K, Cc, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(Cc * k * k))
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        Ho = (H + 2 * pd - k) // st + 1
        res = rng.standard_normal((N, Ho, Ho, K), dtype=np.float32)
        ref = oracle_port.conv2d(x[:2], w, b, st, pd) + res[:2]
        if act == 2:
            ref = np.maximum(ref, 0.0)
        x4, b4, r4 = ops.upload(x), ops.dense_to_device(b), ops.upload(res)
        for mode in (ops.MATH_TF32X3, ops.MATH_TF32):
            p = ops.conv_params(N, H, H, Cc, K, k, st, pd, 1, 1, True, act, 0.0, 0.0, mode)
            p.split = 1
            packed = ops.conv2d_prepack(p, ops.dense_to_device(w))
            fused = ops.conv2d_residual(p, x4, packed, b4, r4)
            q = ops.conv_params(N, H, H, Cc, K, k, st, pd, 1, 1, True, 0, 0.0, 0.0, mode)
            q.split = 1
            plain = ops.conv2d(q, x4, packed, b4, workspace=None)
            two_pass = ops.add_act(plain, r4, act)
            assert torch.equal(fused, two_pass), (N, H, Cc, K, k, mode)
            got = ops.download(fused, K)[:2]
            tol = 3e-4 if mode == ops.MATH_TF32X3 else 2e-3 * np.abs(ref).max()
            assert np.abs(got - ref).max() <= tol, (N, H, Cc, K, mode, float(np.abs(got - ref).max()))
            if ops.up4(K) != K:
                assert float(fused[..., K:].abs().max()) == 0.0
    # a parameter set the tensor cores do not serve is refused, not silently computed another way
    p = ops.conv_params(1, 8, 8, 8, 8, 3, 1, 1, 1, 1, True, 0, 0.0, 0.0, ops.MATH_FP32)
    packed = ops.conv2d_prepack(p, torch.zeros((8, 8, 3, 3), device="cuda"))
    with pytest.raises(_lib.OgleError):
        ops.conv2d_residual(p, torch.zeros((1, 8, 8, 8), device="cuda"), packed, torch.zeros(8, device="cuda"),
                            torch.zeros((1, 8, 8, 8), device="cuda"))


def test_conv_with_channels_on_m_gives_the_same_bits(oracle_port):
    """Channels-on-M form of the tensor-core path (channels_on_m = 2, at most 128 output channels: the filter tile
    is the multiply's 128-row operand and two 128-pixel tiles its 256-column operand, the epilogue transposes):
    same products summed in the same order, so the output must equal the pixels-on-M form's bit for bit, and
    match the oracle. Shapes: an odd number of pixel tiles, a ragged last tile, 3x3 with tiles of whole rows from
    several images, 1x1, channel counts that are no multiple of 32 or of 4, 128 channels (the staging slabs are
    then shared in turns), Relu / Clip, with and without a residual operand, both tensor-core math modes."""
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    rng = np.random.default_rng(93)
    shapes = [  # N, H, C, K, k, s, p, act
        (3, 19, 64, 75, 3, 1, 1, 0), (2, 28, 128, 128, 3, 1, 1, 2), (5, 10, 96, 30, 3, 2, 1, 1), (4, 20, 64, 64, 1, 1, 0, 2),
        (7, 5, 256, 126, 3, 1, 1, 0), (1, 56, 64, 64, 3, 1, 1, 2)]
    for N, H, Cc, K, k, st, pd, act in shapes:
        x = rng.standard_normal((N, H, H, Cc), dtype=np.float32)
        w = rng.standard_normal((K, Cc, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(Cc * k * k))
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        Ho = (H + 2 * pd - k) // st + 1
        res = rng.standard_normal((N, Ho, Ho, K), dtype=np.float32)
        ref = oracle_port.conv2d(x[:2], w, b, st, pd, 1, 1, act, 0.0, 1.5)
        x4, b4, r4 = ops.upload(x), ops.dense_to_device(b), ops.upload(res)
        for mode in (ops.MATH_TF32X3, ops.MATH_TF32):
            outs, outs_res = [], []
            for on_m in (1, 2):
                p = ops.conv_params(N, H, H, Cc, K, k, st, pd, 1, 1, True, act, 0.0, 1.5, mode)
                p.split, p.sm_pair, p.channels_on_m = 1, 1, on_m
                packed = ops.conv2d_prepack(p, ops.dense_to_device(w))
                outs.append(ops.conv2d(p, x4, packed, b4, workspace=None))
                if act != 1:
                    outs_res.append(ops.conv2d_residual(p, x4, packed, b4, r4))
            assert torch.equal(outs[0], outs[1]), (N, H, Cc, K, k, mode)
            if outs_res:
                assert torch.equal(outs_res[0], outs_res[1]), (N, H, Cc, K, k, mode, "residual")
            got = ops.download(outs[1], K)[:2]
            tol = 3e-4 if mode == ops.MATH_TF32X3 else 2e-3 * np.abs(ref).max()
            assert np.abs(got - ref).max() <= tol, (N, H, Cc, K, mode, float(np.abs(got - ref).max()))
            if ops.up4(K) != K:
                assert float(outs[1][..., K:].abs().max()) == 0.0
    assert lib.ogle_cuda_device_status() == 0


def test_conv_on_sm_pairs_gives_the_same_bits(oracle_port):
    """Two-SM form of the tensor-core path (sm_pair = 2: a cluster of two blocks computes 256 pixels x n_tile
    channels, each block loading half of the filter tile): every output value sums its reduction in the same
    order as the one-SM form, so the tensors must be identical bit for bit, and both must match the oracle.
    Shapes: an odd number of 128-pixel tiles (the last pair has one empty half), a ragged last tile, a channel
    count that leaves the last filter tile partly empty, a 3x3 layer (tiles of whole rows), ReLU / Clip, a
    concat slice as destination, both tensor-core math modes."""
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    rng = np.random.default_rng(77)
    shapes = [  # N, H, C, K, k, s, p, act, n_tile
        (3, 19, 512, 600, 1, 1, 0, 0, 256), (4, 19, 256, 512, 1, 1, 0, 2, 256), (5, 10, 128, 128, 1, 1, 0, 1, 128),
        (2, 38, 64, 256, 3, 1, 1, 2, 256), (7, 10, 96, 75, 3, 2, 1, 0, 64), (1, 20, 64, 192, 1, 1, 0, 0, 192)]
    for N, H, Cc, K, k, st, pd, act, nt in shapes:
        x = rng.standard_normal((N, H, H, Cc), dtype=np.float32)
        w = rng.standard_normal((K, Cc, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(Cc * k * k))
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        ref = oracle_port.conv2d(x[:2], w, b, st, pd, 1, 1, act, 0.0, 1.5)
        x4, b4 = ops.upload(x), ops.dense_to_device(b)
        for mode in (ops.MATH_TF32X3, ops.MATH_TF32):
            outs = []
            for pair in (1, 2):
                p = ops.conv_params(N, H, H, Cc, K, k, st, pd, 1, 1, True, act, 0.0, 1.5, mode)
                p.n_tile, p.split, p.sm_pair = nt, 1, pair
                packed = ops.conv2d_prepack(p, ops.dense_to_device(w))
                outs.append(ops.conv2d(p, x4, packed, b4, workspace=None))
            assert torch.equal(outs[0], outs[1]), (N, H, Cc, K, k, mode)
            got = ops.download(outs[1], K)[:2]
            tol = 3e-4 if mode == ops.MATH_TF32X3 else 2e-3 * np.abs(ref).max()
            assert np.abs(got - ref).max() <= tol, (N, H, Cc, K, mode, float(np.abs(got - ref).max()))
            if ops.up4(K) != K:
                assert float(outs[1][..., K:].abs().max()) == 0.0
    # into a channel slice of a wider tensor (a concat written in place)
    N, H, Cc, K = 3, 19, 256, 128
    x = rng.standard_normal((N, H, H, Cc), dtype=np.float32)
    w = rng.standard_normal((K, Cc, 1, 1), dtype=np.float32) * np.float32(0.06)
    b = rng.standard_normal(K, dtype=np.float32)
    x4, b4 = ops.upload(x), ops.dense_to_device(b)
    wide = []
    for pair in (1, 2):
        p = ops.conv_params(N, H, H, Cc, K, 1, 1, 0, 1, 1, True, 0, 0.0, 0.0, ops.MATH_TF32X3)
        p.out_channel_stride, p.out_channel_offset = 320, 64
        p.n_tile, p.split, p.sm_pair = 128, 1, pair
        packed = ops.conv2d_prepack(p, ops.dense_to_device(w))
        out = torch.full((N, H, H, 320), -7.0, device="cuda")
        ops.conv2d(p, x4, packed, b4, out, workspace=None)
        wide.append(out)
    assert torch.equal(wide[0], wide[1])
    assert float((wide[1][..., :64] + 7.0).abs().max()) == 0.0 and float((wide[1][..., 192:] + 7.0).abs().max()) == 0.0
    ref = oracle_port.conv2d(x, w, b, 1, 0)
    assert np.abs(wide[1][..., 64:192].cpu().numpy() - ref).max() <= 3e-4
    assert lib.ogle_cuda_device_status() == 0


def test_conv_split_reduction_through_workspace(oracle_port):
    """Long reductions over few output tiles (3x3 heads on small maps, batch 1): with scratch memory lent
    (ogle_cuda_conv2d_ws) the reduction is split over several blocks per tile and a second kernel adds the slices in
    a fixed order, then bias and activation. Checked against the oracle, against the launch without scratch, and
    for run-to-run bit-reproducibility; ReLU and Clip layers split too."""
    import ctypes as C
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    rng = np.random.default_rng(56)
    shapes = [  # N, H, C, K, k, s, p, act
        (1, 10, 1024, 150, 3, 1, 1, 0), (2, 10, 256, 512, 3, 2, 1, 2), (1, 3, 256, 126, 3, 1, 1, 1), (3, 2, 2048, 64, 1, 1, 0, 2),
        (1, 19, 512, 75, 3, 1, 1, 0), (32, 10, 1024, 150, 3, 1, 1, 0)]
    for N, H, Cc, K, k, st, pd, act in shapes:
        x = rng.standard_normal((N, H, H, Cc), dtype=np.float32)
        w = rng.standard_normal((K, Cc, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(Cc * k * k))
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        ref = oracle_port.conv2d(x[:2], w, b, st, pd, 1, 1, act, 0.0, 1.5)
        for mode in (ops.MATH_TF32X3, ops.MATH_TF32):
            p = ops.conv_params(N, H, H, Cc, K, k, st, pd, 1, 1, True, act, 0.0, 1.5, mode)
            assert lib.ogle_cuda_conv2d_workspace_bytes(C.byref(p)) > 0, (N, H, Cc, K)
            packed = ops.conv2d_prepack(p, ops.dense_to_device(w))
            x4, b4 = ops.upload(x), ops.dense_to_device(b)
            y_ws = ops.conv2d(p, x4, packed, b4)
            y_ws2 = ops.conv2d(p, x4, packed, b4)
            y_plain = ops.conv2d(p, x4, packed, b4, workspace=None)
            assert torch.equal(y_ws, y_ws2)
            got = ops.download(y_ws, K)[:2]
            tol = 3e-4 if mode == ops.MATH_TF32X3 else 2e-3 * np.abs(ref).max()
            assert np.abs(got - ref).max() <= tol, (N, H, Cc, K, mode, float(np.abs(got - ref).max()))
            assert np.abs(ops.download(y_plain, K)[:2] - ref).max() <= tol
            if ops.up4(K) != K:
                assert float(y_ws[..., K:].abs().max()) == 0.0            # padded lanes stay zero
    # the two-output form (stacked heads): same values with and without scratch, to the order of the partial sums
    x = rng.standard_normal((2, 10, 10, 1024), dtype=np.float32)
    w1 = rng.standard_normal((24, 1024, 3, 3), dtype=np.float32) * np.float32(0.01)
    w2 = rng.standard_normal((126, 1024, 3, 3), dtype=np.float32) * np.float32(0.01)
    b1, b2 = rng.standard_normal(24, dtype=np.float32), rng.standard_normal(126, dtype=np.float32)
    args = (ops.upload(x), ops.dense_to_device(w1), ops.dense_to_device(b1), ops.dense_to_device(w2), ops.dense_to_device(b2),
            2, 10, 10, 1024, 3, 1, 1)
    y1, y2 = ops.conv2d_pair(*args)
    z1, z2 = ops.conv2d_pair(*args, use_workspace=False)
    for got, other, wgt, bias, K in ((y1, z1, w1, b1, 24), (y2, z2, w2, b2, 126)):
        ref = oracle_port.conv2d(x, wgt, bias, 1, 1)
        assert np.abs(ops.download(got, K) - ref).max() <= 3e-4
        assert np.abs(ops.download(other, K) - ref).max() <= 3e-4
    assert lib.ogle_cuda_device_status() == 0


def test_conv_small_channel_kernel_shapes(oracle_port):
    """3x3 convolutions over 1-4 input channels on the CUDA cores (the RGB stem kernel where its tile
    shapes fit, the implicit-GEMM kernel otherwise): strides 1 and 2, ragged widths and heights, 1-4 input
    channels, output channel counts that are not multiples of 8."""
    from gpu_ops import run_case_cuda
    from ogle_b200 import _lib, ops
    rng = np.random.default_rng(35)
    shapes = [(2, 300, 300, 3, 32, 2, 1, 2), (1, 97, 131, 3, 32, 2, 1, 1), (2, 64, 50, 4, 32, 2, 0, 0), (1, 33, 21, 1, 30, 2, 1, 2),
              (2, 40, 40, 3, 32, 1, 1, 2), (1, 75, 60, 3, 16, 2, 1, 0), (1, 50, 50, 4, 64, 1, 1, 1), (1, 19, 23, 2, 8, 1, 0, 2)]
    for (N, H, W, C, K, s_, p_, act) in shapes:
        prm = ops.conv_params(N, H, W, C, K, 3, s_, p_, 1, 1, True, act, 0.0, 6.0, ops.MATH_FP32)
        if K == 32:
            assert _lib.cuda_lib().ogle_cuda_conv2d_kernel_name(C_byref(prm)) == b"conv3x3_smallc_kernel", (H, W, C, K)
        x = rng.standard_normal((N, H, W, C), dtype=np.float32)
        w = rng.standard_normal((K, C, 3, 3), dtype=np.float32) * np.float32(0.3)
        b = rng.standard_normal(K, dtype=np.float32)
        case = dict(op="conv2d", x=x, w=w, bias=b, stride=s_, pad=p_, dilation=1, group=1, act=act, lo=0.0, hi=6.0)
        close(run_case_cuda(case), oracle_port.conv2d(x, w, b, s_, p_, 1, 1, act, 0.0, 6.0), atol=1e-5, rtol=1e-5)
    assert _lib.cuda_lib().ogle_cuda_device_status() == 0


@pytest.mark.skipif(os.environ.get("OGLE_TC_GATHER") != "1", reason="gather form is opt-in (OGLE_TC_GATHER=1)")
def test_conv_stem_gather_form(oracle_port):
    """3x3 convolutions over 1-3 input channels (the RGB stem) in the tensor-core modes: the operand
    is gathered from the input window inside the kernel. Same bounds as the other tensor-core
    layers; ragged sizes exercise tiles that hang over the right and bottom edges."""
    from gpu_ops import run_case_cuda
    from ogle_b200 import _lib, ops
    rng = np.random.default_rng(33)
    for (N, H, W, C, K, s, p, act) in [(2, 300, 300, 3, 32, 2, 1, 2), (2, 64, 64, 3, 16, 1, 1, 1), (1, 33, 47, 2, 8, 2, 1, 0),
                                       (2, 17, 29, 1, 5, 1, 1, 0), (1, 150, 150, 3, 64, 1, 0, 2), (3, 40, 40, 3, 100, 2, 0, 1)]:
        x = rng.standard_normal((N, H, W, C), dtype=np.float32)
        w = rng.standard_normal((K, C, 3, 3), dtype=np.float32) * np.float32(1.0 / np.sqrt(C * 9))
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        case = dict(op="conv2d", x=x, w=w, bias=b, stride=s, pad=p, dilation=1, group=1, act=act, lo=0.0, hi=6.0)
        ref = oracle_port.conv2d(x, w, b, s, p, 1, 1, act, 0.0, 6.0)
        scale = np.abs(ref).max()
        got = run_case_cuda(case, ops.MATH_TF32X3)
        assert got.shape == ref.shape
        assert np.abs(got - ref).max() <= 2e-5, (N, H, W, C, K, s, float(np.abs(got - ref).max()))
        got = run_case_cuda(case, ops.MATH_TF32)
        assert np.abs(got - ref).max() / scale <= 2e-3, (N, H, W, C, K, s)
    assert _lib.cuda_lib().ogle_cuda_device_status() == 0


def test_conv_large_filter_stem_gather_form(oracle_port):
    """5x5 and 7x7 convolutions over 1-4 input channels (a ResNet-style 7x7 stride-2 stem) in the
    tensor-core modes: the reduction (k*k*C values, several 32-wide chunks) is gathered from the
    input window inside the kernel. Ragged sizes exercise tiles that hang over the edges."""
    from gpu_ops import run_case_cuda
    from ogle_b200 import _lib, ops
    rng = np.random.default_rng(34)
    cases_ = [(2, 224, 224, 3, 64, 7, 2, 3, 2), (1, 64, 48, 4, 32, 5, 1, 2, 1), (2, 45, 61, 1, 10, 7, 1, 3, 0),
              (1, 70, 70, 2, 130, 5, 2, 0, 2), (3, 39, 39, 3, 24, 7, 2, 0, 0), (1, 128, 128, 4, 16, 7, 1, 3, 1)]
    for (N, H, W, C, K, k, s, p, act) in cases_:
        prm = ops.conv_params(N, H, W, C, K, k, s, p, 1, 1, True, act, 0.0, 6.0, ops.MATH_TF32X3)
        assert _lib.cuda_lib().ogle_cuda_conv2d_kernel_name(C_byref(prm)) == b"conv_tc2_kernel", (H, W, C, k)
        x = rng.standard_normal((N, H, W, C), dtype=np.float32)
        w = rng.standard_normal((K, C, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(C * k * k))
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        case = dict(op="conv2d", x=x, w=w, bias=b, stride=s, pad=p, dilation=1, group=1, act=act, lo=0.0, hi=6.0)
        ref = oracle_port.conv2d(x, w, b, s, p, 1, 1, act, 0.0, 6.0)
        scale = np.abs(ref).max()
        got = run_case_cuda(case, ops.MATH_TF32X3)
        assert got.shape == ref.shape
        assert np.abs(got - ref).max() <= 3e-5, (N, H, W, C, K, k, s, float(np.abs(got - ref).max()))
        got = run_case_cuda(case, ops.MATH_TF32)
        assert np.abs(got - ref).max() / scale <= 2e-3, (N, H, W, C, K, k, s)
    assert _lib.cuda_lib().ogle_cuda_device_status() == 0


def test_conv_stem_gather_form_in_its_own_process():
    """The library reads OGLE_TC_GATHER once per process, so the opt-in path is exercised by running
    the test above in a child interpreter with the switch on."""
    if os.environ.get("OGLE_TC_GATHER") == "1":
        pytest.skip("already running with the gather form on")
    import subprocess
    env = dict(os.environ, OGLE_TC_GATHER="1")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-m", "gpu", "-q", "-x",
                        "-k", "test_conv_stem_gather_form and not own_process"],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "1 passed" in r.stdout, r.stdout[-2000:] + r.stderr[-1000:]


def test_conv_pair_equals_two_convs(oracle_port):
    """Sibling convolutions (the SSD box and class heads of one feature map) in one pass. One-pass
    TF32 accumulates each output in the same order whatever the tile width, so it must be
    bit-identical to the single-output entry point (padded lanes included); the 3-pass mode may
    order its three partial sums differently and is held to 2e-5 and to the oracle."""
    import torch
    from ogle_b200 import _lib, ops
    rng = np.random.default_rng(32)
    for (N, H, C, K1, K2, k, pad) in [(2, 19, 512, 12, 63, 3, 1), (2, 10, 1024, 24, 126, 3, 1), (3, 5, 512, 24, 126, 3, 1),
                                      (4, 1, 128, 24, 126, 3, 1), (2, 19, 64, 33, 7, 1, 0), (2, 9, 96, 64, 64, 3, 1)]:
        x = rng.standard_normal((N, H, H, C), dtype=np.float32)
        w1 = rng.standard_normal((K1, C, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(C * k * k))
        w2 = rng.standard_normal((K2, C, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(C * k * k))
        b1 = rng.standard_normal(K1, dtype=np.float32)
        b2 = rng.standard_normal(K2, dtype=np.float32)
        x4 = ops.upload(x)
        d = ops.dense_to_device
        for mode in (ops.MATH_TF32X3, ops.MATH_TF32):
            y1, y2 = ops.conv2d_pair(x4, d(w1), d(b1), d(w2), d(b2), N, H, H, C, k, 1, pad, math_mode=mode)
            for (w, b, K, y) in ((w1, b1, K1, y1), (w2, b2, K2, y2)):
                p = ops.conv_params(N, H, H, C, K, k, 1, pad, math_mode=mode)
                want = ops.conv2d(p, x4, ops.conv2d_prepack(p, d(w)), d(b))
                # same products; where the reduction is split (into more ranges for the form with fewer tiles) the
                # partial sums are added in a different order
                assert float((y - want).abs().max()) <= 2e-5, (N, H, C, K1, K2, mode)
                assert torch.equal(y[..., K:], want[..., K:])
            if mode == ops.MATH_TF32X3:
                assert np.abs(ops.download(y2, K2) - oracle_port.conv2d(x, w2, b2, 1, pad)).max() <= 3e-4
    assert _lib.cuda_lib().ogle_cuda_device_status() == 0


def test_depthwise_tile_shapes(oracle_port):
    """Depthwise 3x3 over the map sizes of the SSD-300 backbone and some ragged ones: every tile
    shape of the TMA kernel (full-width tiles, maps cut into two or three equal parts, 32/16-column tiles with ragged
    edges, stride 1 and 2, with and without padding) and the register-tiled fallback."""
    from gpu_ops import run_case_cuda
    rng = np.random.default_rng(41)
    for (N, H, W, C, s, p) in [(2, 19, 19, 64, 1, 1), (2, 38, 38, 32, 2, 1), (3, 10, 10, 96, 1, 1), (2, 19, 19, 32, 2, 1),
                               (1, 150, 150, 32, 1, 1), (1, 150, 150, 64, 2, 1), (2, 33, 45, 32, 1, 1), (2, 70, 41, 64, 2, 1),
                               (2, 21, 12, 32, 1, 0), (2, 9, 8, 32, 1, 1), (1, 40, 40, 36, 1, 1), (2, 38, 38, 64, 1, 1),
                               (1, 17, 17, 32, 1, 1), (1, 48, 47, 32, 1, 1), (1, 75, 75, 32, 2, 1)]:
        x = rng.standard_normal((N, H, W, C), dtype=np.float32)
        w = rng.standard_normal((C, 1, 3, 3), dtype=np.float32) * np.float32(0.3)
        b = rng.standard_normal(C, dtype=np.float32)
        case = dict(op="conv2d", x=x, w=w, bias=b, stride=s, pad=p, dilation=1, group=C, act=2, lo=0.0, hi=6.0)
        close(run_case_cuda(case), oracle_port.conv2d(x, w, b, s, p, 1, C, 2, 0.0, 6.0), atol=1e-5, rtol=1e-5)


def test_conv_in_place_concat_offsets(oracle_port):
    """Two producers write their channels straight into one wider tensor (concat in place)."""
    import torch
    from ogle_b200 import ops
    rng = np.random.default_rng(13)
    x = rng.standard_normal((2, 7, 7, 8), dtype=np.float32)
    w1 = rng.standard_normal((8, 8, 1, 1), dtype=np.float32) * 0.3
    w2 = rng.standard_normal((12, 8, 3, 3), dtype=np.float32) * 0.3
    out = torch.zeros((2, 7, 7, 20), dtype=torch.float32, device="cuda")
    x4 = ops.upload(x)
    p1 = ops.conv_params(2, 7, 7, 8, 8, 1, has_bias=False, out_stride=20, out_offset=0)
    p2 = ops.conv_params(2, 7, 7, 8, 12, 3, pad=1, has_bias=False, out_stride=20, out_offset=8)
    ops.conv2d(p1, x4, ops.conv2d_prepack(p1, ops.dense_to_device(w1)), None, out)
    ops.conv2d(p2, x4, ops.conv2d_prepack(p2, ops.dense_to_device(w2)), None, out)
    ref = np.concatenate([oracle_port.conv2d(x, w1), oracle_port.conv2d(x, w2, None, 1, 1)], axis=-1)
    close(ops.download(out, 20), ref)


def test_gemm_reference_shapes(oracle_port):
    """gemm_test.cc:116-134: (10x1024)(1024x1000)+C[10x1000]; (1x2048)(1000x2048)^T + C[1000]."""
    from gpu_ops import run_case_cuda
    rng = np.random.default_rng(14)
    A, B, Cm = rng.random((10, 1024), dtype=np.float32), rng.random((1024, 1000), dtype=np.float32), rng.random((10, 1000), dtype=np.float32)
    got = run_case_cuda(dict(op="gemm", A=A, B=B, Cm=Cm, transB=0, alpha=1.0, beta=1.0))
    close(got, oracle_port.gemm(A, B, Cm), atol=1e-3, rtol=1e-5)   # sums of 1024 products ~ 256
    A, B, Cm = rng.random((1, 2048), dtype=np.float32), rng.random((1000, 2048), dtype=np.float32), rng.random(1000, dtype=np.float32)
    got = run_case_cuda(dict(op="gemm", A=A, B=B, Cm=Cm, transB=1, alpha=1.0, beta=1.0))
    close(got, oracle_port.gemm(A, B, Cm, 1), atol=1e-3, rtol=1e-5)
    # ONNX row-broadcast bias for M > 1 (ResNet classifier: [128,512]x[1000,512]^T + [1000])
    A, B, Cm = rng.standard_normal((128, 512), dtype=np.float32), rng.standard_normal((1000, 512), dtype=np.float32) * 0.05, rng.standard_normal(1000, dtype=np.float32)
    got = run_case_cuda(dict(op="gemm", A=A, B=B, Cm=Cm, transB=1, alpha=1.0, beta=1.0))
    close(got, oracle_port.gemm(A, B, Cm, 1), atol=1e-4, rtol=1e-4)


def test_gemm_tensor_core_packed_and_workspace(oracle_port):
    """Tensor-core gemm: constant B packed once, or a run-time B packed into a lent workspace.
    3xTF32 meets the fp32 bound; one-pass TF32 the looser 2e-3 (10-bit operands, normalised)."""
    from ogle_b200 import ops
    rng = np.random.default_rng(23)
    for (M, K, N, tb) in [(200, 512, 1000, 1), (130, 300, 70, 0), (4, 96, 33, 1), (512, 1024, 512, 0)]:
        A = rng.standard_normal((M, K), dtype=np.float32)
        B = (rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32) * 0.05).astype(np.float32)
        Cm = rng.standard_normal(N, dtype=np.float32)
        ref = oracle_port.gemm(A, B, Cm, tb, 0.5, 2.0)
        scale = np.abs(ref).max()
        A4, B4, C4 = ops.upload(A), ops.upload(B), ops.upload(Cm)
        for mode, bound in ((ops.MATH_TF32X3, 2e-5), (ops.MATH_TF32, 2e-3)):
            packed = ops.gemm_pack_b(B4, M, K, N, tb, mode)
            got = ops.download(ops.gemm_packed(A4, packed, C4, M, K, N, tb, 0.5, 2.0, 2, mode), N)
            assert np.abs(got - ref).max() / scale <= bound, (M, K, N, tb, mode)
            got = ops.download(ops.gemm_ws(A4, B4, C4, M, K, N, tb, 0.5, 2.0, 2, mode), N)
            assert np.abs(got - ref).max() / scale <= bound, (M, K, N, tb, mode)
    from ogle_b200 import _lib
    assert _lib.cuda_lib().ogle_cuda_device_status() == 0


def test_pool_shapes(oracle_port):
    from gpu_ops import run_case_cuda
    rng = np.random.default_rng(15)
    for (N, H, C, k, s, p, t) in [(2, 76, 64, 3, 2, 1, 0), (2, 76, 64, 3, 2, 0, 0), (2, 112, 16, 3, 2, 1, 0),
                                  (3, 7, 512, 7, 1, 0, 1), (2, 10, 24, 10, 1, 0, 1), (1, 9, 5, 3, 1, 1, 1),
                                  (1, 8, 6, 2, 2, 0, 1), (1, 5, 3, 5, 3, 2, 0)]:
        x = rng.standard_normal((N, H, H, C), dtype=np.float32)
        got = run_case_cuda(dict(op="pool", x=x, kernel=k, stride=s, pad=p, type_=t))
        ref = oracle_port.pool(x, k, s, p, t)
        if t == 0:
            assert np.array_equal(got, ref)
        else:
            close(got, ref)


def test_global_average_pool_type2(oracle_port):
    from ogle_b200 import ops
    rng = np.random.default_rng(16)
    x = rng.standard_normal((4, 7, 7, 10), dtype=np.float32)
    p = ops.pool_params(4, 7, 7, 10, 0, 0, 0, 2)
    close(ops.download(ops.pool(p, ops.upload(x)), 10), oracle_port.pool(x, 7, 1, 0, 1))


def test_concat_every_axis_and_ragged(oracle_port):
    """concat_test.cc:98-128: 1- to 4-D shapes with dims <= 10, every axis; plus slice
    boundaries that are not multiples of 4 (true concat)."""
    from gpu_ops import run_case_cuda
    rng = np.random.default_rng(17)
    for rank in (1, 2, 3, 4):
        for axis in range(rank):
            base = [int(v) for v in rng.integers(1, 11, size=rank)]
            xs = []
            for _ in range(3):
                s = list(base)
                s[axis] = int(rng.integers(1, 11))
                xs.append(rng.random(s, dtype=np.float32))
            got = run_case_cuda(dict(op="concat", xs=xs, axis=axis))
            assert np.array_equal(got, np.concatenate(xs, axis=axis))
    xs = [rng.random((32, 19, 19, 256), dtype=np.float32)[:2] for _ in range(4)]
    assert np.array_equal(run_case_cuda(dict(op="concat", xs=xs, axis=3)), np.concatenate(xs, axis=3))


def test_transpose_and_reshape(oracle_port):
    from ogle_b200 import ops
    rng = np.random.default_rng(18)
    x = rng.random((2, 6, 5, 7), dtype=np.float32)
    for perm in [(0, 2, 3, 1), (0, 3, 1, 2), (3, 2, 1, 0), (0, 1, 2, 3)]:
        y4, shape = ops.transpose(ops.upload(x), x.shape, perm)
        assert np.array_equal(ops.download(y4, shape[-1]), x.transpose(perm))
    # SSD head plumbing: [N,h,w,a*C] -> [N,h*w*a,C] with a*C and C padding to different multiples of 4
    x = rng.random((2, 3, 3, 6 * 21), dtype=np.float32)
    y4 = ops.reshape(ops.upload(x), x.shape, (2, 54, 21))
    assert np.array_equal(ops.download(y4, 21), x.reshape(2, 54, 21))
    x = rng.random((4, 100), dtype=np.float32)
    y4 = ops.reshape(ops.upload(x), x.shape, (4, 5, 5, 4))
    assert np.array_equal(ops.download(y4, 4), x.reshape(4, 5, 5, 4))


def test_layout_round_trip_reference_loop():
    """functor_test.cc / context_test.cc: batch 1-4 x size 1..256 x channels 1..20 round trip."""
    from ogle_b200 import ops
    rng = np.random.default_rng(19)
    for n in (1, 3):
        for size in (1, 2, 16, 64):
            for ch in (1, 3, 4, 7, 20):
                x = rng.random((n, size, size, ch), dtype=np.float32)
                x4 = ops.upload(x)
                assert x4.shape[-1] == (ch + 3) // 4 * 4
                host4 = x4.cpu().numpy()
                assert np.array_equal(host4[..., :ch], x) and not host4[..., ch:].any()
                assert np.array_equal(ops.download(x4, ch), x)
    import torch
    x = rng.random((2, 3, 5, 4), dtype=np.float32)  # NCHW
    y = ops.nchw_to_nhwc4(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(y[..., :3], x.transpose(0, 2, 3, 1)) and not y[..., 3:].any()


def test_add_with_activation_equals_two_passes():
    """Fused Add -> Relu / Clip against the separate kernels: bit-identical."""
    import torch
    from ogle_b200 import ops
    g = torch.Generator().manual_seed(53)
    for shape in [(2, 56, 56, 64), (1, 7, 7, 512), (3, 5, 9, 4)]:
        a = torch.randn(shape, generator=g).cuda()
        b = torch.randn(shape, generator=g).cuda()
        assert torch.equal(ops.add_act(a, b, ops.ACT_RELU), ops.relu(ops.add(a, b)))
        assert torch.equal(ops.add_act(a, b, ops.ACT_CLIP, -0.5, 1.25), ops.clip(ops.add(a, b), -0.5, 1.25))
        assert torch.equal(ops.add_act(a, b, ops.ACT_NONE), ops.add(a, b))


def test_preprocess_bgr8_bit_exact(oracle_port):
    """The device front end (BGR8 -> RGB, 8-bit bilinear resize, float, mean) against the CPU
    restatement: integer arithmetic, so bit-exact, for shrinking, enlarging and odd sizes."""
    import torch
    from ogle_b200 import ops
    rng = np.random.default_rng(51)
    for (H, W, dh, dw) in [(480, 640, 300, 300), (300, 300, 300, 300), (117, 93, 300, 300), (1080, 1920, 300, 300),
                           (33, 47, 64, 19), (2, 2, 7, 5), (1, 1, 4, 4)]:
        img = rng.integers(0, 256, (H, W, 3), dtype=np.uint8)
        got = ops.preprocess_bgr8(torch.from_numpy(img).cuda(), dh, dw).cpu().numpy()
        ref = oracle_port.preprocess_bgr8(img, dh, dw)
        assert np.array_equal(got[..., :3], ref), (H, W, dh, dw)
        assert np.all(got[..., 3] == 0.0)


def test_preprocess_bgr8_batch_bit_exact(oracle_port):
    """One launch over a batch of frames of different sizes (table of offsets and sizes in
    device memory) gives, image by image, what the CPU restatement gives."""
    from ogle_b200 import ops
    rng = np.random.default_rng(52)
    sizes = [(480, 640), (300, 300), (117, 93), (33, 47), (2, 2), (1, 1), (301, 299)]
    imgs = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (h, w) in sizes]
    got = ops.preprocess_bgr8_batch(imgs, 300, 300).cpu().numpy()
    assert got.shape == (len(imgs), 300, 300, 4)
    for i, img in enumerate(imgs):
        ref = oracle_port.preprocess_bgr8(img, 300, 300)
        assert np.array_equal(got[i, ..., :3], ref), sizes[i]
        assert np.all(got[i, ..., 3] == 0.0)
    assert ops.preprocess_bgr8_batch([], 8, 8).shape == (0, 8, 8, 4)      # empty batch: no launch


def test_decode_batch_broadcasts_anchors(oracle_port):
    from ogle_b200 import ops
    rng = np.random.default_rng(20)
    pred = rng.standard_normal((5, 1917, 4), dtype=np.float32) * 0.5
    anchors = np.abs(rng.standard_normal((1917, 4), dtype=np.float32)) * 0.3 + 0.01
    got = ops.ssd_decode(ops.dense_to_device(pred), ops.dense_to_device(anchors)).cpu().numpy()
    ref = oracle_port.decode(pred, anchors)
    assert np.abs(got - ref).max() <= 1e-5


def _check_per_class(oracle_port, logits, boxes, thr, k, stride):
    import torch
    from ogle_b200 import ops
    N, A, C = logits.shape
    lg = np.zeros((N, A, stride), np.float32)
    lg[..., :C] = logits
    score, anchor, cls, box, count = [t.cpu().numpy() for t in ops.ssd_detect(
        torch.from_numpy(lg).cuda(), ops.dense_to_device(boxes), C, 1, thr, k)]
    for n in range(N):
        s_ref, a_ref, c_ref = oracle_port.topk_per_class(logits[n], thr, k)
        assert np.array_equal(count[n], c_ref)
        got_s = score[n].reshape(C - 1, k)
        got_a = anchor[n].reshape(C - 1, k)
        # scores agree to fp32 rounding of exp/divide; indices are exact wherever the
        # oracle's neighbouring scores differ by more than that rounding
        assert np.abs(got_s - s_ref).max() <= 2e-6
        mism = got_a != a_ref
        if mism.any():
            for c, r in zip(*np.nonzero(mism)):
                near = np.abs(s_ref[c] - s_ref[c, r]) <= 4e-6
                assert near.sum() > 1, f"image {n} class {c + 1} rank {r}: index differs without a near tie"
        sel = got_a >= 0
        assert np.array_equal(box[n].reshape(C - 1, k, 4)[sel], boxes[n][got_a[sel]])
        assert np.array_equal(cls[n].reshape(C - 1, k)[sel], np.broadcast_to(np.arange(1, C)[:, None], (C - 1, k))[sel])


def test_detect_per_class_topk(oracle_port):
    """Standard-SSD selection: softmax, threshold 0.01, per-class top-200 over 1917 anchors."""
    rng = np.random.default_rng(21)
    logits = rng.standard_normal((3, 1917, 21), dtype=np.float32) * 2
    boxes = rng.random((3, 1917, 4), dtype=np.float32)
    _check_per_class(oracle_port, logits, boxes, 0.01, 200, 24)
    # few candidates (high threshold), ragged anchor count, exact ties on purpose
    logits = rng.standard_normal((2, 333, 5), dtype=np.float32)
    logits[0, 10:40] = logits[0, 9]
    _check_per_class(oracle_port, logits, rng.random((2, 333, 4), dtype=np.float32), 0.3, 16, 5)
    _check_per_class(oracle_port, logits, rng.random((2, 333, 4), dtype=np.float32), 0.999, 8, 8)  # nothing passes


def test_detect_reference_rule(oracle_port):
    """Detector rule (detector.cc:114-228): best foreground class, thr 0.3, top 100, NMS 0.45 on int rects."""
    import torch
    from ogle_b200 import ops
    rng = np.random.default_rng(22)
    N, A, C = 4, 1917, 21
    logits = rng.standard_normal((N, A, C), dtype=np.float32) * 3
    ctr = rng.random((N, A, 2), dtype=np.float32)
    half = rng.random((N, A, 2), dtype=np.float32) * 0.2 + 0.02
    boxes = np.concatenate([ctr - half, ctr + half], axis=-1).astype(np.float32)
    out = ops.ssd_detect(torch.from_numpy(logits).cuda(), ops.dense_to_device(boxes), C, 0, 0.3, 100, 0.45, 300, 300)
    score, anchor, cls, box, count = [t.cpu().numpy() for t in out]
    for n in range(N):
        ref = oracle_port.detect(boxes[n], logits[n], 300, 300, 0.3, 100, 0.45)
        k = len(ref["anchor"])
        assert count[n] == k
        assert np.array_equal(anchor[n, :k], ref["anchor"])
        assert np.array_equal(cls[n, :k], ref["cls"])
        assert np.array_equal(box[n, :k].astype(np.int32), ref["rect"])
        assert np.abs(score[n, :k] - ref["score"]).max() <= 2e-6
        assert (anchor[n, k:] == -1).all()


def test_reshape_placed_and_concat_with_slices_in_place():
    """The two halves of a row-axis concat written in place: the re-padding copy puts its rows at its image's
    slice of the wider tensor (ogle_cuda_reshape_placed), and the concat pass leaves a slice alone whose input
    pointer is null. Together they equal the plain reshape followed by the full concat, bit for bit."""
    import ctypes as C
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    rng = np.random.default_rng(54)
    N = 3
    a = rng.standard_normal((N, 5, 5, 63)).astype(np.float32)       # -> [N, 75, 21]
    b = rng.standard_normal((N, 2, 2, 126)).astype(np.float32)      # -> [N, 24, 21]
    a4, b4 = ops.upload(a), ops.upload(b)
    ra = ops.reshape(a4, a.shape, (N, 75, 21))
    rb = ops.reshape(b4, b.shape, (N, 24, 21))
    want, shape = ops.concat([ra, rb], [(N, 75, 21), (N, 24, 21)], 1)
    assert tuple(shape) == (N, 99, 21)
    out = torch.full((N, 99, 24), float("nan"), dtype=torch.float32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # slice a written in place (75 rows per image, image stride 99 * 24 floats); slice b through the concat pass
    rc = lib.ogle_cuda_reshape_placed(C.c_void_p(a4.data_ptr()), C.c_void_p(out.data_ptr()), a.size, 63, 21, 75, 99 * 24, stream)
    assert rc == 0
    p = ops.ConcatParams()
    p.n_inputs, p.axis = 2, 2
    for i, sh in enumerate([(1, N, 75, 21), (1, N, 24, 21)]):
        p.in_shapes[i][:] = list(sh)
    ptrs = (C.c_void_p * 2)(None, rb.data_ptr())
    assert lib.ogle_cuda_concat(C.byref(p), ptrs, C.c_void_p(out.data_ptr()), stream) == 0
    assert torch.equal(out, want)
    # every slice in place: nothing is launched
    before = ops.launch_count()
    ptrs = (C.c_void_p * 2)(None, None)
    assert lib.ogle_cuda_concat(C.byref(p), ptrs, C.c_void_p(out.data_ptr()), stream) == 0
    assert ops.launch_count() == before
    # a block stride too small for the rows it must hold is refused
    assert lib.ogle_cuda_reshape_placed(C.c_void_p(a4.data_ptr()), C.c_void_p(out.data_ptr()), a.size, 63, 21, 75, 74 * 24, stream) == -1


def test_bounded_waits_run_out_cleanly(oracle_port):
    """Failure detection without a fault: with the roles' wait limit set to zero polls, every wait inside the
    tensor-core kernel gives up at once. The launch must return (the block waits for its own operand copies,
    frees its tensor memory and retires), the status word must name the wait that gave up, and - after the limit
    is restored and the word cleared - the same convolutions must be served correctly by the next launches."""
    from gpu_ops import run_case_cuda
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    rng = np.random.default_rng(55)
    cases = []
    for (N, H, C, K, k, p) in [(2, 19, 64, 64, 1, 0),      # two reduction chunks: the ring never wraps
                               (2, 19, 256, 96, 3, 1),     # 72 chunks: the producers reach their own wait
                               (4, 38, 128, 256, 1, 0)]:   # several tiles per block
        x = rng.standard_normal((N, H, H, C), dtype=np.float32)
        w = rng.standard_normal((K, C, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(C * k * k))
        b = rng.standard_normal(K, dtype=np.float32)
        cases.append(dict(op="conv2d", x=x, w=w, bias=b, stride=1, pad=p, dilation=1, group=1, act=2, lo=0.0, hi=0.0))
    assert lib.ogle_cuda_device_status() == 0
    try:
        for case in cases:
            for mode in (ops.MATH_TF32, ops.MATH_TF32X3):
                assert lib.ogle_cuda_set_wait_limit(0) == 0
                run_case_cuda(case, mode)                           # returns: no hang, no fault
                assert lib.ogle_cuda_device_status() == -6          # OGLE_ERR_TIMEOUT
                assert 1 <= lib.ogle_cuda_device_status_detail() <= 7
                assert lib.ogle_cuda_clear_device_status() == 0
                lib.ogle_cuda_set_wait_limit(-1)
                got = run_case_cuda(case, mode)
                assert lib.ogle_cuda_device_status() == 0
                ref = oracle_port.conv2d(case["x"], case["w"], case["bias"], 1, case["pad"], 1, 1, 2)
                tol = 3e-4 if mode == ops.MATH_TF32X3 else 2e-3 * np.abs(ref).max()
                assert np.abs(got - ref).max() <= tol
    finally:
        lib.ogle_cuda_set_wait_limit(-1)
        lib.ogle_cuda_clear_device_status()


def test_bounded_waits_of_the_sm_pair_and_channels_on_m_forms(oracle_port):
    """The same drill for the other two forms of the tensor-core kernel: with zero polls allowed every role's wait
    gives up at once; the launch returns, the status word names a wait of that form (11-18: the SM-pair form,
    where the abort flag is raised in both blocks of the pair and the pair meets at a cluster barrier before
    either frees its tensor memory; 21-27: the channels-on-M form), and with the limit restored the same call
    gives the same bits as the one-SM pixels-on-M form."""
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    rng = np.random.default_rng(57)
    N, H, Cc, K, k, pd = 4, 19, 256, 128, 3, 1
    x = rng.standard_normal((N, H, H, Cc), dtype=np.float32)
    w = rng.standard_normal((K, Cc, k, k), dtype=np.float32) * np.float32(1.0 / np.sqrt(Cc * k * k))
    b = rng.standard_normal(K, dtype=np.float32)
    x4, b4, w4 = ops.upload(x), ops.dense_to_device(b), ops.dense_to_device(w)
    assert lib.ogle_cuda_device_status() == 0

    def params(mode, sm_pair, on_m):
        p = ops.conv_params(N, H, H, Cc, K, k, 1, pd, 1, 1, True, 2, 0.0, 0.0, mode)
        p.n_tile, p.split, p.sm_pair, p.channels_on_m = 128, 1, sm_pair, on_m
        return p

    try:
        for mode in (ops.MATH_TF32, ops.MATH_TF32X3):
            packed = ops.conv2d_prepack(params(mode, 1, 1), w4)
            want = ops.conv2d(params(mode, 1, 1), x4, packed, b4, workspace=None)
            for sm_pair, on_m, codes in ((2, 1, range(11, 19)), (1, 2, range(21, 28))):
                p = params(mode, sm_pair, on_m)
                assert lib.ogle_cuda_set_wait_limit(0) == 0
                ops.conv2d(p, x4, packed, b4, workspace=None)           # returns: no hang, no fault
                assert lib.ogle_cuda_device_status() == -6              # OGLE_ERR_TIMEOUT
                assert lib.ogle_cuda_device_status_detail() in codes
                assert lib.ogle_cuda_clear_device_status() == 0
                lib.ogle_cuda_set_wait_limit(-1)
                got = ops.conv2d(p, x4, packed, b4, workspace=None)
                assert lib.ogle_cuda_device_status() == 0
                assert torch.equal(got, want)
    finally:
        lib.ogle_cuda_set_wait_limit(-1)
        lib.ogle_cuda_clear_device_status()


def test_empty_and_error_paths():
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    x = torch.zeros(8, device="cuda")
    assert lib.ogle_cuda_relu(x.data_ptr() + 4, x.data_ptr(), 4, None) == -4   # misaligned
    p = ops.conv_params(1, 4, 4, 4, 4, 3, pad=1)
    assert lib.ogle_cuda_conv2d(p, None, None, None, None, None) == -1
    before = ops.launch_count()
    ops.relu(ops.upload(np.ones((1, 4), np.float32)))
    assert ops.launch_count() == before + 2
