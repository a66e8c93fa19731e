"""CPU tests of the oracle itself: the restatement (oracle/liboracle.so) against
(a) the committed outputs of the reference's own code (tests/golden/) and
(b) that code run live (oracle/_ref/libogle_ref.so), where it is built.
Bit-exact: both evaluate the shader expressions with one rounding per operation."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_port_matches_committed_reference_outputs(oracle_port, name):
    got = cases.run_case(oracle_port, cases.CASES[name]())
    assert got.shape == GOLDEN[name].shape
    assert np.array_equal(got, GOLDEN[name]), f"max diff {np.abs(got - GOLDEN[name]).max()}"


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_port_matches_live_reference(oracle_port, oracle_ref, name):
    case = cases.CASES[name]()
    assert np.array_equal(cases.run_case(oracle_port, case), cases.run_case(oracle_ref, case))


def test_reference_conv_sweep_bit_exact(oracle_port, oracle_ref):
    """The reference's own shape loop (kernel_test_utils.h:59-65: sizes 1..256 in
    powers of two, channels 1..20), thinned so it runs in seconds."""
    rng = np.random.default_rng(7)
    for size in (1, 2, 4, 8, 16, 32):
        for ch in (1, 3, 4, 7, 12, 20):
            x = rng.random((1, size, size, ch), dtype=np.float32)
            w = rng.random((ch + 1, ch, 3, 3), dtype=np.float32)
            a = oracle_port.conv2d(x, w, None, 1, 1)
            b = oracle_ref.conv2d(x, w, None, 1, 1)
            assert np.array_equal(a, b)
            wd = rng.random((ch, 1, 3, 3), dtype=np.float32)
            assert np.array_equal(oracle_port.conv2d(x, wd, None, 1, 1, 1, ch), oracle_ref.conv2d(x, wd, None, 1, 1, 1, ch))


def test_port_against_torch_conv(oracle_port):
    """Independent cross-check (not the oracle): torch's CPU conv agrees to fp32 rounding."""
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 11, 9, 6), dtype=np.float32)
    w = rng.standard_normal((10, 6, 3, 3), dtype=np.float32) * 0.2
    b = rng.standard_normal(10, dtype=np.float32)
    got = oracle_port.conv2d(x, w, b, 2, 1, 1, 1, 2)
    ref = F.relu(F.conv2d(torch.from_numpy(x).permute(0, 3, 1, 2), torch.from_numpy(w), torch.from_numpy(b), 2, 1))
    assert np.abs(got - ref.permute(0, 2, 3, 1).numpy()).max() < 1e-5


def test_gemm_row_bias_for_many_rows_is_outside_reference(oracle_ref):
    """gemm.glsl reads C at the output texel, so a [N] bias is defined only for M == 1."""
    A = np.ones((2, 4), np.float32)
    with pytest.raises(ValueError):
        oracle_ref.gemm(A, np.ones((4, 4), np.float32), np.ones(4, np.float32))


def test_detect_postprocess_small(oracle_port):
    """Hand-checkable case of the Detector rule: best foreground class, threshold, top-k, NMS."""
    logits = np.array([[0.0, 3.0, 0.0], [0.0, 0.0, 2.0], [5.0, 0.0, 0.0], [0.0, 2.9, 0.0]], np.float32)
    boxes = np.array([[0.1, 0.1, 0.5, 0.5], [0.6, 0.6, 0.9, 0.9], [0.0, 0.0, 1.0, 1.0], [0.1, 0.1, 0.5, 0.52]], np.float32)
    d = oracle_port.detect(boxes, logits, 100, 100, score_thr=0.3, top_k=10, nms_thr=0.45)
    # anchor 2 is background-dominated; anchor 3 overlaps anchor 0 and scores lower
    assert d["anchor"].tolist() == [0, 1]
    assert d["cls"].tolist() == [1, 2]
    assert d["rect"].tolist() == [[10, 10, 40, 40], [60, 60, 29, 29]] or d["rect"][0].tolist() == [10, 10, 40, 40]


def _detect_golden():
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_detect_golden as g
    return g, np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_detect_outputs.npz"))


def test_detect_matches_committed_reference_outputs(oracle_port):
    """The pin of the Detector rule: bit-exact (rectangles, scores, classes, order) against what the reference's
    own GenerateBoxInfo / GetTopK / NMS kept, committed in tests/golden/reference_detect_outputs.npz."""
    g, data = _detect_golden()
    for i, ((boxes, logits), (_, _, w, h, thr, k, nms, _)) in enumerate(zip(g.detect_cases(), g.CASES)):
        d = oracle_port.detect(boxes, logits, w, h, thr, k, nms)
        assert np.array_equal(d["rect"], data[f"rect{i}"]), g.CASES[i]
        assert np.array_equal(d["score"], data[f"score{i}"]), g.CASES[i]
        assert np.array_equal(d["cls"], data[f"cls{i}"]), g.CASES[i]
        # the anchor index (which the reference does not record) names the box each row came from
        scale = np.array([w, h, w, h], np.float32)
        px = boxes[d["anchor"]] * scale
        want = np.stack([px[:, 0], px[:, 1], px[:, 2] - px[:, 0], px[:, 3] - px[:, 1]], axis=1).astype(np.int32)
        assert np.array_equal(d["rect"], want)


def test_detect_matches_live_reference(oracle_port, oracle_ref):
    """The same pin against the compiled reference on fresh seeded inputs of many sizes. Exactly tied scores
    (saturated softmax) are ordered by std::sort in the reference and by anchor index here: such cases are
    compared as sets of candidates, all others row by row."""
    rng = np.random.default_rng(23)
    for t in range(40):
        A, C = int(rng.integers(5, 2500)), int(rng.integers(2, 30))
        logits = (rng.standard_normal((A, C)) * rng.choice([1, 3, 6])).astype(np.float32)
        ctr = rng.random((A, 2), dtype=np.float32)
        half = rng.random((A, 2), dtype=np.float32) * 0.2 + 0.02
        boxes = np.concatenate([ctr - half, ctr + half], -1).astype(np.float32)
        W, H = int(rng.integers(50, 2000)), int(rng.integers(50, 2000))
        thr, k, nms = float(rng.choice([0.3, 0.1, 0.6])), int(rng.choice([100, 10, 400])), float(rng.choice([0.45, 0.3, 0.7]))
        a, b = oracle_port.detect(boxes, logits, W, H, thr, k, nms), oracle_ref.ref_detect(boxes, logits, W, H, thr, k, nms)
        cand = oracle_port.detect(boxes, logits, W, H, thr, k, 1.0)["score"]
        if len(np.unique(cand)) == len(cand):
            for key in ("rect", "score", "cls"):
                assert np.array_equal(a[key], b[key]), (t, key)
        else:
            ca = oracle_port.detect(boxes, logits, W, H, thr, A, 1.0)
            cb = oracle_ref.ref_detect(boxes, logits, W, H, thr, A, 1.0)
            rows = lambda d: sorted(zip(d["score"].tolist(), d["cls"].tolist(), map(tuple, d["rect"].tolist())))
            assert rows(ca) == rows(cb), t


def test_softmax_matches_reference(oracle_port, oracle_ref):
    """Per-class top-k is an extension without a reference counterpart; the softmax it ranks by is the
    reference's (common.cc:86-97): with threshold 0 and k = anchors the scores of every class are that
    softmax, bit for bit, committed and live."""
    g, data = _detect_golden()
    for i, row in enumerate(g.softmax_rows()):
        want = data[f"softmax{i}"]
        assert np.array_equal(oracle_ref.ref_softmax(row), want)
        s, a, c = oracle_port.topk_per_class(row[None, :], score_thr=0.0, top_k=1)
        assert np.array_equal(s[:, 0], want[1:])


def test_topk_per_class_orders_ties_by_anchor(oracle_port):
    logits = np.zeros((6, 3), np.float32)
    logits[:, 1] = [1, 2, 2, 0, 2, 1]
    s, a, c = oracle_port.topk_per_class(logits, score_thr=0.0, top_k=4)
    assert c.tolist() == [4, 4]
    assert a[0].tolist() == [1, 2, 4, 0]


def test_preprocess_restatement_known_answers(oracle_port):
    """Detector::Preprocess with OpenCV's 8-bit bilinear rule restated. Properties that hold whatever
    the rounding details: same-size resize is the identity (channel swap + mean only), constants stay
    constant, a 2x upscale of a horizontal ramp interpolates with weights 1/4 : 3/4, and the first/last
    outputs clamp to the edge pixels."""
    rng = np.random.default_rng(50)
    img = rng.integers(0, 256, (37, 53, 3), dtype=np.uint8)
    mean = np.array([123.0, 117.0, 104.0], np.float32)
    assert np.array_equal(oracle_port.preprocess_bgr8(img, 37, 53), img[..., ::-1].astype(np.float32) - mean)
    const = np.full((9, 11, 3), 200, np.uint8)
    assert np.all(oracle_port.preprocess_bgr8(const, 300, 300, (0, 0, 0)) == 200.0)
    ramp = np.zeros((2, 4, 3), np.uint8)
    ramp[:, :, 0] = np.array([0, 40, 80, 120], np.uint8)            # blue channel -> output channel 2
    up = oracle_port.preprocess_bgr8(ramp, 2, 8, (0, 0, 0))[0, :, 2]
    assert list(up) == [0.0, 10.0, 30.0, 50.0, 70.0, 90.0, 110.0, 120.0]
    down = oracle_port.preprocess_bgr8(img, 10, 10)
    assert down.shape == (10, 10, 3) and np.all(down + mean >= 0) and np.all(down + mean <= 255)


def test_preprocess_matches_committed_opencv_outputs(oracle_port):
    """The pin: bit-exact against cv2.cvtColor + cv2.resize outputs committed in tests/golden/preprocess_cv2.npz
    (written by tests/golden/make_preprocess_golden.py), the calls detector.cc:99-109 makes."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_preprocess_golden as g
    data = np.load(os.path.join(os.path.dirname(__file__), "golden", "preprocess_cv2.npz"))
    for i, (img, (_, _, dh, dw)) in enumerate(zip(g.frames(), g.CASES)):
        assert np.array_equal(img, data[f"src{i}"])
        got = oracle_port.preprocess_bgr8(img, dh, dw, (0.0, 0.0, 0.0))
        assert np.array_equal(got, data[f"dst{i}"].astype(np.float32)), g.CASES[i]


def test_preprocess_matches_live_opencv(oracle_port):
    """The same pin against the installed OpenCV on frames of many sizes, edge rows and columns included
    (vertical taps outside the image keep their fractional weights on the clamped row; horizontal ones do not)."""
    cv2 = pytest.importorskip("cv2")
    rng = np.random.default_rng(51)
    sizes = [(480, 640, 300, 300), (1080, 1920, 300, 300), (97, 131, 300, 300), (21, 33, 48, 64), (150, 200, 160, 160),
             (600, 600, 300, 300), (150, 150, 300, 300), (299, 301, 300, 300), (5, 3, 2, 2)]
    sizes += [tuple(int(v) for v in rng.integers(1, 200, 4)) for _ in range(40)]
    mean = np.array([123.0, 117.0, 104.0], np.float32)
    for (h, w, dh, dw) in sizes:
        img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        want = cv2.resize(cv2.cvtColor(img, cv2.COLOR_BGR2RGB), (dw, dh)).reshape(dh, dw, 3).astype(np.float32) - mean
        assert np.array_equal(oracle_port.preprocess_bgr8(img, dh, dw), want), (h, w, dh, dw)
