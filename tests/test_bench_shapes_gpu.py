"""GPU parity at the launch configurations the benchmark times.

Tile shape, N-tile width, split reduction, accumulator count and the depthwise tile
cuts are chosen from the number of tiles against the number of SMs, so a layer at
batch 256 (one GPU of the benchmark), at batch 32 (one GPU of eight sharing a batch
of 256) and at batch 2 (the other tests) runs through different code paths. Images do
not interact, so the oracle only has to run the sampled images: the device computes
the whole batch, the CPU computes a handful of its images, and those must agree to the
same bounds the small-batch tests use.
"""
import os
import sys
import tempfile

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
import detect_checks  # noqa: E402

pytestmark = pytest.mark.gpu


def _norm_err(got, ref):
    return float(np.abs(got - ref).max() / max(1e-30, np.abs(ref).max()))


def _images(batch, seed0):
    """uniform [0,1] RGB normalised (x-0.5)/0.5, one seed per image (the benchmark's input rule)."""
    x = np.empty((batch, 300, 300, 3), np.float32)
    for i in range(batch):
        x[i] = (np.random.default_rng(seed0 + i).random((300, 300, 3), dtype=np.float32) - 0.5) / 0.5
    return x


def _sample(batch):
    return sorted({0, 1, batch // 2 - 1, batch // 2, batch - 2, batch - 1})


@pytest.mark.parametrize("batch", [256, 32])
def test_mobilenet_ssd_benchmark_batches_sampled_against_oracle(oracle_port, batch):
    """MobileNet-v1-SSD-300, 21 classes, default 3xTF32 mode, at the batch sizes the benchmark runs
    per GPU: logits, box regressions, decoded boxes and per-class top-200 of six sampled images."""
    from ogle_b200 import models, session
    from oracle import graph_oracle
    model, _ = models.mobilenet_v1_ssd(batch=batch, num_classes=21, seed=3, weight_std="he")
    pick = _sample(batch)
    small, _ = models.mobilenet_v1_ssd(batch=len(pick), num_classes=21, seed=3, weight_std="he")
    x = _images(batch, 41000)
    ref = graph_oracle.run_graph(small, {"input": x[pick]}, oracle_port, keep={"cls_logits", "box_preds", "anchors"})
    ref_boxes = oracle_port.decode(ref["box_preds"], ref["anchors"])
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ssd.dlx")
        model.save(path)
        det = session.Detector(path, mode=1, score_thr=0.01, top_k=200, math_mode=2)
        for rep in range(3):                    # eager pass, graph capture, graph replay
            out = det.detect(x)
        sess = det.session()
        assert sess.graph_captured()
        logits = sess.GetOutputs(["cls_logits"], ["ANY"])[0]
        preds = sess.GetOutputs(["box_preds"], ["ANY"])[0]
        det.close()
    assert logits.shape == (batch, 1917, 21)
    e = _norm_err(logits[pick], ref["cls_logits"])
    assert e <= 2e-4, f"cls_logits normalised error {e:.3e}"
    e = _norm_err(preds[pick], ref["box_preds"])
    assert e <= 2e-4, f"box_preds normalised error {e:.3e}"
    assert np.abs(logits[pick] - ref["cls_logits"]).max() <= 1e-3 * max(1.0, np.abs(ref["cls_logits"]).max())
    for j, n in enumerate(pick):
        s_ref, a_ref, c_ref = oracle_port.topk_per_class(ref["cls_logits"][j], 0.01, 200)
        got_s = out["score"][n].reshape(20, 200)
        got_a = out["anchor"][n].reshape(20, 200)
        assert np.abs(got_s - s_ref).max() <= 1e-4
        detect_checks.near_tie_only(got_a, a_ref, s_ref, 2e-4)
        # a count may differ only by candidates whose score is within tolerance of the threshold
        detect_checks.per_class_counts_differ_only_at_threshold(out["count"][n], c_ref, got_s, s_ref, 0.01, 2e-4, f"image {n}")
        sel = got_a >= 0
        got_box = out["box"][n].reshape(20, 200, 4)[sel]
        assert np.abs(got_box - ref_boxes[j][got_a[sel]]).max() <= 1e-3


def test_mobilenet_ssd_batch32_reference_rule_indices(oracle_port):
    """The reference Detector's rule (best class, top-100, NMS on integer rectangles) at 32 images:
    where the kept set differs from the oracle's, every difference must trace to a near tie."""
    from ogle_b200 import models, ops, session
    from oracle import graph_oracle
    batch = 32
    model, _ = models.mobilenet_v1_ssd(batch=batch, num_classes=21, seed=5, weight_std="he")
    pick = _sample(batch)
    small, _ = models.mobilenet_v1_ssd(batch=len(pick), num_classes=21, seed=5, weight_std="he")
    x = _images(batch, 42000)
    ref = graph_oracle.run_graph(small, {"input": x[pick]}, oracle_port, keep={"cls_logits", "box_preds", "anchors"})
    boxes = oracle_port.decode(ref["box_preds"], ref["anchors"])
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ssd.dlx")
        model.save(path)
        det = session.Detector(path, mode=0, score_thr=0.3, top_k=100, nms_thr=0.45, math_mode=2)
        out = det.detect(x)
        sess = det.session()
        logits = sess.GetOutputs(["cls_logits"], ["ANY"])[0]
        preds = sess.GetOutputs(["box_preds"], ["ANY"])[0]
        det.close()
    gpu_boxes = ops.ssd_decode(ops.dense_to_device(preds), ops.dense_to_device(ref["anchors"])).cpu().numpy()
    exact = 0
    for j, n in enumerate(pick):
        exact += detect_checks.reference_rule(oracle_port, out, n, gpu_boxes[n], logits[n], boxes[j], ref["cls_logits"][j],
                                              (300, 300), 0.3, 100, 0.45, 2e-4)
    assert exact >= len(pick) // 2, "most images are expected to match the oracle's kept anchors exactly"


@pytest.mark.parametrize("name", ["conv3x3", "pointwise", "depthwise", "maxpool", "concat"])
def test_operator_sweep_shapes_at_32_images(oracle_port, name):
    """The single-operator benchmark shapes at their full batch of 32, N(0,1) activations and N(0,0.05)
    weights; the oracle runs images 0 and 31. 3xTF32 for the dense convolutions, as benchmarked."""
    from gpu_ops import run_case_cuda
    from ogle_b200 import ops
    rng = np.random.default_rng(61)
    N, pick = 32, [0, 31]
    if name in ("conv3x3", "pointwise", "depthwise"):
        H, C, K, k, s, p, g = {"conv3x3": (38, 256, 256, 3, 1, 1, 1), "pointwise": (19, 512, 1024, 1, 1, 0, 1),
                               "depthwise": (38, 512, 512, 3, 2, 1, 512)}[name]
        x = rng.standard_normal((N, H, H, C), dtype=np.float32)
        w = rng.standard_normal((K, C // g, k, k), dtype=np.float32) * np.float32(0.05)
        b = rng.standard_normal(K, dtype=np.float32) * np.float32(0.05)
        case = dict(op="conv2d", x=x, w=w, bias=b, stride=s, pad=p, dilation=1, group=g, act=2, lo=0.0, hi=0.0)
        got = run_case_cuda(case, ops.MATH_TF32X3)
        ref = oracle_port.conv2d(x[pick], w, b, s, p, 1, g, 2)
        err = float(np.abs(got[pick] - ref).max())
        assert err <= 1e-3 and err <= 1e-4 * np.abs(ref).max(), (err, float(np.abs(ref).max()))
    elif name == "maxpool":
        x = rng.standard_normal((N, 76, 76, 256), dtype=np.float32)
        got = run_case_cuda(dict(op="pool", x=x, kernel=3, stride=2, pad=1, type_=0))
        assert np.array_equal(got[pick], oracle_port.pool(x[pick], 3, 2, 1, 0))
    else:
        xs = [rng.standard_normal((N, 19, 19, 256), dtype=np.float32) for _ in range(4)]
        got = run_case_cuda(dict(op="concat", xs=xs, axis=3))
        assert got.shape == (N, 19, 19, 1024)
        assert np.array_equal(got, np.concatenate(xs, axis=3))
        assert np.array_equal(got[pick], oracle_port.concat([x[pick] for x in xs], 3))


def test_gemm_4096_cubed_sampled_rows(oracle_port):
    """gemm M=N=K=4096 (N(0,1) x N(0,0.05)), 3xTF32: eight rows of A through the oracle."""
    import torch
    from ogle_b200 import ops
    g = torch.Generator().manual_seed(62)
    A = torch.randn((4096, 4096), generator=g).numpy()
    B = (torch.randn((4096, 4096), generator=g) * 0.05).numpy()
    rows = [0, 1, 127, 128, 2047, 2048, 4094, 4095]
    y = ops.gemm(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), None, 4096, 4096, 4096, 0, 1.0, 1.0, 0,
                 ops.MATH_TF32X3).cpu().numpy()
    ref = oracle_port.gemm(A[rows], B, None, 0, 1.0, 1.0)
    err = np.abs(y[rows] - ref).max()
    assert err <= 1e-3 and err / np.abs(ref).max() <= 1e-4, (float(err), float(np.abs(ref).max()))


def test_decoder_config_1024_images(oracle_port):
    """SSD decoder standalone at its benchmark size: 1024 images x 1917 anchors x 21 classes, deltas
    N(0,0.5), logits N(0,2), softmax + threshold 0.01 + per-class top-200; images 0, 1, 511, 1023 through the
    oracle. Scores to fp32 rounding, indices exact off near ties, boxes exactly those of the kept anchors."""
    import torch
    from ogle_b200 import models, ops
    g = torch.Generator().manual_seed(63)
    N, A, C = 1024, 1917, 21
    loc = (torch.randn((N, A, 4), generator=g) * 0.5).numpy()
    conf = np.zeros((N, A, 24), np.float32)
    conf[..., :C] = (torch.randn((N, A, C), generator=g) * 2).numpy()
    priors = models.ssd_prior_boxes()
    boxes = ops.ssd_decode(torch.from_numpy(loc).cuda(), ops.dense_to_device(priors))
    score, anchor, cls, box, count = [t.cpu().numpy() for t in ops.ssd_detect(
        torch.from_numpy(conf).cuda(), boxes, C, 1, 0.01, 200)]
    boxes = boxes.cpu().numpy()
    for n in (0, 1, 511, 1023):
        ref_box = oracle_port.decode(loc[n:n + 1], priors)[0]
        assert np.abs(boxes[n] - ref_box).max() <= 1e-5
        s_ref, a_ref, c_ref = oracle_port.topk_per_class(conf[n, :, :C], 0.01, 200)
        assert np.array_equal(count[n], c_ref)
        got_s, got_a = score[n].reshape(20, 200), anchor[n].reshape(20, 200)
        assert np.abs(got_s - s_ref).max() <= 2e-6
        detect_checks.near_tie_only(got_a, a_ref, s_ref, 4e-6)
        sel = got_a >= 0
        assert np.array_equal(box[n].reshape(20, 200, 4)[sel], boxes[n][got_a[sel]])


def test_resnet18_batch128_sampled_against_oracle(oracle_port):
    """ResNet-18 224x224 at its benchmark batch of 128 (3xTF32): logits of four sampled images."""
    from ogle_b200 import models, session
    from oracle import graph_oracle
    batch, pick = 128, [0, 63, 64, 127]
    model, _ = models.resnet18(batch=batch, seed=4, weight_std="he")
    small, _ = models.resnet18(batch=len(pick), seed=4, weight_std="he")
    x = np.random.default_rng(64).standard_normal((batch, 224, 224, 3), dtype=np.float32)
    ref = graph_oracle.run_graph(small, {"input": x[pick]}, oracle_port, keep={"logits"})["logits"]
    sess = session.FBOSession()
    sess.set_option("math_mode", 2)
    sess.LoadGraph(model)
    for _ in range(3):
        sess.Run({"input": x})
    assert sess.graph_captured()
    got = sess.GetOutputs(["logits"], ["ANY"])[0]
    sess.close()
    assert got.shape == (batch, 1000)
    e = _norm_err(got[pick], ref)
    assert e <= 5e-4, f"normalised error {e:.3e}"
