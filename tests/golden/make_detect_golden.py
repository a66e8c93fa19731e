"""Writes tests/golden/reference_detect_outputs.npz: the detections that the reference's own
post-process (examples/ssd/detector.cc GenerateBoxInfo -> GetTopK -> NMS and common.cc iou,
compiled for the CPU into oracle/_ref/libogle_ref.so by oracle/ref_detector.cc) keeps for
seeded boxes and logits, and its softmax of seeded rows. Inputs are regenerated from the
seeds by detect_cases(); the file holds only the reference's outputs.

    make -C oracle ref && python tests/golden/make_detect_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [  # anchors, classes, image_w, image_h, score_thr, top_k, nms_thr, logit scale
    (1917, 21, 300, 300, 0.3, 100, 0.45, 3.0), (1917, 2, 300, 300, 0.3, 100, 0.45, 2.0), (333, 5, 640, 480, 0.1, 10, 0.3, 1.0),
    (50, 3, 100, 100, 0.6, 400, 0.7, 2.0), (700, 10, 1920, 1080, 0.2, 200, 0.5, 3.0), (64, 4, 300, 300, 0.9999, 100, 0.45, 1.0)]


def detect_cases():
    """Seeded (boxes [A,4] corner form in [0,1], logits [A,C]) per case; scores are continuous, so no two tie."""
    out = []
    for i, (A, C, _, _, _, _, _, scale) in enumerate(CASES):
        rng = np.random.default_rng(9000 + i)
        logits = (rng.standard_normal((A, C), dtype=np.float32) * np.float32(scale)).astype(np.float32)
        ctr = rng.random((A, 2), dtype=np.float32)
        half = rng.random((A, 2), dtype=np.float32) * np.float32(0.2) + np.float32(0.02)
        out.append((np.concatenate([ctr - half, ctr + half], axis=-1).astype(np.float32), logits))
    return out


def softmax_rows():
    rng = np.random.default_rng(9100)
    return [(rng.standard_normal(n, dtype=np.float32) * np.float32(3)).astype(np.float32) for n in (2, 5, 21, 21, 91)]


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import oracle
    ref = oracle.load("reference")
    out = {}
    for i, ((boxes, logits), (_, _, w, h, thr, k, nms, _)) in enumerate(zip(detect_cases(), CASES)):
        r = ref.ref_detect(boxes, logits, w, h, thr, k, nms)
        out[f"rect{i}"], out[f"score{i}"], out[f"cls{i}"] = r["rect"], r["score"], r["cls"]
        print(CASES[i], "->", len(r["score"]), "kept")
    for i, row in enumerate(softmax_rows()):
        out[f"softmax{i}"] = ref.ref_softmax(row)
    path = os.path.join(HERE, "reference_detect_outputs.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")
