"""Writes tests/golden/preprocess_cv2.npz: what OpenCV gives for the detector's image front end
(Detector::Preprocess, ogl_runtime/opengl/examples/ssd/detector.cc:99-109 in kl456123/OGLE:
cv::cvtColor BGR->RGB, cv::resize with the default INTER_LINEAR) on small seeded frames that
shrink, enlarge, halve and keep their size. Needs cv2; the committed file lets the pin run
where cv2 is absent.

    python tests/golden/make_preprocess_golden.py
"""
import os

import numpy as np

CASES = [  # src_h, src_w, dst_h, dst_w
    (48, 64, 30, 30), (13, 10, 30, 30), (33, 21, 64, 48), (60, 60, 30, 30), (30, 30, 30, 30), (2, 2, 7, 5), (1, 1, 4, 4),
    (31, 29, 30, 30), (97, 131, 40, 52)]


def frames():
    rng = np.random.default_rng(4242)
    return [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (h, w, _, _) in CASES]


if __name__ == "__main__":
    import cv2
    out = {}
    for i, (img, (_, _, dh, dw)) in enumerate(zip(frames(), CASES)):
        out[f"src{i}"] = img
        out[f"dst{i}"] = cv2.resize(cv2.cvtColor(img, cv2.COLOR_BGR2RGB), (dw, dh)).reshape(dh, dw, 3)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "preprocess_cv2.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes; cv2", cv2.__version__)
