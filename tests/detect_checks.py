"""Checks of kept anchor indices against the oracle that accept a difference only where it
traces to a near tie: bit-exact wherever scores (or the pixel a box edge truncates to) are not
tied within tolerance. Shared by the whole-graph GPU tests."""
import numpy as np


def near_tie_only(got_idx, ref_idx, ref_score, tol):
    """Per-class top-k tables [C-1, k]: every position where the kept index differs must sit in a
    group of oracle scores within tol of each other."""
    for pos in zip(*np.nonzero(got_idx != ref_idx)):
        row = ref_score[pos[:-1]]
        assert (np.abs(row - row[pos[-1]]) <= tol).sum() > 1, f"index differs at {pos} without a near tie"


def per_class_counts_differ_only_at_threshold(got_count, ref_count, got_score, ref_score, thr, tol, what=""):
    for c in np.nonzero(got_count != ref_count)[0]:
        lo, hi = sorted((int(got_count[c]), int(ref_count[c])))
        edge = np.concatenate([ref_score[c, lo:hi], got_score[c, lo:hi]])
        edge = edge[edge > 0]
        assert edge.size and np.abs(edge - thr).max() <= tol, f"{what} class {c + 1}: count differs away from the threshold"


def reference_rule(oracle, got, n, gpu_boxes, gpu_logits, ref_boxes, ref_logits, size, thr, top_k, nms_thr, tol,
                   pixel_tol=0.05):
    """Detections of image n under the reference Detector's rule (best class, threshold, top-k, greedy
    suppression on integer rectangles) against the oracle.

    got: the detector's output dict; gpu_boxes / gpu_logits: what the device network produced for the
    image; ref_boxes / ref_logits: the oracle network's. An exact match of kept anchors passes.
    Otherwise (1) the device's post-process must equal the oracle's post-process of the device's own
    network outputs exactly, and (2) the two ordered candidate lists before suppression may differ only by
    score near ties (against the threshold, the top-k cut or a neighbour in the order) or by a rectangle
    edge within pixel_tol of the integer it truncates to; with identical candidate lists the kept sets
    cannot differ."""
    H, W = size
    r = oracle.detect(ref_boxes, ref_logits, W, H, thr, top_k, nms_thr)
    cnt = int(got["count"][n])
    kept = got["anchor"][n, :cnt]
    assert (got["anchor"][n, cnt:] == -1).all()
    if cnt == len(r["anchor"]) and np.array_equal(kept, r["anchor"]):
        assert np.array_equal(got["cls"][n, :cnt], r["cls"])
        assert np.abs(got["score"][n, :cnt] - r["score"]).max() <= max(tol, 2e-6)
        assert np.abs(got["box"][n, :cnt] - r["rect"]).max() <= 1
        return True
    own = oracle.detect(gpu_boxes, gpu_logits, W, H, thr, top_k, nms_thr)
    assert np.array_equal(kept, own["anchor"]), f"image {n}: post-process differs from the oracle's on the same inputs"
    assert np.array_equal(got["cls"][n, :cnt], own["cls"])
    assert np.array_equal(got["box"][n, :cnt].astype(np.int32), own["rect"])
    cr = oracle.detect(ref_boxes, ref_logits, W, H, thr, top_k, 1.0)      # IoU > 1 never holds: candidates only
    cg = oracle.detect(gpu_boxes, gpu_logits, W, H, thr, top_k, 1.0)
    explained = 0
    score_of = dict(zip(cr["anchor"].tolist(), cr["score"].tolist()))
    score_of.update({a: s for a, s in zip(cg["anchor"].tolist(), cg["score"].tolist()) if a not in score_of})
    cut = float(cr["score"][-1]) if len(cr["score"]) >= top_k else thr
    for a in set(cr["anchor"].tolist()) ^ set(cg["anchor"].tolist()):
        s = score_of[a]
        assert min(abs(s - thr), abs(s - cut)) <= tol, f"image {n}: candidate {a} (score {s:.6f}) differs away from the cut"
        explained += 1
    common = [a for a in cr["anchor"].tolist() if a in set(cg["anchor"].tolist())]
    order_g = [a for a in cg["anchor"].tolist() if a in set(common)]
    for a, b in zip(common, order_g):
        if a != b:
            assert abs(score_of[a] - score_of[b]) <= tol, f"image {n}: order of {a} and {b} differs without a near tie"
            explained += 1
    rect_r = dict(zip(cr["anchor"].tolist(), cr["rect"].tolist()))
    rect_g = dict(zip(cg["anchor"].tolist(), cg["rect"].tolist()))
    scale = np.array([W, H, W, H], np.float32)
    for a in common:
        if rect_r[a] != rect_g[a]:
            px = ref_boxes[a] * scale
            edges = np.array([px[0], px[1], px[2] - px[0], px[3] - px[1]])
            assert np.abs(edges - np.round(edges)).min() <= pixel_tol, f"image {n}: rectangle of {a} differs away from a pixel edge"
            explained += 1
    assert explained > 0, f"image {n}: kept sets differ although the candidate lists are identical"
    return False
