"""GPU parity of whole graphs through the host runtime (dlx -> FBOSession -> CUDA
kernels) against the CPU oracle running the same dlx graph.

Tolerance (north star): max-abs 1e-3 and rel 1e-3 on feature maps and box
coordinates in fp32 mode, written as |diff| <= 1e-3 * max(1, max|ref|) per tensor
plus a tighter normalised bound that fp32 arithmetic actually meets.
"""
import os
import tempfile

import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
import detect_checks  # noqa: E402

pytestmark = pytest.mark.gpu


def _norm_err(got, ref):
    return float(np.abs(got - ref).max() / max(1e-30, np.abs(ref).max()))


def _mode_name(m):
    return {0: "fp32", 1: "tf32", 2: "tf32x3"}[m]


def test_registry_holds_the_reference_operator_names():
    from ogle_b200 import session
    names = set(session.registered_kernels())
    assert names == {"Conv", "BatchNormalization", "Relu", "Clip", "Add", "MaxPool", "AveragePool", "GlobalAveragePool",
                     "Gemm", "Concat", "Decoder", "Const", "Constant", "Transpose", "Reshape", "Flatten", "Shape",
                     "Gather", "Unsqueeze"}


def test_single_conv_session_round_trip(oracle_port):
    """conv2d_test.cc:139-204: run, read back output (NHWC), weights (NCHW) and bias (ANY)."""
    from ogle_b200 import models, session
    rng = np.random.default_rng(31)
    for (H, C, K, k, s, p, g) in [(8, 3, 5, 3, 1, 1, 1), (16, 8, 8, 3, 2, 1, 8), (7, 6, 10, 1, 1, 0, 1), (9, 4, 8, 3, 1, 1, 2)]:
        x = rng.random((2, H, H, C), dtype=np.float32)
        w = rng.random((K, C // g, k, k), dtype=np.float32)
        b = rng.random(K, dtype=np.float32)
        sess = session.FBOSession()
        sess.set_option("math_mode", 0)
        sess.LoadGraph(models.single_conv(x.shape, w, b, s, p, 1, g))
        sess.Run({"input": x})
        out, w_back, b_back = sess.GetOutputs(["output", "conv2d1.weight", "conv2d1.bias"], ["NHWC", "NCHW", "ANY"])
        assert np.array_equal(w_back, w) and np.array_equal(b_back, b)
        ref = oracle_port.conv2d(x, w, b, s, p, 1, g)
        assert np.abs(out - ref).max() <= 1e-5 + 1e-5 * np.abs(ref).max()
        sess.close()


def test_unknown_operator_and_bad_file_are_errors_not_aborts():
    from ogle_b200 import dlx, session
    s = dlx.Scope()
    x = s.add_input("input", [1, 3, 4, 4])
    s.add_node("y", "NoSuchOp", [x])
    sess = session.FBOSession()
    with pytest.raises(session.OgleError, match="unsupported kernel name NoSuchOp"):
        sess.LoadGraph(s.model)
    with pytest.raises(session.OgleError):
        sess.LoadGraph("/nonexistent/model.dlx")
    with pytest.raises(session.OgleError, match="malformed"):
        sess.LoadGraph(b"\x0a\xff\xff\xff\xff\x0f")
    sess.close()


@pytest.mark.parametrize("math_mode,bound", [(0, 2e-5), (2, 2e-4), (1, 3e-2)])
def test_mobilenet_ssd_feature_maps_and_outputs(oracle_port, math_mode, bound):
    """MobileNet-v1-SSD 300x300, batch 2, 21 classes, He-scaled weights so every layer
    carries signal. Normalised error bounds per math mode: fp32 FMA 2e-5; 3xTF32 2e-4 (the
    tensor core's fp32 accumulation is not round-to-nearest, so it trails FMA by a few
    ulps per layer, still 5x inside the 1e-3 target); one-pass TF32 3e-2 (10-bit operands
    through 47 layers), the stated looser bound for that mode."""
    from ogle_b200 import models, session
    from oracle import graph_oracle
    model, info = models.mobilenet_v1_ssd(batch=2, num_classes=21, seed=3, weight_std="he")
    rng = np.random.default_rng(32)
    x = ((rng.random((2, 300, 300, 3), dtype=np.float32) - 0.5) / 0.5).astype(np.float32)
    convs = [n.name for n in model.nodes if n.type == "Conv"]
    probe = [convs[0], convs[1], convs[2], convs[12], convs[22], convs[26], convs[30], convs[34]]
    ref = graph_oracle.run_graph(model, {"input": x}, oracle_port, keep=set(probe) | {"cls_logits", "box_preds"})
    sess = session.FBOSession()
    sess.set_option("math_mode", math_mode)
    sess.LoadGraph(model)
    sess.Run({"input": x})
    for name in probe:
        got = sess.GetOutputs([name], ["NHWC"])[0]
        e = _norm_err(got, ref[name])
        assert e <= bound, f"{_mode_name(math_mode)} {name}: normalised error {e:.3e}"
        if math_mode != 1:
            assert np.abs(got - ref[name]).max() <= 1e-3 * max(1.0, np.abs(ref[name]).max())
    for name in ("cls_logits", "box_preds"):
        got = sess.GetOutputs([name], ["ANY"])[0]
        assert got.shape == ref[name].shape
        e = _norm_err(got, ref[name])
        assert e <= bound, f"{_mode_name(math_mode)} {name}: normalised error {e:.3e}"
    # steady state: the second and third runs replay a CUDA graph and give the same bits
    first = sess.GetOutputs(["cls_logits"], ["ANY"])[0]
    sess.Run({"input": x})
    sess.Run({"input": x})
    assert sess.graph_captured()
    assert np.array_equal(sess.GetOutputs(["cls_logits"], ["ANY"])[0], first)
    sess.close()


def test_sibling_fusion_is_transparent():
    """The six box/class head pairs of the SSD graph run as six passes instead of twelve; switching
    the fusion off gives the same tensors to within the arithmetic's own accuracy: a stacked pair and its two
    single convolutions may split their reductions into different numbers of ranges, and the tensor core's
    accumulator truncates at every step, so the grouping of a 9216-term sum shows at 1e-4 of the tensor's scale
    (the modes' bounds against the oracle are 2e-4 and 3e-2)."""
    from ogle_b200 import models, session
    model, _ = models.mobilenet_v1_ssd(batch=2, num_classes=21, seed=6, weight_std="he")
    x = ((np.random.default_rng(36).random((2, 300, 300, 3), dtype=np.float32) - 0.5) / 0.5).astype(np.float32)
    for mode in (1, 2):
        outs, counts = [], []
        for fuse in (1, 0):
            sess = session.FBOSession()
            sess.set_option("math_mode", mode)
            sess.set_option("fuse_siblings", fuse)
            sess.set_option("tune", 0)
            sess.LoadGraph(model)
            sess.Run({"input": x})
            outs.append(sess.GetOutputs(["cls_logits", "box_preds"], ["ANY", "ANY"]))
            counts.append(sess.num_active_kernels())
            sess.close()
        assert counts[1] - counts[0] == 6
        for a, b in zip(*outs):
            assert np.abs(a - b).max() <= 3e-4 * max(1.0, np.abs(b).max())


def test_branch_overlap_is_transparent():
    """The captured graph records independent branches (SSD heads against the layers that continue
    from their feature map) on side streams; the tensors are bit-identical to a graph recorded as one
    chain, run after run (every node does the same arithmetic; only the order in time changes)."""
    from ogle_b200 import models, session
    model, _ = models.mobilenet_v1_ssd(batch=3, num_classes=21, seed=8, weight_std="he")
    rng = np.random.default_rng(38)
    xs = [((rng.random((3, 300, 300, 3), dtype=np.float32) - 0.5) / 0.5).astype(np.float32) for _ in range(2)]
    outs, branches = {}, {}
    for streams in (1, 3, 8):
        sess = session.FBOSession()
        sess.set_option("streams", streams)
        sess.set_option("tune", 0)            # sessions compared bit for bit: same launch shapes in each
        sess.LoadGraph(model)
        got = []
        for rep in range(4):                       # eager, capture, two replays
            sess.Run({"input": xs[rep & 1]})
            got.append(sess.GetOutputs(["cls_logits", "box_preds"], ["ANY", "ANY"]))
        assert sess.graph_captured()
        outs[streams], branches[streams] = got, sess.num_branches()
        sess.close()
    assert branches[1] == 0 and branches[3] >= 2 and branches[8] >= 2
    for streams in (3, 8):
        for rep in range(4):
            for a, b in zip(outs[streams][rep], outs[1][rep]):
                assert np.array_equal(a, b), (streams, rep)
    for a, b in zip(outs[3][0], outs[3][2]):       # same input, eager pass vs replay
        assert np.array_equal(a, b)


def test_mobilenet_ssd_config0_batch1_two_classes(oracle_port):
    """The reference's own CPU-runnable case: batch 1, 2 classes, N(0,0.02) weights."""
    from ogle_b200 import models, session
    from oracle import graph_oracle
    model, _ = models.mobilenet_v1_ssd(batch=1, num_classes=2, seed=0, weight_std=0.02)
    x = ((np.random.default_rng(33).random((1, 300, 300, 3), dtype=np.float32) - 0.5) / 0.5).astype(np.float32)
    ref = graph_oracle.run_graph(model, {"input": x}, oracle_port, keep={"cls_logits", "box_preds"})
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ssd.dlx")
        model.save(path)
        sess = session.FBOSession()
        sess.LoadGraph(path)
        sess.Run({"input": x})
        for name in ("cls_logits", "box_preds"):
            got = sess.GetOutputs([name], ["ANY"])[0]
            assert np.abs(got - ref[name]).max() <= 1e-3 and _norm_err(got, ref[name]) <= 1e-3
        sess.close()


def test_resnet18_logits(oracle_port):
    from ogle_b200 import models, session
    from oracle import graph_oracle
    model, _ = models.resnet18(batch=2, seed=4, weight_std="he")
    x = np.random.default_rng(34).standard_normal((2, 224, 224, 3), dtype=np.float32)
    ref = graph_oracle.run_graph(model, {"input": x}, oracle_port, keep={"logits"})["logits"]
    for mode in (0, 2):
        sess = session.FBOSession()
        sess.set_option("math_mode", mode)
        sess.LoadGraph(model)
        sess.Run({"input": x})
        got = sess.GetOutputs(["logits"], ["ANY"])[0]
        assert got.shape == (2, 1000)
        assert _norm_err(got, ref) <= (5e-5 if mode == 0 else 5e-4), f"{_mode_name(mode)}: {_norm_err(got, ref):.3e}"
        sess.close()


def test_pinned_host_array_round_trip():
    """Upload buffers from the runtime's pinned allocator: writable from numpy, usable as the source of an
    asynchronous upload, released without a trace."""
    import torch
    from ogle_b200 import session
    buf = session.PinnedArray((3, 300, 300, 3), np.float32)
    assert buf.ptr % (2 << 20) == 0 and not buf.array.any()
    rng = np.random.default_rng(40)
    buf.array[...] = rng.random(buf.shape, dtype=np.float32)
    dev = torch.empty(buf.shape, dtype=torch.float32, device="cuda")
    dev.copy_(torch.from_numpy(buf.array), non_blocking=True)
    torch.cuda.synchronize()
    assert np.array_equal(dev.cpu().numpy(), buf.array)
    buf.close()
    buf.close()                                         # idempotent


def test_activation_fusion_is_transparent():
    """ResNet's eight Add -> Relu tails run as eight passes instead of sixteen; the logits are
    bit-identical with the fusion off, and reading an Add result that is no longer produced fails
    with a message instead of returning stale memory."""
    from ogle_b200 import models, session
    model, _ = models.resnet18(batch=2, seed=4, weight_std="he")
    x = np.random.default_rng(39).standard_normal((2, 224, 224, 3), dtype=np.float32)
    add_out = next(model.tensor_names[n.output_index[0]] for n in model.nodes if n.type == "Add")
    outs, counts = [], []
    for fuse in (1, 0):
        sess = session.FBOSession()
        sess.set_option("fuse_activations", fuse)
        sess.set_option("tune", 0)
        sess.LoadGraph(model)
        for _ in range(3):                        # eager, capture, replay
            sess.Run({"input": x})
        outs.append(sess.GetOutputs(["logits"], ["ANY"])[0])
        counts.append(sess.num_active_kernels())
        if fuse:
            with pytest.raises(session.OgleError, match="not materialised"):
                sess.GetOutputs([add_out], ["ANY"])
        else:
            assert sess.GetOutputs([add_out], ["ANY"])[0].shape[0] == 2
        sess.close()
    assert counts[1] - counts[0] == 8
    assert np.array_equal(outs[0], outs[1])


def test_residual_fusion_is_transparent():
    """ResNet's eight residual tails (conv -> Add -> Relu) run inside the second convolution of each block
    (ogle_cuda_conv2d_residual): eight launches fewer again, the same logits as with the fusion off, and the
    convolution's own result, which is no longer produced, cannot be read."""
    from ogle_b200 import models, session
    model, _ = models.resnet18(batch=2, seed=6, weight_std="he")
    x = np.random.default_rng(41).standard_normal((2, 224, 224, 3), dtype=np.float32)
    add = next(n for n in model.nodes if n.type == "Add")
    conv_out = model.tensor_names[add.input_index[0]]
    outs, counts, fused = [], [], []
    for fuse in (1, 0):
        sess = session.FBOSession()
        sess.set_option("fuse_residuals", fuse)
        sess.set_option("tune", 0)
        sess.LoadGraph(model)
        for _ in range(3):                        # eager, capture, replay
            sess.Run({"input": x})
        outs.append(sess.GetOutputs(["logits"], ["ANY"])[0])
        counts.append(sess.num_active_kernels())
        fused.append(sess.num_residuals())
        if fuse:
            with pytest.raises(session.OgleError, match="not materialised"):
                sess.GetOutputs([conv_out], ["ANY"])
        else:
            assert sess.GetOutputs([conv_out], ["ANY"])[0].shape[0] == 2
        sess.close()
    assert fused == [8, 0]
    assert counts[1] - counts[0] == 8
    # the fused pass performs the separate passes' operations in their order (bit-identical at the operator level:
    # test_conv_with_residual_operand_equals_the_separate_passes), but a convolution with a residual operand never
    # splits its reduction, while the same layer on its own may: the partial sums can be grouped differently
    assert np.abs(outs[0] - outs[1]).max() <= 3e-4 * max(1.0, float(np.abs(outs[1]).max()))


def test_detector_end_to_end_matches_oracle_post_process(oracle_port):
    """Detector::Detect (detector.cc:275-295): network, decode, softmax / threshold / top-k / NMS."""
    from ogle_b200 import models, ops, session
    from oracle import graph_oracle
    model, info = models.mobilenet_v1_ssd(batch=3, num_classes=21, seed=5, weight_std="he")
    x = ((np.random.default_rng(35).random((3, 300, 300, 3), dtype=np.float32) - 0.5) / 0.5).astype(np.float32)
    ref = graph_oracle.run_graph(model, {"input": x}, oracle_port, keep={"cls_logits", "box_preds", "anchors"})
    boxes = oracle_port.decode(ref["box_preds"], ref["anchors"])
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ssd.dlx")
        model.save(path)
        det = session.Detector(path, mode=0, score_thr=0.3, top_k=100, nms_thr=0.45, math_mode=0)
        out = det.detect(x)
        sess = det.session()
        logits, preds = sess.GetOutputs(["cls_logits", "box_preds"], ["ANY", "ANY"])
        gpu_boxes = ops.ssd_decode(ops.dense_to_device(preds), ops.dense_to_device(ref["anchors"])).cpu().numpy()
        for n in range(3):
            # kept anchors and classes are exact; a difference must trace to a near tie (scores within 1e-4,
            # or a rectangle edge within 0.05 px of the integer it truncates to)
            detect_checks.reference_rule(oracle_port, out, n, gpu_boxes[n], logits[n], boxes[n], ref["cls_logits"][n],
                                         (300, 300), 0.3, 100, 0.45, 1e-4)
        det.close()
        det = session.Detector(path, mode=1, score_thr=0.01, top_k=200, math_mode=0)
        out = det.detect(x)
        for n in range(3):
            s_ref, a_ref, c_ref = oracle_port.topk_per_class(ref["cls_logits"][n], 0.01, 200)
            got_s, got_a = out["score"][n].reshape(20, 200), out["anchor"][n].reshape(20, 200)
            assert np.abs(got_s - s_ref).max() <= 1e-4
            detect_checks.near_tie_only(got_a, a_ref, s_ref, 1e-4)
            detect_checks.per_class_counts_differ_only_at_threshold(out["count"][n], c_ref, got_s, s_ref, 0.01, 1e-4, f"image {n}")
        det.close()


def test_concat_in_place_is_transparent(oracle_port):
    """Convolutions whose results only a channel Concat reads write straight into their slices of its tensor
    (widths 8, 12, 16 and a ragged last one of 6) and the Concat leaves the sequence; the tensors downstream are
    bit-identical to the copying Concat, in the CUDA-core and the tensor-core modes, eager and replayed."""
    from ogle_b200 import models, session
    from oracle import graph_oracle
    x = np.random.default_rng(41).standard_normal((3, 19, 17, 32)).astype(np.float32)
    # branches that differ in window or activation (no two can run as one sibling pass), then four 3x3 branches with
    # the sibling fusion off: a convolution that already shares its pass with a sibling keeps its own tensor
    for kernels, siblings in (((1, 3), 1), ((3,), 0)):
        model = models.concat_of_convs(x.shape, [8, 12, 16, 6], seed=9, kernels=kernels)
        ref = graph_oracle.run_graph(model, {"input": x}, oracle_port, keep={"cat", "output"})
        for mode in (0, 2):
            outs, counts = [], []
            for fuse in (1, 0):
                sess = session.FBOSession()
                sess.set_option("math_mode", mode)
                sess.set_option("fuse_siblings", siblings)
                sess.set_option("fuse_concats", fuse)
                sess.set_option("tune", 0)
                sess.LoadGraph(model)
                for _ in range(3):                        # eager, capture, replay
                    sess.Run({"input": x})
                outs.append(sess.GetOutputs(["cat", "output"], ["NHWC", "NHWC"]))
                counts.append(sess.num_active_kernels())
                assert sess.num_placed() == (4 if fuse else 0)
                if fuse:
                    with pytest.raises(session.OgleError, match="fuse_concats"):
                        sess.GetOutputs(["branch1"], ["NHWC"])
                sess.close()
            assert counts[1] - counts[0] == 1             # the Concat itself
            for a, b in zip(*outs):
                assert np.array_equal(a, b), (kernels, mode)
            bound = 1e-5 if mode == 0 else 2e-4
            assert _norm_err(outs[0][0], ref["cat"]) <= bound and _norm_err(outs[0][1], ref["output"]) <= bound


def test_ssd_class_heads_write_their_concat_in_place():
    """MobileNet-SSD: the six class heads end in a re-padding copy ([N,h,w,a*21] -> [N,h*w*a,21]); those copies
    write into the [N,1917,21] tensor directly and the class Concat disappears. The box heads are aliases of their
    convolutions' outputs and keep their Concat. Same bits as with the switch off."""
    from ogle_b200 import models, session
    model, _ = models.mobilenet_v1_ssd(batch=3, num_classes=21, seed=6, weight_std="he")
    x = ((np.random.default_rng(42).random((3, 300, 300, 3), dtype=np.float32) - 0.5) / 0.5).astype(np.float32)
    outs, counts = [], []
    for fuse in (1, 0):
        sess = session.FBOSession()
        sess.set_option("fuse_concats", fuse)
        sess.set_option("tune", 0)
        sess.LoadGraph(model)
        for _ in range(3):
            sess.Run({"input": x})
        outs.append(sess.GetOutputs(["cls_logits", "box_preds"], ["ANY", "ANY"]))
        counts.append(sess.num_active_kernels())
        assert sess.num_placed() == (6 if fuse else 0)
        sess.close()
    assert counts[1] - counts[0] == 1
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


def test_exported_shape_arithmetic_heads(oracle_port):
    """The head plumbing as an ONNX export writes it - Shape -> Gather -> Unsqueeze -> Concat -> Reshape
    (nn/kernels/shape.cc, gather.cc + gather.glsl:7-18, unsqueeze.cc:22-55) - runs in the setup pass and gives
    the same tensors as constant reshape targets; none of those nodes is left in the steady-state sequence."""
    from ogle_b200 import models, session
    from oracle import graph_oracle
    for batch in (1, 2):
        plain, _ = models.mobilenet_v1_ssd(batch=batch, num_classes=5, seed=11, weight_std="he")
        exported, _ = models.mobilenet_v1_ssd(batch=batch, num_classes=5, seed=11, weight_std="he", exported_shape_ops=True)
        assert {n.type for n in exported.nodes} >= {"Shape", "Gather", "Unsqueeze"}
        x = ((np.random.default_rng(43).random((batch, 300, 300, 3), dtype=np.float32) - 0.5) / 0.5).astype(np.float32)
        ref = graph_oracle.run_graph(exported, {"input": x}, oracle_port, keep={"cls_logits", "box_preds"})
        got = {}
        for name, model in (("plain", plain), ("exported", exported)):
            with tempfile.TemporaryDirectory() as d:
                path = os.path.join(d, "ssd.dlx")
                model.save(path)
                sess = session.FBOSession()
                sess.set_option("math_mode", 0)
                sess.LoadGraph(path)
                sess.Run({"input": x})
                got[name] = (sess.GetOutputs(["cls_logits", "box_preds"], ["ANY", "ANY"]), sess.num_active_kernels())
                sess.close()
        assert got["plain"][1] == got["exported"][1]
        for a, b, key in zip(got["plain"][0], got["exported"][0], ("cls_logits", "box_preds")):
            assert a.shape == ref[key].shape and np.array_equal(a, b)
            assert _norm_err(b, ref[key]) <= 2e-5


def test_shape_gather_unsqueeze_values():
    """Shape of a stored-NHWC tensor and Gather's index mapping (ONNX index 0, 1, 2, 3 -> N, C, H, W)."""
    from ogle_b200 import dlx, session
    s = dlx.Scope()
    x = s.add_input("input", [2, 5, 7, 9])                 # N, C, H, W
    dims = s.add_node("dims", "Shape", [x], {"shape_attr": {}})
    for i in range(4):
        idx = s.add_const(f"i{i}", np.array(i, np.float32), dlx.ANY, dlx.ANY4)
        g = s.add_node(f"g{i}", "Gather", [dims, idx], {"gather_attr": {"axis": 0}})
        s.add_node(f"u{i}", "Unsqueeze", [g], {"unsqueeze_attr": {"axes": [0]}})
    sess = session.FBOSession()
    sess.LoadGraph(s.model)
    sess.Run({"input": np.zeros((2, 7, 9, 5), np.float32)})
    assert sess.num_active_kernels() == 0
    assert sess.GetOutputs(["dims"], ["ANY"])[0].tolist() == [2.0, 7.0, 9.0, 5.0]
    got = [sess.GetOutputs([f"u{i}"], ["ANY"])[0] for i in range(4)]
    assert [g.shape for g in got] == [(1,)] * 4
    assert [float(g[0]) for g in got] == [2.0, 5.0, 7.0, 9.0]
    sess.close()


def test_decoder_node(oracle_port):
    """The Decoder operator inside a graph (nn/kernels/decoder.cc:12-92): deltas [1,A,4] against anchors
    [1,h,w,4]; the kernel's own variances; batch 1 only, as the reference defines it."""
    from ogle_b200 import models, session
    from oracle import graph_oracle
    model, anchors = models.box_decoder_graph(27, 71, seed=3)
    x = (np.random.default_rng(44).standard_normal((1, 27, 71, 4)) * 0.5).astype(np.float32)
    ref = graph_oracle.run_graph(model, {"input": x}, oracle_port, keep={"boxes"})["boxes"]
    sess = session.FBOSession()
    sess.LoadGraph(model)
    for _ in range(3):
        sess.Run({"input": x})
    got = sess.GetOutputs(["boxes"], ["ANY"])[0]
    sess.close()
    assert got.shape == (1, 27 * 71, 4) and np.abs(got - ref).max() <= 1e-5
    two, _ = models.box_decoder_graph(3, 4)
    two.nodes[0].attr["input_attr"]["dims"][0] = 2
    sess = session.FBOSession()
    sess.LoadGraph(two)
    with pytest.raises(session.OgleError):                 # anchors are per graph, predictions for two images
        sess.Run({"input": np.zeros((2, 3, 4, 4), np.float32)})
    sess.close()


def test_detector_scales_boxes_by_each_frames_own_size(oracle_port):
    """Reference rule on raw frames of different sizes: the pixel rectangles (and with them the suppression)
    use each frame's own rows x cols (origin_input_sizes_, detector.cc:102,179-180), not the network input size."""
    from ogle_b200 import models, ops, session
    rng = np.random.default_rng(45)
    model, _ = models.mobilenet_v1_ssd(batch=3, num_classes=21, seed=12, weight_std="he")
    sizes = [(480, 640), (300, 300), (123, 77)]
    # pixels within a few counts of the mean that Preprocess subtracts, so that the random-weight network sees inputs
    # of the usual size and decodes boxes of sane extent
    mean_bgr = np.array([104, 117, 123], np.int64)
    frames = [(mean_bgr + rng.integers(-2, 3, (h, w, 3))).astype(np.uint8) for (h, w) in sizes]
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ssd.dlx")
        model.save(path)
        det = session.Detector(path, mode=0, score_thr=0.3, top_k=100, nms_thr=0.45, math_mode=0)
        det.detect_bgr8_async(frames, 300, 300)
        out = det.wait()
        sess = det.session()
        logits, preds, anchors = sess.GetOutputs(["cls_logits", "box_preds", "anchors"], ["ANY", "ANY", "ANY"])
        det.close()
    boxes = ops.ssd_decode(ops.dense_to_device(preds), ops.dense_to_device(anchors)).cpu().numpy()
    for n, (h, w) in enumerate(sizes):
        r = oracle_port.detect(boxes[n], logits[n], w, h, 0.3, 100, 0.45)
        k = len(r["anchor"])
        assert out["count"][n] == k and np.array_equal(out["anchor"][n, :k], r["anchor"])
        assert k > 0 and np.abs(r["rect"]).max() < 1 << 20
        assert np.array_equal(out["box"][n, :k].astype(np.int32), r["rect"]), (h, w)


def test_detector_raw_frames_equal_host_preprocess(oracle_port):
    """Frames of different sizes through detect_bgr8_async (upload as bytes, resize + mean on the device)
    give the same detections as the float path fed with the oracle's preprocess of the same frames -
    the device preprocess is bit-exact, so everything downstream is identical. Two calls in flight."""
    from ogle_b200 import models, session
    rng = np.random.default_rng(37)
    model, _ = models.mobilenet_v1_ssd(batch=3, num_classes=21, seed=7, weight_std="he")
    sets = [[rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (h, w) in sizes]
            for sizes in ([(480, 640), (300, 300), (123, 77)], [(720, 1280), (64, 64), (301, 299)])]
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ssd.dlx")
        model.save(path)
        det = session.Detector(path, mode=1, score_thr=0.01, top_k=200)
        want = []
        for frames in sets:
            x = np.stack([oracle_port.preprocess_bgr8(f, 300, 300) for f in frames])
            want.append(det.detect(x))
        for frames in sets:                      # both calls in flight before the first wait
            det.detect_bgr8_async(frames, 300, 300)
        for w in want:
            got = det.wait()
            for key in ("score", "anchor", "cls", "box", "count"):
                assert np.array_equal(got[key], w[key]), key
        det.close()


def test_sharded_detector_fed_frames_equals_fed_tensors(oracle_port):
    """ShardedDetector (one rank here): a step published as 8-bit BGR frames in the shared host region and run
    with submit(frames=True) gives the detections of the same step published as the fp32 tensors that the
    reference's host-side preprocess makes of those frames; both come back through the shared result region."""
    from ogle_b200 import models, sharding
    rng = np.random.default_rng(61)
    n = 3
    model, _ = models.mobilenet_v1_ssd(batch=n, num_classes=21, seed=9, weight_std="he")
    frames = rng.integers(0, 256, (n, 300, 300, 3), dtype=np.uint8)
    tensors = np.stack([oracle_port.preprocess_bgr8(f, 300, 300) for f in frames])
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ssd.dlx")
        model.save(path)
        sd = sharding.ShardedDetector(path, n, 0, 1, "test_frames_%d" % os.getpid(), 21, (300, 300), mode=1,
                                      score_thr=0.01, top_k=200, with_frames=True)
        try:
            got = []
            for step, as_frames in ((0, False), (1, True)):
                if as_frames:
                    sd.batch.frame_slot(step)[...] = frames
                else:
                    sd.batch.input_slot(step)[...] = tensors
                sd.batch.publish(step)
                sd.submit(step, frames=as_frames)
                assert sd.retire() == step
                out = sd.batch.gather(step, timeout=10.0, merged=True)
                got.append({k: v.copy() for k, v in out.items()})
                sd.batch.release(step)
        finally:
            sd.close()
    assert got[0]["count"].sum() > 0
    for key in ("score", "anchor", "cls", "box", "count"):
        assert np.array_equal(got[0][key], got[1][key]), key


def test_profile_tool_reports_per_type_table(tmp_path):
    """ogle_profile (the headless counterpart of nn/profile_main.cc): loads a dlx file, runs it and
    prints the per-node-type table; --json gives the same numbers for scripts."""
    import json
    import subprocess
    from ogle_b200 import build, models
    build.build_all()
    model, _ = models.mobilenet_v1_ssd(batch=2, num_classes=21, seed=8, weight_std=0.02)
    path = str(tmp_path / "ssd.dlx")
    model.save(path)
    exe = os.path.join(os.path.dirname(build.__file__), "ogle_profile")
    r = subprocess.run([exe, path, "5", "--batch", "2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert "ExecTimePerRound" in r.stdout and "Node Type\tTime\tCount" in r.stdout
    conv_line = [l for l in r.stdout.splitlines() if l.startswith("Conv")]
    assert conv_line and conv_line[0].split()[-1] == "41"          # 47 convolutions, 6 head pairs fused
    r = subprocess.run([exe, path, "3", "--batch", "2", "--json", "--math", "tf32"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    d = json.loads(r.stdout)
    assert d["graph"] is True and d["nodes"]["Conv"]["count"] == 41 and d["exec_ms_per_round"] > 0
