"""dlx wire format: Python writer/reader round trips, converter-contract checks and
the BN fold, all on the CPU."""
import numpy as np

from ogle_b200 import dlx, models


def test_wire_round_trip_is_stable():
    m, info = models.mobilenet_v1_ssd(batch=1, num_classes=2)
    raw = m.encode()
    m2 = dlx.decode(raw)
    assert m2.encode() == raw
    assert m2.producer_name == "ONNX"
    assert [n.type for n in m2.nodes] == [n.type for n in m.nodes]
    assert info["conv_nodes"] == 47 and info["num_anchors"] == 1917
    assert abs(info["flops_per_image"] - 2.370e9) < 1e6


def test_varint_negative_and_packed_fields():
    s = dlx.Scope()
    x = s.add_input("input", [1, 3, 8, 8])
    shape = s.add_const("shape", np.array([1, -1, 4], np.float32))
    s.add_node("r", "Reshape", [x, shape], {"reshape_attr": {}})
    s.add_node("c", "Concat", [x, x], {"concat_attr": {"axis": -1}})
    m = dlx.decode(s.model.encode())
    assert m.nodes[3].attr["concat_attr"]["axis"] == -1
    assert m.nodes[0].attr["input_attr"]["dims"] == [1, 3, 8, 8]
    assert m.nodes[1].attr["const_attr"]["value"].float_data.tolist() == [1.0, -1.0, 4.0]


def test_model_follows_converter_contract():
    """Const before first use, filter ANY->HWN4C4, others ANY->ANY4, tensor name == node name,
    nodes topologically ordered (onnx_converter.cc:99-151, graph.cc:233-326)."""
    m, _ = models.mobilenet_v1_ssd(batch=2, num_classes=21)
    produced = set()
    for node in m.nodes:
        assert all(i in produced for i in node.input_index), node.name
        assert len(node.output_index) == 1
        assert m.tensor_names[node.output_index[0]] == node.name
        produced.add(node.output_index[0])
        if node.type == "Conv":
            wnode = next(n for n in m.nodes if n.output_index[0] == node.input_index[1])
            v = wnode.attr["const_attr"]["value"]
            assert (v.data_format, v.target_data_format) == (dlx.ANY, dlx.HWN4C4) and len(v.dims) == 4
            if len(node.input_index) > 2:
                b = next(n for n in m.nodes if n.output_index[0] == node.input_index[2]).attr["const_attr"]["value"]
                assert (b.data_format, b.target_data_format) == (dlx.ANY, dlx.ANY4) and len(b.dims) == 1
            a = node.attr["conv2d_attr"]
            assert len(a["pads"]) == 4 and len(a["strides"]) == 2 and a["group"] >= 1 and len(a["dilations"]) >= 1
    assert set(m.output_names) == {"cls_logits", "box_preds", "anchors"}


def test_bn_fold_matches_unfused(oracle_port):
    """remapper.cc:142-149: conv -> BN -> relu equals the folded conv with fused relu."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 9, 9, 6), dtype=np.float32)
    w = rng.standard_normal((8, 6, 3, 3), dtype=np.float32) * 0.2
    b = rng.standard_normal(8, dtype=np.float32)
    g, be, mu = (rng.standard_normal(8, dtype=np.float32) for _ in range(3))
    var = np.abs(rng.standard_normal(8, dtype=np.float32)) + 0.1
    unfused = oracle_port.relu(oracle_port.batchnorm(oracle_port.conv2d(x, w, b, 1, 1), g, be, mu, var, 1e-5))
    wf, bf = models.fold_batchnorm(w, b, g, be, mu, var, 1e-5)
    fused = oracle_port.conv2d(x, wf, bf, 1, 1, 1, 1, 2)
    assert np.abs(fused - unfused).max() < 2e-5


def test_prior_boxes_shape_and_range():
    p = models.ssd_prior_boxes()
    assert p.shape == (1917, 4) and p.min() >= 0 and p.max() <= 1
    assert np.allclose(p[0, :2], [0.5 / 19, 0.5 / 19]) and np.isclose(p[0, 2], 0.2)
