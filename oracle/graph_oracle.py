"""Test infrastructure only: runs a dlx graph on the CPU by chaining oracle ops.

Mirrors the session's rules (ogl_runtime/opengl/core/fbo_session.cc:127-252 and
the kernels under nn/kernels/): nodes run in file order; image tensors are stored
NHWC ("NHWC4" after the upload), so Transpose remaps an ONNX perm through
{0,3,1,2} and Reshape/Flatten keep the stored element order. Tensors are logical
(unpadded) numpy arrays. Only tests, the smoke check and the benchmark's
CPU-baseline leg import this.
"""
import numpy as np


def run_graph(model, inputs, lib, stop_after=None, keep=None):
    """model: ogle_b200.dlx.Model; inputs: {name: NHWC array}; lib: oracle.Oracle.
    Returns {tensor_name: array} for every tensor (or only `keep` names)."""
    vals = [None] * len(model.tensor_names)
    fmt = [None] * len(model.tensor_names)       # "image" (stored NHWC) or "plain"
    onnx = model.producer_name == "ONNX"
    for node in model.nodes:
        t, a = node.type, node.attr
        ins = [vals[i] for i in node.input_index]
        infmt = fmt[node.input_index[0]] if node.input_index else None
        out_fmt = infmt
        if t == "Input":
            out = np.ascontiguousarray(inputs[node.name], dtype=np.float32)
            out_fmt = "image"
        elif t in ("Const", "Constant"):
            c = a["const_attr"]["value"]
            out = np.asarray(c.float_data, dtype=np.float32).reshape(c.dims)
            out_fmt = "plain"
        elif t == "Conv":
            p = a["conv2d_attr"]
            act = {"": 0, "Clip": 1, "Relu": 2}[p.get("activation_type", "")]
            dil = p.get("dilations", [1])
            out = lib.conv2d(ins[0], ins[1], ins[2] if len(ins) > 2 else None, p["strides"][0], p["pads"][0],
                             dil[0] if dil else 1, p.get("group", 1) or 1, act, p.get("min", 0.0), p.get("max", 0.0))
        elif t in ("MaxPool", "AveragePool"):
            p = a["maxpool_attr"]
            out = lib.pool(ins[0], p["kernel_shape"][0], p["strides"][0], p["pads"][0], 0 if t == "MaxPool" else 1)
        elif t == "GlobalAveragePool":
            out = lib.pool(ins[0], ins[0].shape[1], 1, 0, 1)
        elif t == "BatchNormalization":
            out = lib.batchnorm(ins[0], ins[1], ins[2], ins[3], ins[4], a["batchnorm_attr"].get("epsilon", 0.0))
        elif t == "Relu":
            out = lib.relu(ins[0])
        elif t == "Clip":
            out = lib.clip(ins[0], a["clip_attr"].get("min", 0.0), a["clip_attr"].get("max", 0.0))
        elif t == "Add":
            out = lib.add(ins[0], ins[1])
        elif t == "Gemm":
            p = a["gemm_attr"]
            out = lib.gemm(ins[0], ins[1], ins[2] if len(ins) > 2 else None, p.get("transB", 0), p.get("alpha", 0.0),
                           p.get("beta", 0.0))
            out_fmt = "plain"
        elif t == "Transpose":
            perm = list(a["transpose_attr"]["perm"])
            if onnx and infmt == "image":
                perm = [{0: 0, 1: 3, 2: 1, 3: 2}[q] for q in perm]
            out = lib.transpose(ins[0], perm)
            out_fmt = "plain"
        elif t == "Reshape":
            shape = [int(round(float(v))) for v in ins[1].reshape(-1)]
            shape = [ins[0].shape[i] if d == 0 else d for i, d in enumerate(shape)]
            out = ins[0].reshape(shape)
            out_fmt = "plain"
        elif t == "Flatten":
            axis = a.get("flatten_attr", {}).get("axis", 0)
            lead = int(np.prod(ins[0].shape[:axis], dtype=np.int64)) if axis else 1
            out = ins[0].reshape(lead, -1) if axis else ins[0].reshape(-1)
            out_fmt = "plain"
        elif t == "Concat":
            axis = a["concat_attr"].get("axis", 0)
            if onnx and infmt == "image" and axis >= 0:
                axis = {0: 0, 1: 3, 2: 1, 3: 2}[axis]
            out = lib.concat(ins, axis)
            out_fmt = "plain"
        elif t == "Shape":
            # nn/kernels/shape.cc:32-47: the stored dims (NHWC order for image tensors), as floats
            out = np.asarray(ins[0].shape, dtype=np.float32)
            out_fmt = "plain"
        elif t == "Gather":
            # nn/glsl/gather.glsl:7-18: a scalar index into the first texel of a shape tensor, the ONNX
            # (NCHW) index mapped onto the stored order: 0 -> x, 1 -> w, 2 -> y, anything else -> z
            sel = int(np.asarray(ins[1]).reshape(-1)[0])
            lane = {0: 0, 1: 3, 2: 1}.get(sel, 2)
            data = np.asarray(ins[0], dtype=np.float32).reshape(-1)
            out = np.full(np.asarray(ins[1]).shape, data[lane] if lane < data.size else 0.0, np.float32)
            out_fmt = "plain"
        elif t == "Unsqueeze":
            out = np.expand_dims(ins[0], int(a["unsqueeze_attr"]["axes"][0]))
            out_fmt = "plain"
        elif t == "Decoder":
            # nn/kernels/decoder.cc:12-92: prediction [1,A,4], anchors [1,h,w,4] with h*w == A
            out = lib.decode(ins[0], np.ascontiguousarray(ins[1]).reshape(-1, 4))
            out_fmt = "plain"
        else:
            raise NotImplementedError(t)
        vals[node.output_index[0]] = out
        fmt[node.output_index[0]] = out_fmt
        if stop_after is not None and node.name == stop_after:
            break
    names = model.tensor_names
    return {n: v for n, v in zip(names, vals) if v is not None and (keep is None or n in keep)}
