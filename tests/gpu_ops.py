"""Runs one golden/oracle case through the CUDA C ABI (upload -> op -> download),
the same round trip a reference unit test makes through its session."""
import numpy as np
import torch

from ogle_b200 import ops


def run_case_cuda(case, math_mode=ops.MATH_FP32):
    c = dict(case)
    op = c.pop("op")
    if op == "conv2d":
        x, w, b = c["x"], c["w"], c["bias"]
        N, H, W, Cin = x.shape
        K, _, k, _ = w.shape
        p = ops.conv_params(N, H, W, Cin, K, k, c["stride"], c["pad"], c["dilation"], c["group"],
                            b is not None, c["act"], c["lo"], c["hi"], math_mode)
        packed = ops.conv2d_prepack(p, ops.dense_to_device(w))
        y4 = ops.conv2d(p, ops.upload(x), packed, ops.dense_to_device(b) if b is not None else None)
        return ops.download(y4, K)
    if op == "pool":
        x = c["x"]
        N, H, W, Cc = x.shape
        kernel, type_ = c["kernel"], c["type_"]
        p = ops.pool_params(N, H, W, Cc, kernel, c["stride"], c["pad"], type_)
        return ops.download(ops.pool(p, ops.upload(x)), Cc)
    if op == "batchnorm":
        x = c["x"]
        d = ops.dense_to_device
        y4 = ops.batchnorm(ops.upload(x), d(c["gamma"]), d(c["beta"]), d(c["mean"]), d(c["var"]), x.shape[-1], c["eps"])
        return ops.download(y4, x.shape[-1])
    if op == "relu":
        return ops.download(ops.relu(ops.upload(c["x"])), c["x"].shape[-1])
    if op == "clip":
        return ops.download(ops.clip(ops.upload(c["x"]), c["lo"], c["hi"]), c["x"].shape[-1])
    if op == "add":
        return ops.download(ops.add(ops.upload(c["a"]), ops.upload(c["b"])), c["a"].shape[-1])
    if op == "gemm":
        A, B, Cm = c["A"], c["B"], c.get("Cm")
        M, K = A.shape
        N = B.shape[0] if c["transB"] else B.shape[1]
        mode = 0 if Cm is None else (1 if Cm.ndim == 2 else 2)
        C4 = None if Cm is None else ops.upload(Cm)
        y4 = ops.gemm(ops.upload(A), ops.upload(B), C4, M, K, N, c["transB"], c["alpha"], c["beta"], mode, math_mode)
        return ops.download(y4, N)
    if op == "concat":
        xs = c["xs"]
        y4, shape = ops.concat([ops.upload(x) for x in xs], [x.shape for x in xs], c["axis"])
        return ops.download(y4, shape[-1])
    if op == "transpose":
        x = c["x"]
        y4, shape = ops.transpose(ops.upload(x), x.shape, c["perm"])
        return ops.download(y4, shape[-1])
    if op == "decode":
        out = ops.ssd_decode(ops.dense_to_device(c["pred"]), ops.dense_to_device(c["anchors"]))
        return out.cpu().numpy()
    if op == "pad4":
        return ops.upload(c["x"]).cpu().numpy()
    raise KeyError(op)
