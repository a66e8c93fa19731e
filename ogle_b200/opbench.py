"""Per-operator roofline table: the single-op shapes of the benchmark sweep, each launched through
the C ABI with inputs resident in HBM, timed launch by launch with CUDA events.

    python -m ogle_b200.opbench [--reps 200] [--warmup 20] [--json out.json]

Protocol: `warmup` untimed launches, then `reps` timed ones; before every timed launch a 256 MB
buffer is overwritten so that nothing of the previous launch is left in the 126 MB L2; each
launch has its own event pair on the launching stream; median and best are reported. Inputs
follow the sweep's distributions (N(0,1) activations, N(0,0.05) weights), one seeded CPU
generator per tensor. Fractions are of the measured peaks in MEASURED_PEAKS.json (HBM copy
bandwidth; bf16/2 for one-pass TF32, bf16/4 for 3xTF32), else of the stated fallback.

    python -m ogle_b200.opbench --one-conv N H C K kernel stride pad [--math tf32x3] [--n-tile T] [--split S]
                                [--sm-pair 0|1|2] [--channels-on-m 0|1|2] [--reps R]

runs one convolution layer with the launch variant pinned (the fields of OgleConvParams that the session's
tuning otherwise chooses) and prints its time: for comparing variants of a layer and for profiler captures of one.

This is the headless counterpart of the reference's per-op profile tool (nn/profile_main.cc):
a table per operator type, and JSON for scripts.
"""
import argparse
import ctypes as C
import json
import os
import statistics

import torch

from . import _lib, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=float(d["hbm_gbs"]), bf16=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, bf16=1400.0, source="fallback")


def randn(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).cuda()


class Timer:
    def __init__(self, reps, warmup):
        self.reps, self.warmup = reps, warmup
        self.flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")   # 256 MB

    def __call__(self, launch):
        for _ in range(self.warmup):
            launch()
        times = []
        for _ in range(self.reps):
            self.flush.fill_(1.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            launch()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1000.0)
        return statistics.median(times), min(times)


def conv_case(name, N, H, C_, K, k, s, p, group, seed):
    x4 = ops.upload(randn((N, H, H, C_), seed).cpu().numpy())
    w = randn((K, C_ // group, k, k), seed + 1, 0.05)
    b = randn((K,), seed + 2, 0.05)
    Ho = (H - k + 2 * p) // s + 1
    flops = 2.0 * N * Ho * Ho * K * (C_ // group) * k * k
    nbytes = 4.0 * (N * H * H * C_ + N * Ho * Ho * K + K * (C_ // group) * k * k + K)
    return dict(name=name, x4=x4, w=w, b=b, dims=(N, H, H, C_, K, k, s, p, group), flops=flops, bytes=nbytes)


def run_conv(case, mode, timer):
    N, H, W, C_, K, k, s, p, group = case["dims"]
    prm = ops.conv_params(N, H, W, C_, K, k, s, p, 1, group, True, ops.ACT_RELU, 0.0, 0.0, mode)
    packed = ops.conv2d_prepack(prm, case["w"])
    out = ops.conv2d(prm, case["x4"], packed, case["b"])
    lib = _lib.cuda_lib()
    kernel = lib.ogle_cuda_conv2d_kernel_name(C.byref(prm)).decode()
    args = (C.byref(prm), ops._p(case["x4"]), ops._p(packed), ops._p(case["b"]), ops._p(out), ops._stream())
    med, best = timer(lambda: lib.ogle_cuda_conv2d(*args))
    return kernel, med, best


def one_conv(args):
    """One layer, launch variant pinned; prints median microseconds per launch (back-to-back launches)."""
    N, H, Cc, K, k, st, pd = args.one_conv
    mode = {"fp32": ops.MATH_FP32, "tf32": ops.MATH_TF32, "tf32x3": ops.MATH_TF32X3}[args.math]
    x = randn((N, H, H, ops.up4(Cc)), 1)
    w = randn((K, Cc, k, k), 2, 0.05)
    b = randn((K,), 3, 0.05)
    p = ops.conv_params(N, H, H, Cc, K, k, st, pd, 1, 1, True, ops.ACT_RELU, 0.0, 0.0, mode)
    p.n_tile, p.split, p.sm_pair, p.channels_on_m = args.n_tile, args.split, args.sm_pair, args.channels_on_m
    packed = ops.conv2d_prepack(p, w)
    ws = ops.conv_workspace(p)
    y = ops.conv2d(p, x, packed, b, workspace=ws)
    torch.cuda.synchronize()
    times = []
    for _ in range(max(1, args.reps)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.conv2d(p, x, packed, b, y, workspace=ws)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0)
    Ho = (H + 2 * pd - k) // st + 1
    gflop = 2.0 * N * Ho * Ho * K * Cc * k * k / 1e9
    med = statistics.median(times)
    print(json.dumps({"op": "conv", "shape": args.one_conv, "math_mode": args.math,
                      "kernel": _lib.cuda_lib().ogle_cuda_conv2d_kernel_name(C.byref(p)).decode(),
                      "n_tile": args.n_tile, "split": args.split, "sm_pair": args.sm_pair, "channels_on_m": args.channels_on_m,
                      "us_median": med, "us_best": min(times), "tflops": gflop / med * 1e3,
                      "device_status": _lib.cuda_lib().ogle_cuda_device_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--one-conv", type=int, nargs=7, metavar=("N", "H", "C", "K", "KERNEL", "STRIDE", "PAD"))
    ap.add_argument("--math", default="tf32x3", choices=["fp32", "tf32", "tf32x3"])
    ap.add_argument("--n-tile", type=int, default=0)
    ap.add_argument("--split", type=int, default=0)
    ap.add_argument("--sm-pair", type=int, default=0)
    ap.add_argument("--channels-on-m", type=int, default=0)
    ap.add_argument("--reps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="", help="comma-separated case names")
    args = ap.parse_args()
    if args.one_conv:
        one_conv(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("opbench needs a CUDA device")
    pk = peaks()
    timer = Timer(args.reps, args.warmup)
    lib = _lib.cuda_lib()
    rows = []
    only = set(args.only.split(",")) if args.only else None
    # TF32 runs at half the bf16 rate; the fp32-grade mode issues one TF32 pass plus one BF16 pass of equal
    # tensor time per reduction chunk: two pass-equivalents
    modes = [("fp32", ops.MATH_FP32, None), ("tf32", ops.MATH_TF32, pk["bf16"] / 2), ("tf32x3", ops.MATH_TF32X3, pk["bf16"] / 4)]

    def add(name, mode, kernel, med, best, flops, nbytes, tensor_peak):
        tf, gb = flops / med / 1e6, nbytes / med / 1e3
        row = dict(op=name, math_mode=mode, kernel=kernel, us_median=med, us_best=best, tflops=tf, gbs=gb,
                   frac_hbm=gb / pk["hbm"], frac_tensor=(tf / tensor_peak if tensor_peak else None),
                   gflop=flops / 1e9, mbytes=nbytes / 1e6, peak_source=pk["source"])
        rows.append(row)
        print(json.dumps(row), flush=True)

    convs = [("conv3x3_n32_38x38_c256_k256", 32, 38, 256, 256, 3, 1, 1, 1, 1000),
             ("pointwise_n32_19x19_c512_k1024", 32, 19, 512, 1024, 1, 1, 0, 1, 1010),
             ("depthwise_n32_38x38_c512_s2", 32, 38, 512, 512, 3, 2, 1, 512, 1020)]
    for spec in convs:
        if only and spec[0] not in only:
            continue
        case = conv_case(*spec)
        for mname, mode, tpeak in modes:
            if spec[8] != 1 and mode != ops.MATH_FP32:
                continue      # depthwise has one path
            kernel, med, best = run_conv(case, mode, timer)
            add(spec[0], mname, kernel, med, best, case["flops"], case["bytes"], tpeak if spec[8] == 1 else None)
        del case
        torch.cuda.empty_cache()

    if not only or "gemm_4096" in only:
        M = K = N = 4096
        A4, B4 = randn((M, K), 1030), randn((K, N), 1031, 0.05)
        flops, nbytes = 2.0 * M * N * K, 4.0 * (M * K + K * N + M * N)
        out = torch.empty((M, N), dtype=torch.float32, device="cuda")
        for mname, mode, tpeak in modes:
            p = ops._gemm_params(A4, B4, None, M, K, N, 0, 1.0, 1.0, 0, mode)
            if mode == ops.MATH_FP32:
                call = lambda: lib.ogle_cuda_gemm(C.byref(p), ops._p(A4), ops._p(B4), None, ops._p(out), ops._stream())
                kernel = "gemm_simt_kernel"
            else:
                packed = ops.gemm_pack_b(B4, M, K, N, 0, mode)     # B is a constant (weights): packed once
                call = lambda: lib.ogle_cuda_gemm_packed(C.byref(p), ops._p(A4), ops._p(packed), None, ops._p(out), ops._stream())
                kernel = "conv_tc2_kernel"
            med, best = timer(call)
            add("gemm_4096", mname, kernel, med, best, flops, nbytes, tpeak)
        del A4, B4, out
        torch.cuda.empty_cache()

    if not only or "maxpool_n32_76x76_c256" in only:
        x4 = randn((32, 76, 76, 256), 1040)
        p = ops.pool_params(32, 76, 76, 256, 3, 2, 1, 0)          # pad 1 -> 38x38
        out = ops.pool(p, x4)
        nbytes = 4.0 * (x4.numel() + out.numel())
        med, best = timer(lambda: lib.ogle_cuda_pool(C.byref(p), ops._p(x4), ops._p(out), ops._stream()))
        add("maxpool_n32_76x76_c256", "fp32", "pool_kernel", med, best, 0.0, nbytes, None)
        del x4, out

    if not only or "concat_4x_n32_19x19_c256" in only:
        xs = [randn((32, 19, 19, 256), 1050 + i) for i in range(4)]
        shapes = [(32, 19, 19, 256)] * 4
        out, _ = ops.concat(xs, shapes, 3)
        cp = ops.ConcatParams()
        cp.n_inputs, cp.axis = 4, 3
        for i in range(4):
            cp.in_shapes[i][:] = list(shapes[i])
        ptrs = (C.c_void_p * 4)(*[x.data_ptr() for x in xs])
        nbytes = 4.0 * 2 * out.numel()
        med, best = timer(lambda: lib.ogle_cuda_concat(C.byref(cp), ptrs, ops._p(out), ops._stream()))
        add("concat_4x_n32_19x19_c256", "fp32", "concat_vec_kernel", med, best, 0.0, nbytes, None)
        del xs, out

    if not only or "ssd_decode_detect_n1024" in only:
        from . import models
        Nn, A, Cc = 1024, 1917, 21
        loc, conf = randn((Nn, A, 4), 2000, 0.5), randn((Nn, A, 24), 2001, 2.0)
        conf[..., Cc:] = 0.0
        pri = torch.from_numpy(models.ssd_prior_boxes()).cuda()
        boxes = ops.ssd_decode(loc, pri)
        v = (C.c_float * 4)(0.1, 0.1, 0.2, 0.2)
        med, best = timer(lambda: lib.ogle_cuda_ssd_decode(ops._p(loc), ops._p(pri), ops._p(boxes), Nn, A, v, ops._stream()))
        add("ssd_decode_n1024", "fp32", "ssd_decode_kernel", med, best, 0.0, 4.0 * (2 * loc.numel() + pri.numel()), None)
        dp = ops.DetectParams()
        dp.N, dp.A, dp.C, dp.logit_stride, dp.mode = Nn, A, Cc, 24, 1
        dp.score_thr, dp.top_k, dp.nms_thr, dp.image_w, dp.image_h = 0.01, 200, 0.0, 300, 300
        outs = ops.ssd_detect(conf, boxes, Cc, 1, 0.01, 200)
        score, anchor, cls, box, count = outs
        call = lambda: lib.ogle_cuda_ssd_detect(C.byref(dp), ops._p(conf), ops._p(boxes), ops._p(score),
                                                C.c_void_p(anchor.data_ptr()), C.c_void_p(cls.data_ptr()), ops._p(box),
                                                C.c_void_p(count.data_ptr()), ops._stream())
        med, best = timer(call)
        # logits (21 of 24 lanes are data) + boxes read once, results written once
        nbytes = 4.0 * (Nn * A * Cc + boxes.numel()) + 28.0 * score.numel()
        add("ssd_detect_per_class_top200_n1024", "fp32", "ssd_detect_kernel", med, best, 0.0, nbytes, None)

    status = lib.ogle_cuda_device_status()
    if status != 0:
        raise SystemExit("device status %d after the sweep" % status)

    print("\n| op | mode | kernel | median us | best us | GB/s | % HBM | TFLOP/s | % tensor |")
    print("|---|---|---|---|---|---|---|---|---|")
    for r in rows:
        ft = "%.0f%%" % (100 * r["frac_tensor"]) if r["frac_tensor"] else "-"
        print("| %s | %s | `%s` | %.1f | %.1f | %.0f | %.0f%% | %s | %s |" % (
            r["op"], r["math_mode"], r["kernel"], r["us_median"], r["us_best"], r["gbs"], 100 * r["frac_hbm"],
            ("%.1f" % r["tflops"]) if r["gflop"] else "-", ft))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
