"""Benchmark of the OGLE hot path on B200: MobileNet-v1-SSD-300 fp32 images/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch B] [--math fp32|tf32|tf32x3] [--mode 0|1]

Workload (BASELINE.json configs[3]): MobileNet-v1-SSD 300x300, 21 classes, batch
256 per GPU, seeded random weights N(0,0.02) with identity BN folded, inputs
uniform [0,1] normalised (x-0.5)/0.5, seeded per image. One step = one batch
through the network, the SSD box decoder and the detection post-process.
Image-sharded: every rank runs its own batch, no collective on the data path.

Prints ONE JSON line (rank 0). `value` = device-resident images/s over all ranks;
`e2e` = the same through the Detector call with pinned HOST input and the
detections copied back, copies inside the timed region; `roofline` = the dominant
kernel family timed live with CUDA events; `cpu_baseline` = the CPU oracle on a
bounded sample of the same workload.

--impl reference times the reference's own arithmetic on the host cores instead
(its shaders compiled for the CPU where built, else the restatement).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "mobilenet_ssd300_fp32_images_per_s"
UNIT = "images/s"
MATH = {"fp32": 0, "tf32": 1, "tf32x3": 2}
# Dense TF32 throughput of this pool's B200 (torch.matmul fp32 with TF32 allowed, 8192^3,
# best of 10), measured once by profiles/ recipe; MEASURED_PEAKS.json holds bf16 and HBM only.
TF32_PEAK_TFLOPS_FALLBACK = None


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--classes", type=int, default=21)
    ap.add_argument("--math", default="tf32x3", choices=list(MATH))
    ap.add_argument("--mode", type=int, default=1, help="0 reference Detector rule, 1 per-class top-k")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--host-alloc", default="ogle", choices=["ogle", "torch"],
                    help="pinned input batches from ogle_host_alloc_pinned (2 MB pages, default) or torch's cudaHostAlloc")
    ap.add_argument("--no-host-binding", action="store_true",
                    help="leave this process's CPU affinity and memory policy alone (default: bind to the GPU's NUMA node)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the baseline sample")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def make_inputs(batch, seed0):
    """uniform [0,1] RGB normalised (x-0.5)/0.5, one seed per image."""
    import numpy as np
    x = np.empty((batch, 300, 300, 3), np.float32)
    for i in range(batch):
        x[i] = (np.random.default_rng(seed0 + i).random((300, 300, 3), dtype=np.float32) - 0.5) / 0.5
    return x


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 20 ms while the timed regions run."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def conv_costs(model, batch):
    """Per Conv node: (flops, algorithmic bytes) for `batch` images:
    2*N*Ho*Wo*K*(C/g)*k^2 and 4*(N*H*W*C + N*Ho*Wo*K + K*(C/g)*k^2 + K), unpadded channels."""
    shapes = {}
    costs = {}
    for n in model.nodes:
        if n.type == "Input":
            d = n.attr["input_attr"]["dims"]
            shapes[n.output_index[0]] = (d[2], d[3], d[1])
        elif n.type == "Conv":
            a = n.attr["conv2d_attr"]
            H, W, C = shapes[n.input_index[0]]
            wnode = next(m for m in model.nodes if m.output_index[0] == n.input_index[1])
            K, Cg, k, _ = wnode.attr["const_attr"]["value"].dims
            s, p = a["strides"][0], a["pads"][0]
            Ho, Wo = (H - k + 2 * p) // s + 1, (W - k + 2 * p) // s + 1
            shapes[n.output_index[0]] = (Ho, Wo, K)
            flops = 2 * batch * Ho * Wo * K * Cg * k * k
            byts = 4 * (batch * H * W * C + batch * Ho * Wo * K + K * Cg * k * k + K)
            costs[n.name] = (flops, byts)
    return costs


def cpu_baseline(model_builder, classes, target_seconds, kind=None):
    """Times the CPU oracle on a bounded sample of the workload, all host threads."""
    import numpy as np
    from oracle import graph_oracle, oracle
    if kind is None:
        kind = "reference" if oracle.available("reference") else "port"
    lib = oracle.load(kind)
    keep = {"cls_logits", "box_preds", "anchors"}
    post = oracle.load("port")   # the post-process exists only in the restatement
    # every host core this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib.set_threads(cores)
    post.set_threads(cores)

    def run(n):
        model, _ = model_builder(n)
        x = make_inputs(n, 900000)
        t0 = time.perf_counter()
        out = graph_oracle.run_graph(model, {"input": x}, lib, keep=keep)
        boxes = lib.decode(out["box_preds"], out["anchors"])
        for i in range(n):
            post.topk_per_class(out["cls_logits"][i], 0.01, 200)
        return time.perf_counter() - t0, boxes

    t1, _ = run(1)
    n = int(max(2, min(64, target_seconds / max(t1, 1e-3))))
    t, _ = run(n)
    return {"value": n / t, "unit": UNIT, "cores": lib.threads(), "kind": kind,
            "sample": f"{n} images of the same workload (network + decode + per-class top-k) in {t:.1f} s"}


def run_reference(args, rank):
    if rank != 0:
        return
    from ogle_b200 import models
    builder = lambda n: models.mobilenet_v1_ssd(batch=n, num_classes=args.classes, seed=0, weight_std=0.02)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    # each step is a bounded sample; the whole run stays within a few minutes
    per_step = min(args.cpu_seconds, 120.0 / (steps + warm))
    vals, last = [], None
    for i in range(warm + steps):
        last = cpu_baseline(builder, args.classes, per_step)
        if i >= warm:
            vals.append(last["value"])
    v = sum(vals) / len(vals)
    last["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": 1000.0 * args.batch / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "MobileNet-v1-SSD-300 21 classes, CPU sample scaled to batch %d" % args.batch,
                   "global_batch": args.batch * args.gpus},
        "cpu_baseline": last, "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from ogle_b200 import models, ops, session

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    # one process per GPU: this process and the pinned buffers it uploads from belong on the GPU's NUMA node
    affinity0 = os.sched_getaffinity(0)
    placement = None if args.no_host_binding else session.bind_host_to_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    peaks = measured_peaks()

    model, info = models.mobilenet_v1_ssd(batch=B, num_classes=args.classes, seed=0, weight_std=0.02)
    tmp = tempfile.mkdtemp(prefix="ogle_bench_")
    path = os.path.join(tmp, "ssd.dlx")
    model.save(path)

    stream = torch.cuda.Stream()
    det = session.Detector(path, mode=args.mode, score_thr=0.01 if args.mode == 1 else 0.3,
                           top_k=200 if args.mode == 1 else 100, nms_thr=0.45, math_mode=MATH[args.math],
                           device=local_rank, stream=stream.cuda_stream)
    sess = det.session()

    # two different pinned host batches, alternated, so no step re-reads what the last left in L2
    def pinned(array):
        if args.host_alloc == "torch":
            return torch.from_numpy(array).pin_memory()
        buf = session.PinnedArray(array.shape, array.dtype)
        buf.array[...] = array
        pinned_buffers.append(buf)
        return torch.from_numpy(buf.array)

    pinned_buffers = []
    host = [pinned(make_inputs(B, 1000 * (rank + 1) + j * B)) for j in range(2)]
    det.detect_async(host[0].data_ptr(), B, 300, 300)   # sizes the session (weight packing included); eager pass
    det.wait(fetch=False)
    launches0 = ops.launch_count()
    det.detect_async(host[1].data_ptr(), B, 300, 300)   # captures the CUDA graph: every kernel of a step passes the counter once
    det.wait(fetch=False)
    launches_per_step = ops.launch_count() - launches0

    # device-resident inputs in the padded layout
    with torch.cuda.stream(stream):
        dev_in = [ops.upload(h.numpy()) for h in host]
    stream.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, drain=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        if drain:
            drain()     # host-blocks until the last result is in host memory, so e1 is stamped after it
        e1.record(stream)
        stream.synchronize()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    resident = lambda i: det.detect_device_async(dev_in[i & 1].data_ptr(), B, 300, 300, False)

    # the user-facing call pattern: keep two batches in flight, so the upload of batch i+1 and the
    # copy-back of batch i-1 overlap the network of batch i; every batch is uploaded from pinned
    # host memory and its detections are back on the host before the timed region ends
    def e2e_step(i):
        det.detect_async(host[i & 1].data_ptr(), B, 300, 300)
        if det.in_flight() == 2:
            det.wait(fetch=False)

    def e2e_drain():
        while det.in_flight():
            det.wait(fetch=False)

    for i in range(W):
        resident(i)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(resident, K)
    value = world * B * K / (ms / 1000.0)

    for i in range(W):
        e2e_step(i)
    e2e_drain()
    ms_e2e = timed(e2e_step, K, e2e_drain)
    clocks = sampler.stop()     # sampled across both timed regions
    inf = det.info()
    e2e = {"value": world * B * K / (ms_e2e / 1000.0), "unit": UNIT, "h2d_bytes_per_step": inf["h2d_bytes"],
           "d2h_bytes_per_step": inf["d2h_bytes"]}

    # the same pipeline fed the way the reference's Detector::Detect is (8-bit BGR frames; resize and
    # mean subtraction on the device): a quarter of the upload bytes. Reported beside `e2e`, not in its place.
    frames = [pinned(torch.randint(0, 256, (B, 300, 300, 3), dtype=torch.uint8,
                                   generator=torch.Generator().manual_seed(7000 + 10 * rank + j)).numpy()) for j in range(2)]

    def frames_step(i):
        det.detect_bgr8_frames_async(frames[i & 1].data_ptr(), B, 300, 300, 300, 300)
        if det.in_flight() == 2:
            det.wait(fetch=False)

    for i in range(W):
        frames_step(i)
    e2e_drain()
    ms_frames = timed(frames_step, K, e2e_drain)
    inf8 = det.info()
    e2e_frames = {"value": world * B * K / (ms_frames / 1000.0), "unit": UNIT, "input": "8-bit BGR frames 300x300",
                  "h2d_bytes_per_step": inf8["h2d_bytes"], "d2h_bytes_per_step": inf8["d2h_bytes"]}

    # roofline of the dominant kernel family, timed live: eager passes with an event pair per node
    roof = None
    if rank == 0:
        costs = conv_costs(model, B)
        fam = {}
        reps = 3
        for _ in range(reps):
            for name, type_, kernel, t_ms in sess.Profile({"input": host[0].numpy()}):
                # conv nodes report "family:device kernel"; group by the device kernel
                key = kernel.split(":")[1] if ":" in kernel else kernel
                f = fam.setdefault(key, dict(ms=0.0, launches=0, flops=0, bytes=0))
                f["ms"] += t_ms
                f["launches"] += 1
                for part in name.split("+"):        # a fused sibling pair reports as "first+second"
                    if part in costs:
                        f["flops"] += costs[part][0]
                        f["bytes"] += costs[part][1]
        top = max((k for k in fam if fam[k]["bytes"] > 0), key=lambda k: fam[k]["ms"])
        f = fam[top]
        sec = f["ms"] / 1000.0
        gbs = f["bytes"] / sec / 1e9
        tfl = f["flops"] / sec / 1e12
        # TF32 runs at half the bf16 rate on these tensor cores; the 3-pass mode issues three
        # TF32 products per useful multiply-add
        tf32_peak = peaks["bf16_tflops_sustained"] / 2.0
        passes = {0: None, 1: 1, 2: 3}[MATH[args.math]]
        tensor_peak = tf32_peak / passes if passes else None
        hbm_frac = gbs / peaks["hbm_gbs"]
        ten_frac = tfl / tensor_peak if (tensor_peak and "tc" in top) else 0.0
        if ten_frac > hbm_frac:
            roof = {"bound": "tensor", "achieved": tfl, "peak": tensor_peak, "unit": "TFLOP/s", "frac": ten_frac,
                    "hbm_frac": hbm_frac}
        else:
            roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": hbm_frac}
        per_launch_bytes = f["bytes"] / f["launches"]
        roof.update({"kernel": top, "launches_per_step": f["launches"] // reps, "avg_launch_us": 1000.0 * f["ms"] / f["launches"],
                     "share_of_step": f["ms"] / sum(v["ms"] for v in fam.values()), "peak_source": peaks["source"],
                     # ncu (profiles/dram_traffic_*): DRAM bytes of a launch = 1.01 x its algorithmic bytes
                     "traffic": 1.01 * per_launch_bytes, "algorithmic_bytes_per_launch": per_launch_bytes,
                     "kernels": {k: {"ms_per_step": v["ms"] / reps, "launches": v["launches"] // reps,
                                     "GB/s": (v["bytes"] / (v["ms"] / 1000.0) / 1e9) if v["bytes"] else None,
                                     "TFLOP/s": (v["flops"] / (v["ms"] / 1000.0) / 1e12) if v["flops"] else None}
                                 for k, v in sorted(fam.items(), key=lambda kv: -kv[1]["ms"])}})

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        builder = lambda n: models.mobilenet_v1_ssd(batch=n, num_classes=args.classes, seed=0, weight_std=0.02)
        os.sched_setaffinity(0, affinity0)       # the CPU baseline uses every core this process was given
        cpu = cpu_baseline(builder, args.classes, args.cpu_seconds)

    graph_captured = sess.graph_captured()
    det.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "MobileNet-v1-SSD-300, %d classes, batch %d per GPU, image-sharded; network + SSD decode + %s"
                               % (args.classes, B, "per-class top-200 (thr 0.01)" if args.mode == 1 else "reference Detector rule"),
                   "global_batch": B * world, "math_mode": args.math, "gflop_per_image": info["flops_per_image"] / 1e9,
                   "l2": "inputs larger than L2 (%.0f MB per step, two batches alternated)" % (B * 300 * 300 * 16 / 1e6),
                   "parallelism": "image-sharded x%d, no collective" % world, "cuda_graph": graph_captured,
                   "host_placement": placement, "host_alloc": args.host_alloc},
        "e2e": e2e, "e2e_bgr8_frames": e2e_frames, "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step,
        "clocks": clocks, "roofline": roof, "cpu_baseline": cpu}), flush=True)


if __name__ == "__main__":
    main()
