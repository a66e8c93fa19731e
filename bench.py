"""Benchmark of the OGLE hot path on B200: MobileNet-v1-SSD-300 fp32 images/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--global-batch G] [--math fp32|tf32|tf32x3] [--mode 0|1]

Workload (the benchmark configuration "batch 256, image-sharded across 1/2/4/8 B200"):
MobileNet-v1-SSD 300x300, 21 classes, ONE batch of 256 images per step split by image over
the N ranks (256 / 128 / 64 / 32 images per GPU), seeded random weights N(0,0.02) with
identity BN folded, inputs uniform [0,1] normalised (x-0.5)/0.5, seeded per image. One step
= the batch through the network, the SSD box decoder and the detection post-process.
No collective on the data path: rank 0 writes the batch into host memory shared by the
ranks, every rank uploads its block of images from there, and every rank's GPU copies its
detections into a shared result region where rank 0 reads all of them (ogle_b200/sharding.py).

Prints ONE JSON line (rank 0):
  value     images/s with each rank's images already resident on its GPU ("scaling": "strong");
  e2e       the same through the sharded Detector call with the batch in HOST memory as 8-bit BGR
            frames (what the reference's Detector::Detect is given): uploads, conversion on the
            device, copy-back of the detections and rank 0's gather inside the timed region;
  e2e_fp32_tensors  the same with the batch as fp32 tensors (what FBOSession::Run is given:
            four times the upload bytes);
  h2d_only  the bare upload of the fp32 bytes from the same buffers, for reading that against;
  roofline  the dominant kernel timed live with CUDA events, its tensor-bound and HBM-bound
            layers reported as two families;
  weak_256_per_gpu  (N > 1) the figure with 256 images on EVERY GPU instead;
  latency_b1        (N = 1) the batch-1, 2-class configuration: microseconds per image;
  cpu_baseline      (N = 1) the CPU oracle on a bounded sample of the same workload.

--impl reference times the reference's own arithmetic on the host cores instead
(its shaders compiled for the CPU where built, else the restatement).
--peaks-only prints the dense TF32 throughput of the GPU (a library GEMM, the roofline's
cross-check) and exits.
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
# Tensor-core passes of equal cost that one useful multiply-add takes: one-pass TF32 = 1; the
# fp32-grade mode issues one TF32 pass plus one BF16 pass over a K-concatenated operand pair, and
# a BF16 instruction covers twice the reduction depth in the same time, so the pair costs 2.
PASSES_EQUIV = {"fp32": None, "tf32": 1, "tf32x3": 2}
# DRAM bytes of a conv_tc2_kernel launch over its algorithmic bytes, from one ncu capture of every
# launch of a step at 32 images (dram__bytes_read.sum + dram__bytes_write.sum), read on the layers
# whose tensors exceed L2: reads equal the input bytes within 1-2 %, nothing is re-read. Every
# tensor's leading dimension is the image index, so a launch over more images moves
# proportionally more bytes.
NCU_TRAFFIC_RATIO = {"conv_tc2_kernel": 1.01}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--global-batch", type=int, default=256, help="images per step over all GPUs")
    ap.add_argument("--batch", type=int, default=0, help="images per GPU per step (sets --global-batch = batch * gpus)")
    ap.add_argument("--classes", type=int, default=21)
    ap.add_argument("--math", default="tf32x3", choices=list(MATH))
    ap.add_argument("--mode", type=int, default=1, help="0 reference Detector rule, 1 per-class top-k")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the weak-scaling, batch-1 latency and 8-bit-frame legs")
    ap.add_argument("--no-host-binding", action="store_true",
                    help="leave this process's CPU affinity and memory policy alone (default: bind to the GPU's NUMA node)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the baseline sample")
    ap.add_argument("--peaks-only", action="store_true")
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


def tf32_peak(seconds=1.5):
    """Dense TF32 throughput of this GPU by a library GEMM (torch.matmul fp32 with TF32 allowed, 8192^3): best of
    10 (burst) and back to back for `seconds` (sustained). A cross-check of the roofline denominator only."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        for _ in range(3):
            a @ b
        torch.cuda.synchronize()
        best = 1e9
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(10):
            e0.record()
            a @ b
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        t0, count = time.time(), 0
        e0.record()
        while time.time() - t0 < seconds:
            for _ in range(10):
                a @ b
            count += 10
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        return {"burst_tflops": 2 * n ** 3 / best / 1e9, "sustained_tflops": 2 * n ** 3 * count / e0.elapsed_time(e1) / 1e9,
                "how": "torch.matmul fp32, TF32 allowed, 8192^3: best of 10 / back to back for %.1f s" % seconds}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 20 ms. The process is started ahead of the timed
    regions (it needs a few hundred ms to produce its first line); mark() is called when they begin and stop()
    when they end, and only the samples in between count. A region shorter than the sampling period can fall
    between two samples: then the last sample before it and the first after it are used, and "window" says so."""
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

    def wait_first(self, seconds=3.0):
        t0 = time.time()
        while self.proc and not self.rows and time.time() - t0 < seconds:
            time.sleep(0.01)

    def mark(self):
        self.first = len(self.rows)

    def stop(self):
        window = "timed regions"
        first = getattr(self, "first", 0)
        if self.proc and len(self.rows) <= first:
            time.sleep(0.05)                      # one more sample, taken right after the region
            window = "nearest samples before and after the timed regions"
            first = max(0, first - 1)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows[first:]:
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
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


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
    from oracle import graph_oracle, oracle
    if kind is None:
        kind = "reference" if oracle.available("reference") else "port"
    lib = oracle.load(kind)
    keep = {"cls_logits", "box_preds", "anchors"}
    post = oracle.load("port")   # per-class top-k exists only in the restatement
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
    return {"value": n / t, "unit": UNIT, "cores": lib.threads(), "kind": kind, "sample_images": n, "sample_seconds": t,
            "sample": f"rate from a {n}-image sample of the same workload (network + decode + per-class top-k) that took {t:.1f} s"}


def run_reference(args, rank):
    if rank != 0:
        return
    from ogle_b200 import models
    builder = lambda n: models.mobilenet_v1_ssd(batch=n, num_classes=args.classes, seed=0, weight_std=0.02)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    # each step is a bounded sample; the whole run stays within a few minutes
    per_step = min(args.cpu_seconds, 120.0 / (steps + warm))
    vals, secs, last = [], [], None
    for i in range(warm + steps):
        last = cpu_baseline(builder, args.classes, per_step)
        if i >= warm:
            vals.append(last["value"])
            secs.append(last["sample_seconds"])
    v = sum(vals) / len(vals)
    last["value"] = v
    G = args.batch * args.gpus if args.batch else args.global_batch
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": 1000.0 * sum(secs) / len(secs), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "MobileNet-v1-SSD-300, %d classes; a step here is one %d-image CPU sample of the batch of %d "
                               "(the rate is measured on the sample, not extrapolated to steps that were not run)"
                               % (args.classes, last["sample_images"], G),
                   "global_batch": G, "images_per_timed_step": last["sample_images"]},
        "cpu_baseline": last, "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)


def classify_layers(rows, costs, peaks, passes_equiv):
    """Groups one profiled pass (name, type, kernel, ms) by device kernel; the tensor-core kernel's launches are
    further split by which floor of the layer is higher: flops / tensor peak or algorithmic bytes / HBM peak."""
    tensor_peak = peaks["bf16_tflops_sustained"] / 2.0 / passes_equiv if passes_equiv else None
    fam = {}
    for name, _type, kernel, t_ms in rows:
        key = kernel.split(":")[1] if ":" in kernel else kernel
        flops = sum(costs[p][0] for p in name.split("+") if p in costs)      # a fused sibling pair reports as "first+second"
        byts = sum(costs[p][1] for p in name.split("+") if p in costs)
        bound = None
        if byts:
            t_hbm = byts / (peaks["hbm_gbs"] * 1e9)
            t_ten = flops / (tensor_peak * 1e12) if (tensor_peak and "tc" in key) else 0.0
            bound = "tensor" if t_ten > t_hbm else "hbm"
        for k in ((key, None), (key, bound)) if bound else ((key, None),):
            f = fam.setdefault(k, dict(ms=0.0, launches=0, flops=0, bytes=0))
            f["ms"] += t_ms
            f["launches"] += 1
            f["flops"] += flops
            f["bytes"] += byts
    return fam, tensor_peak


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
    from ogle_b200 import models, ops, session, sharding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    if args.peaks_only:
        if rank == 0:
            print(json.dumps({"tf32_peak": tf32_peak(4.0), "measured_peaks": measured_peaks()}), flush=True)
        return
    # one process per GPU: this process and the pinned buffers it uploads from belong on the GPU's NUMA node
    affinity0 = os.sched_getaffinity(0)
    placement = None if args.no_host_binding else session.bind_host_to_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    G = args.batch * world if args.batch else args.global_batch
    K, W = args.steps, max(args.warmup, 3)
    lo, hi = sharding.shard_range(G, rank, world)
    B = hi - lo
    if B == 0:
        raise SystemExit("fewer images than ranks")
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ms(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    tmp = tempfile.mkdtemp(prefix="ogle_bench_")
    builder = lambda n, c=args.classes: models.mobilenet_v1_ssd(batch=n, num_classes=c, seed=0, weight_std=0.02)

    def dlx_for(n, c=args.classes):
        model, info = builder(n, c)
        path = os.path.join(tmp, "ssd_%d_%d.dlx" % (n, c))
        model.save(path)
        return model, info, path

    model, info, path = dlx_for(B)
    stream = torch.cuda.Stream()
    thr, topk = (0.01, 200) if args.mode == 1 else (0.3, 100)
    tag = "bench_%s" % os.environ.get("MASTER_PORT", str(os.getpid()))
    sd = sharding.ShardedDetector(path, G, rank, world, tag, args.classes, (300, 300), mode=args.mode, score_thr=thr,
                                  top_k=topk, nms_thr=0.45, math_mode=MATH[args.math], device=local_rank,
                                  stream=stream.cuda_stream, barrier=(dist.barrier if world > 1 else None),
                                  with_frames=True)
    det, sb = sd.det, sd.batch
    sess = det.session()

    # two different host batches, alternated, so no step re-reads what the last left in L2; rank 0 writes each once
    if rank == 0:
        for j in range(2):
            sb.input_slot(j)[...] = make_inputs(G, 1000 + j * G)
            sb.frame_slot(j)[...] = torch.randint(0, 256, (G, 300, 300, 3), dtype=torch.uint8,
                                                  generator=torch.Generator().manual_seed(7000 + j)).numpy()
    barrier()
    step_no = [0]
    feed_frames = [False]      # which host input the steps are fed from: fp32 tensors or 8-bit frames

    def sharded_step(_i):
        s = step_no[0]
        step_no[0] += 1
        if rank == 0:
            sb.publish(s)
        sd.submit(s, frames=feed_frames[0])
        if sd.in_flight() == 2:
            done = sd.retire()
            if rank == 0:
                sb.gather(done)        # every rank's detections of that step are on the host, in image order
                sb.release(done)

    def sharded_drain():
        while sd.in_flight():
            done = sd.retire()
            if rank == 0:
                sb.gather(done)
                sb.release(done)

    sharded_step(0)                     # sizes the session (weight packing included); eager pass
    sharded_drain()
    launches0 = ops.launch_count()
    sharded_step(1)                     # captures the CUDA graph: every kernel of a step passes the counter once
    sharded_drain()
    launches_per_step = ops.launch_count() - launches0

    # device-resident inputs in the padded layout: this rank's images of the two batches
    with torch.cuda.stream(stream):
        dev_in = [ops.upload(np.ascontiguousarray(sb.input_slot(j)[lo:hi])) for j in range(2)]
    stream.synchronize()

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
        return max_ms(e0.elapsed_time(e1))

    resident = lambda i: det.detect_device_async(dev_in[i & 1].data_ptr(), B, 300, 300, False)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(W):
        resident(i)
    sampler.wait_first()
    sampler.mark()
    ms = timed(resident, K)
    value = G * K / (ms / 1000.0)

    for i in range(W):
        sharded_step(i)
    sharded_drain()
    ms_e2e = timed(sharded_step, K, sharded_drain)

    def e2e_record(ms_region, what):
        inf = det.info()
        h2d = torch.tensor([float(inf["h2d_bytes"]), float(inf["d2h_bytes"])], device="cuda")
        if world > 1:
            dist.all_reduce(h2d)
        return {"value": G * K / (ms_region / 1000.0), "unit": UNIT, "h2d_bytes_per_step": int(h2d[0].item()),
                "d2h_bytes_per_step": int(h2d[1].item()), "ms_per_step": ms_region / K, "input": what,
                "gather": "rank 0 reads every rank's detections from shared pinned host memory"}

    e2e_fp32 = e2e_record(ms_e2e, "fp32 RGB tensors 300x300x3, mean already subtracted (what FBOSession::Run is given)")
    # the same steps fed the way the reference's Detector::Detect is: 8-bit BGR frames in host memory; colour order,
    # float conversion and mean subtraction run on the device. A quarter of the upload bytes.
    feed_frames[0] = True
    if step_no[0] & 1:
        sharded_step(0)         # steps alternate slots and start on an even one
        sharded_drain()
    for i in range(W):
        sharded_step(i)
    sharded_drain()
    ms_frames = timed(sharded_step, K, sharded_drain)
    clocks = sampler.stop()     # sampled across the timed regions
    e2e = e2e_record(ms_frames, "8-bit BGR frames 300x300 (what Detector::Detect is given)")
    feed_frames[0] = False

    # the bare upload of the same bytes from the same host buffers (no compute): the ceiling e2e can be read against
    rt = session.rt_lib()
    sink = torch.empty((B, 300, 300, 3), dtype=torch.float32, device="cuda")

    def upload_only(i):
        rt.ogle_host_upload_async(sink.data_ptr(), sb.local_input_ptr(i & 1), B * sb.image_bytes, stream.cuda_stream)

    for i in range(W):
        upload_only(i)
    ms_up = timed(upload_only, K)
    h2d_only = {"GB/s": G * sb.image_bytes * K / (ms_up / 1000.0) / 1e9, "images/s": G * K / (ms_up / 1000.0),
                "bytes_per_step": G * sb.image_bytes, "huge_page_bytes": sb.inputs.huge_page_bytes(),
                "buffer": "POSIX shared memory, cudaHostRegister'd in every rank"}
    del sink

    extras = {}

    # roofline of the dominant kernel, timed live: eager passes with an event pair per node
    roof = None
    if rank == 0:
        costs = conv_costs(model, B)
        reps = 3
        rows = []
        x_local = np.ascontiguousarray(sb.input_slot(0)[lo:hi])
        for _ in range(reps):
            rows += sess.Profile({"input": x_local})
        fam, tensor_peak = classify_layers(rows, costs, peaks, PASSES_EQUIV[args.math])
        whole = {k[0]: v for k, v in fam.items() if k[1] is None}
        top = max((k for k in whole if whole[k]["bytes"] > 0), key=lambda k: whole[k]["ms"])
        total_ms = sum(v["ms"] for v in whole.values())

        def describe(f, bound):
            sec = f["ms"] / 1000.0
            gbs, tfl = f["bytes"] / sec / 1e9, f["flops"] / sec / 1e12
            d = {"launches_per_step": f["launches"] // reps, "ms_per_step": f["ms"] / reps, "share_of_step": f["ms"] / total_ms,
                 "TFLOP/s": tfl, "GB/s": gbs, "hbm_frac": gbs / peaks["hbm_gbs"]}
            if tensor_peak:
                d["tensor_frac"] = tfl / tensor_peak
            d["frac"] = d["tensor_frac"] if (bound == "tensor" and tensor_peak) else d["hbm_frac"]
            return d

        families = {b: describe(fam[(top, b)], b) for b in ("tensor", "hbm") if (top, b) in fam}
        lead = max(families, key=lambda b: families[b]["ms_per_step"]) if families else "hbm"
        f = fam[(top, lead)] if families else whole[top]
        sec = f["ms"] / 1000.0
        per_launch_bytes = f["bytes"] / f["launches"]
        ratio = NCU_TRAFFIC_RATIO.get(top)
        if lead == "tensor" and tensor_peak:
            roof = {"bound": "tensor", "achieved": f["flops"] / sec / 1e12, "peak": tensor_peak, "unit": "TFLOP/s"}
        else:
            roof = {"bound": "hbm", "achieved": f["bytes"] / sec / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s"}
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof.update({
            "kernel": top, "family": "%s-bound layers of %s" % (lead, top), "launches_per_step": f["launches"] // reps,
            "avg_launch_us": 1000.0 * f["ms"] / f["launches"], "share_of_step": f["ms"] / total_ms,
            "peak_source": peaks["source"], "passes_equiv": PASSES_EQUIV[args.math],
            "peak_rule": "bf16_tflops_sustained / 2 (TF32 rate) / passes_equiv" if tensor_peak else None,
            "traffic": ratio * per_launch_bytes if ratio else None, "algorithmic_bytes_per_launch": per_launch_bytes,
            "traffic_source": ("ncu capture at 32 images per launch, scaled by images: %.2f x algorithmic" % ratio) if ratio else None,
            "families": families,
            "kernels": {k: {"ms_per_step": v["ms"] / reps, "launches": v["launches"] // reps,
                            "GB/s": (v["bytes"] / (v["ms"] / 1000.0) / 1e9) if v["bytes"] else None,
                            "TFLOP/s": (v["flops"] / (v["ms"] / 1000.0) / 1e12) if v["flops"] else None}
                        for k, v in sorted(whole.items(), key=lambda kv: -kv[1]["ms"])}})

    graph_captured = sess.graph_captured()
    placed = sess.num_placed()
    sd.close()

    # ---- N > 1: the figure with 256 images on every GPU (weak scaling), as an extra key
    if world > 1 and not args.no_extras:
        _, _, path_w = dlx_for(G)
        det_w = session.Detector(path_w, mode=args.mode, score_thr=thr, top_k=topk, nms_thr=0.45, math_mode=MATH[args.math],
                                 device=local_rank, stream=stream.cuda_stream)
        host_w = [session.PinnedArray((G, 300, 300, 3), np.float32) for _ in range(2)]
        for j, h in enumerate(host_w):
            h.array[...] = make_inputs(G, 5000 * (rank + 1) + j * G)

        def weak_e2e(i):
            det_w.detect_async(host_w[i & 1].ptr, G, 300, 300)
            if det_w.in_flight() == 2:
                det_w.wait(fetch=False)

        def weak_drain():
            while det_w.in_flight():
                det_w.wait(fetch=False)

        for i in range(2):
            weak_e2e(i)
        weak_drain()
        with torch.cuda.stream(stream):
            dev_w = [ops.upload(h.array) for h in host_w]
        stream.synchronize()
        weak_res = lambda i: det_w.detect_device_async(dev_w[i & 1].data_ptr(), G, 300, 300, False)
        for i in range(W):
            weak_res(i)
        ms_w = timed(weak_res, K)
        for i in range(W):
            weak_e2e(i)
        weak_drain()
        ms_we = timed(weak_e2e, K, weak_drain)
        extras["weak_256_per_gpu"] = {"value": world * G * K / (ms_w / 1000.0), "e2e": world * G * K / (ms_we / 1000.0),
                                      "unit": UNIT, "global_batch": world * G, "ms_per_step": ms_w / K,
                                      "note": "every GPU runs its own batch of %d: N independent copies of the 1-GPU job" % G}
        det_w.close()
        del dev_w
        for h in host_w:
            h.close()

    # ---- N = 1: the batch-1, 2-class configuration (the reference's own setting): latency per image
    if world == 1 and rank == 0 and not args.no_extras:
        m1, _, path1 = dlx_for(1, 2)
        det1 = session.Detector(path1, mode=0, score_thr=0.3, top_k=100, nms_thr=0.45, math_mode=MATH[args.math],
                                device=local_rank, stream=stream.cuda_stream)
        pin1 = session.PinnedArray((1, 300, 300, 3), np.float32)
        pin1.array[...] = make_inputs(1, 77)
        for _ in range(5):
            det1.detect_async(pin1.ptr, 1, 300, 300)
            det1.wait(fetch=False)
        lat = []
        for _ in range(300):
            t0 = time.perf_counter()
            det1.detect_async(pin1.ptr, 1, 300, 300)       # upload, graph replay, decode, post-process, copy-back
            det1.wait(fetch=False)
            lat.append((time.perf_counter() - t0) * 1e6)
        with torch.cuda.stream(stream):
            dev1 = ops.upload(pin1.array)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dev_lat = []
        for _ in range(300):
            e0.record(stream)
            det1.detect_device_async(dev1.data_ptr(), 1, 300, 300, False)
            e1.record(stream)
            stream.synchronize()
            dev_lat.append(e0.elapsed_time(e1) * 1000.0)
        s1 = det1.session()
        per_kernel = {}
        for _ in range(3):
            for name, _t, kernel, t_ms in s1.Profile({"input": pin1.array}):
                key = kernel.split(":")[1] if ":" in kernel else kernel
                k = per_kernel.setdefault(key, [0, 0.0])
                k[0] += 1
                k[1] += t_ms * 1000.0 / 3
        lat.sort()
        dev_lat.sort()
        extras["latency_b1"] = {
            "workload": "MobileNet-v1-SSD-300, batch 1, 2 classes, reference Detector rule (thr 0.3, top-100, NMS 0.45)",
            "e2e_us_median": lat[len(lat) // 2], "e2e_us_p90": lat[int(len(lat) * 0.9)], "device_us_median": dev_lat[len(dev_lat) // 2],
            "n": len(lat), "launches_per_image": s1.num_active_kernels() + 2, "cuda_graph": s1.graph_captured(),
            "per_kernel_us_eager": {k: {"launches": v[0] // 3, "us": v[1]} for k, v in sorted(per_kernel.items(), key=lambda kv: -kv[1][1])},
            "note": "per_kernel_us_eager: one eager pass with an event pair per node (each pair adds a few us); "
                    "device_us_median: the whole step as one graph replay plus decode and post-process"}
        det1.close()
        pin1.close()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        os.sched_setaffinity(0, affinity0)       # the CPU baseline uses every core this process was given
        cpu = cpu_baseline(builder, args.classes, args.cpu_seconds)

    peak_check = tf32_peak() if (rank == 0 and world == 1 and not args.no_extras) else None
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "MobileNet-v1-SSD-300, %d classes, one batch of %d image-sharded over %d GPU(s) (%d per GPU); "
                               "network + SSD decode + %s"
                               % (args.classes, G, world, B, "per-class top-200 (thr 0.01)" if args.mode == 1 else "reference Detector rule"),
                   "global_batch": G, "images_per_gpu": B, "math_mode": args.math, "gflop_per_image": info["flops_per_image"] / 1e9,
                   "l2": "inputs larger than L2 (%.0f MB per GPU per step, two batches alternated)" % (B * 300 * 300 * 16 / 1e6),
                   "parallelism": "image-sharded x%d, no collective; host scatter/gather through shared pinned memory" % world,
                   "cuda_graph": graph_captured, "concat_inputs_written_in_place": placed, "host_placement": placement},
        "e2e": e2e, "e2e_fp32_tensors": e2e_fp32, "h2d_only": h2d_only, "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step,
        "clocks": clocks, "roofline": roof, "cpu_baseline": cpu, "tf32_peak_check": peak_check}
    line.update(extras)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
