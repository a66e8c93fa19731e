"""One batch, image-sharded over the GPUs of one box: one process (session, streams, CUDA graph)
per GPU, no collective and no peer access on the data path.

The reference's Detector::Detect serves one frame in one process
(ogl_runtime/opengl/examples/ssd/detector.cc:275-295 in kl456123/OGLE). Here the process that
owns a batch (rank 0) writes the images ONCE into host memory shared by all ranks; every rank
uploads its contiguous block of images straight from that memory, runs it, and its GPU copies the
detections straight back into a shared result region at that rank's offset. Rank 0 then reads
all detections in place, in image order. The only traffic between processes is a handful of
sequence counters in a shared control block, which also tell rank 0 when a rank has stopped
answering (ShardTimeout) or has reported a failure (ShardFailed).

ShardedBatch is the host-side part (regions, counters, scatter/gather bookkeeping) and needs no
GPU; ShardedDetector adds the per-rank Detector.
"""
import ctypes as C
import os
import time

import numpy as np

from ._lib import OgleError


def shard_range(n_images, rank, world):
    """Contiguous block [lo, hi) of image indices owned by `rank`; sizes differ by at most one."""
    base, rem = divmod(n_images, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def gather_detections(local, lo, group=None, dst=0):
    """local: list of per-image detection records for images lo, lo+1, ... of this rank.
    Returns on `dst` the list for ALL images in image order (None elsewhere). Uses the
    object gather of the given (CPU-capable, e.g. gloo) process group: the portable path for
    ranks that share no memory; ShardedBatch is the in-place one for ranks of one box."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    payload = (lo, local)
    out = [None] * world if rank == dst else None
    dist.gather_object(payload, out, dst=dst, group=group)
    if rank != dst:
        return None
    merged = {}
    for start, items in out:
        for i, item in enumerate(items):
            if start + i in merged:
                raise ValueError(f"image {start + i} reported by two ranks")
            merged[start + i] = item
    return [merged[i] for i in sorted(merged)]


def max_over_ranks(value, group=None):
    """Slowest rank's value (timings are reported as the max over ranks)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class ShardTimeout(OgleError):
    """A rank did not report a step within the time allowed. `.ranks` lists the silent ones."""

    def __init__(self, what, ranks):
        super().__init__(f"{what}: no answer from rank(s) {ranks}")
        self.ranks = list(ranks)


class ShardFailed(OgleError):
    """A rank reported that it cannot serve its shard. `.ranks` lists them."""

    def __init__(self, ranks):
        super().__init__(f"rank(s) {ranks} reported a failure")
        self.ranks = list(ranks)


def result_layout(mode, num_classes, top_k, n_images):
    """Byte offsets inside one Detector result block: dict(score, anchor, cls, box, count, total, rows, counts_per_image)."""
    from . import session
    off = (C.c_size_t * 6)()
    rows, cpi = C.c_int(), C.c_int()
    if session.rt_lib().ogle_detector_result_layout(mode, num_classes, top_k, n_images, off, C.byref(rows), C.byref(cpi)) != 0:
        raise OgleError("result_layout: bad arguments")
    return dict(score=off[0], anchor=off[1], cls=off[2], box=off[3], count=off[4], total=off[5], rows=rows.value,
                counts_per_image=cpi.value)


class SharedRegion:
    """Named host memory shared by the ranks of one box (ogle_host_shared_open). pin=True registers it with CUDA
    in this process. Views returned by view() die with close()."""

    def __init__(self, name, nbytes, create, pin):
        from . import session
        self._lib = session.rt_lib()
        self.name, self.nbytes = name, int(nbytes)
        self.ptr = self._lib.ogle_host_shared_open(name.encode(), self.nbytes, int(bool(create)), int(bool(pin)))
        if not self.ptr:
            raise OgleError(f"shared region {name}: {self._lib.ogle_rt_last_error().decode()}")
        self._buf = (C.c_char * self.nbytes).from_address(self.ptr)

    def view(self, offset, shape, dtype):
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        if offset < 0 or offset + n > self.nbytes:
            raise ValueError("view outside the region")
        return np.frombuffer(self._buf, dtype=dtype, count=int(np.prod(shape)), offset=offset).reshape(shape)

    def huge_page_bytes(self):
        return int(self._lib.ogle_host_huge_page_bytes(self.ptr))

    def close(self, unlink=False):
        if getattr(self, "ptr", None):
            self._buf = None
            self._lib.ogle_host_shared_close(self.ptr, int(bool(unlink)))
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _round_up(v, m):
    return (v + m - 1) // m * m


class ShardedBatch:
    """Regions and counters for one image-sharded batch stream.

    Two slots alternate by step parity, so that step s+1 can be written and uploaded while step s
    is still being computed or read. Per step:
      owner  : fill input_slot(s), publish(s)
      ranks  : wait_input(s) -> upload own images -> ... -> report(s) once the detections of the
               rank are in result_block(s, rank)
      owner  : gather(s) -> read views -> release(s)
    A rank may start step s only when the owner has released step s-2 (wait_input checks it)."""

    LINE = 64      # counters live on separate cache lines

    def __init__(self, tag, global_batch, image_shape, rank, world, mode, num_classes, top_k, pin=True, barrier=None,
                 owner=0, with_frames=False):
        self.rank, self.world, self.owner, self.global_batch = rank, world, owner, int(global_batch)
        self.image_shape = tuple(int(d) for d in image_shape)            # (H, W, channels) of one image, fp32
        self.mode, self.num_classes, self.top_k = mode, num_classes, top_k
        self.ranges = [shard_range(self.global_batch, r, world) for r in range(world)]
        self.layouts = [result_layout(mode, num_classes, top_k, max(hi - lo, 1)) for lo, hi in self.ranges]
        self.block_offset, off = [], 0
        for L in self.layouts:
            self.block_offset.append(off)
            off += _round_up(L["total"], 4096)
        self.slot_bytes = off
        self.image_bytes = int(np.prod(self.image_shape)) * 4
        self.input_slot_bytes = _round_up(self.global_batch * self.image_bytes, 4096)
        # optional second input region: the same batch as 8-bit frames (what Detector::Detect is given,
        # detector.cc:275-295), a quarter of the bytes; a step is fed from one region or the other
        self.frame_bytes = int(np.prod(self.image_shape))
        self.frame_slot_bytes = _round_up(self.global_batch * self.frame_bytes, 4096)
        uid = os.getuid() if hasattr(os, "getuid") else 0
        base = f"/ogle_{uid}_{tag}"
        create = rank == owner
        if not create and barrier:
            barrier()                                  # the owner creates first
        self.inputs = SharedRegion(base + "_in", 2 * self.input_slot_bytes, create, pin)
        self.frames = SharedRegion(base + "_u8", 2 * self.frame_slot_bytes, create, pin) if with_frames else None
        self.results = SharedRegion(base + "_out", 2 * self.slot_bytes, create, pin)
        self.control = SharedRegion(base + "_ctl", self.LINE * (world + 2), create, False)
        if create and barrier:
            barrier()
        words = self.LINE // 8
        ctl = self.control.view(0, ((world + 2) * words,), np.int64)
        self._input_seq = ctl[0:1]                                   # last step published by the owner
        self._released = ctl[words:words + 1]                        # last step the owner has finished reading
        self._done = [ctl[(2 + r) * words:(2 + r) * words + 1] for r in range(world)]   # last step reported per rank
        if create:
            self._input_seq[0] = -1
            self._released[0] = -1
            for d in self._done:
                d[0] = -1
        if barrier:
            barrier()                                  # every rank has opened; counters are initialised
        self._opened_by_all = barrier is not None

    # ---- layout
    def local_range(self, rank=None):
        return self.ranges[self.rank if rank is None else rank]

    def input_slot(self, step):
        """The whole batch of step `step`: float32 [global_batch, H, W, channels] (the owner fills it)."""
        return self.inputs.view((step & 1) * self.input_slot_bytes, (self.global_batch,) + self.image_shape, np.float32)

    def local_input_ptr(self, step):
        lo, _ = self.local_range()
        return self.inputs.ptr + (step & 1) * self.input_slot_bytes + lo * self.image_bytes

    def frame_slot(self, step):
        """The whole batch of step `step` as 8-bit frames: uint8 [global_batch, H, W, channels] (with_frames=True)."""
        return self.frames.view((step & 1) * self.frame_slot_bytes, (self.global_batch,) + self.image_shape, np.uint8)

    def local_frame_ptr(self, step):
        lo, _ = self.local_range()
        return self.frames.ptr + (step & 1) * self.frame_slot_bytes + lo * self.frame_bytes

    def result_ptr(self, slot, rank=None):
        return self.results.ptr + slot * self.slot_bytes + self.block_offset[self.rank if rank is None else rank]

    def result_block(self, step, rank):
        """Views into rank `rank`'s detections of step `step`: dict(score, anchor, cls, box, count)."""
        lo, hi = self.ranges[rank]
        n, L = hi - lo, self.layouts[rank]
        base = (step & 1) * self.slot_bytes + self.block_offset[rank]
        rows = L["rows"]
        return dict(score=self.results.view(base + L["score"], (n, rows), np.float32),
                    anchor=self.results.view(base + L["anchor"], (n, rows), np.int32),
                    cls=self.results.view(base + L["cls"], (n, rows), np.int32),
                    box=self.results.view(base + L["box"], (n, rows, 4), np.float32),
                    count=self.results.view(base + L["count"], (n, L["counts_per_image"]), np.int32))

    # ---- counters
    @staticmethod
    def _wait(cond, timeout, what, who):
        t0 = time.monotonic()
        spins = 0
        while not cond():
            spins += 1
            if spins > 2000:
                time.sleep(0.0002)                     # yield the core after a short busy wait
            if time.monotonic() - t0 > timeout:
                raise ShardTimeout(what, who())
        return True

    def publish(self, step):
        """Owner: the images of `step` are in input_slot(step)."""
        self._input_seq[0] = step

    def wait_input(self, step, timeout=30.0):
        """Any rank: block until the owner has published `step` and released step-2 (whose slots `step` reuses)."""
        self._wait(lambda: self._input_seq[0] >= step and self._released[0] >= step - 2, timeout,
                   f"waiting for the images of step {step}", lambda: [self.owner])

    def report(self, step):
        """This rank's detections of `step` are in its result block."""
        self._done[self.rank][0] = step

    def fail(self):
        """This rank cannot go on (raised an exception, lost its device): the owner's gather raises ShardFailed."""
        self._done[self.rank][0] = -2

    def gather(self, step, timeout=30.0, merged=False):
        """Owner: block until every rank has reported `step`; returns per-rank view dicts in rank (= image) order, or
        with merged=True one dict of arrays over all images (a copy). Raises ShardFailed / ShardTimeout."""
        def ready():
            bad = [r for r in range(self.world) if self._done[r][0] == -2]
            if bad:
                raise ShardFailed(bad)
            return all(self._done[r][0] >= step for r in range(self.world))
        self._wait(ready, timeout, f"gathering step {step}", lambda: [r for r in range(self.world) if self._done[r][0] < step])
        blocks = [self.result_block(step, r) for r in range(self.world) if self.ranges[r][1] > self.ranges[r][0]]
        if not merged:
            return blocks
        return {k: np.concatenate([b[k] for b in blocks], axis=0) for k in blocks[0]}

    def release(self, step):
        """Owner: done reading the detections of `step`; its slots may be reused by step+2."""
        self._released[0] = step

    def close(self):
        unlink = self.rank == self.owner
        for region in (self.inputs, self.frames, self.results, self.control):
            if region is not None:
                region.close(unlink=unlink)


class ShardedDetector:
    """The per-rank half of an image-sharded SSD detector: a Detector sized for this rank's block of images, fed
    from and reporting into a ShardedBatch. Every rank of the box constructs one (same arguments, its own rank
    and device); `barrier` is a callable that returns once all ranks have reached it (e.g. torch.distributed's
    barrier on a gloo or nccl group) and orders the creation of the shared regions.

    model_path is the dlx model for THIS rank's shard size (dlx files carry their batch size in the input
    dims, as the converter writes them)."""

    def __init__(self, model_path, global_batch, rank, world, tag, num_classes, image_hw=(300, 300), mode=1,
                 score_thr=0.01, top_k=200, nms_thr=0.45, math_mode=-1, device=-1, stream=None, barrier=None,
                 with_frames=False):
        from . import session
        self.batch = ShardedBatch(tag, global_batch, (image_hw[0], image_hw[1], 3), rank, world, mode, num_classes, top_k,
                                  pin=True, barrier=barrier, with_frames=with_frames)
        lo, hi = self.batch.local_range()
        self.local = hi - lo
        self.H, self.W = image_hw
        self.det = None
        if self.local > 0:
            self.det = session.Detector(model_path, mode=mode, score_thr=score_thr, top_k=top_k, nms_thr=nms_thr,
                                        math_mode=math_mode, device=device, stream=stream)
            L = self.batch.layouts[rank]
            session._check(session.rt_lib().ogle_detector_use_result_buffers(
                self.det._h, self.batch.result_ptr(0), self.batch.result_ptr(1), L["total"]), "use_result_buffers")
            self._slot = 0          # the detector alternates its two result slots call by call
        self._pending = []

    def submit(self, step, timeout=30.0, frames=False):
        """Upload and run this rank's images of `step` (asynchronous; at most two steps in flight). frames=True:
        the step was published as 8-bit BGR frames of the network's input size (frame_slot); they are uploaded as
        bytes and converted on the device (BGR -> RGB, float, mean subtraction), as Detector::Detect does on the host."""
        self.batch.wait_input(step, timeout)
        if self.det is not None:
            if (step & 1) != self._slot:
                raise OgleError("steps must be submitted in order, starting with an even step")
            if frames:
                self.det.detect_bgr8_frames_async(self.batch.local_frame_ptr(step), self.local, self.H, self.W, self.H, self.W)
            else:
                self.det.detect_async(self.batch.local_input_ptr(step), self.local, self.H, self.W)
            self._slot ^= 1
        self._pending.append(step)

    def in_flight(self):
        return len(self._pending)

    def retire(self):
        """Block until the oldest submitted step's detections are in the shared result region, then report it."""
        step = self._pending.pop(0)
        if self.det is not None:
            self.det.wait(fetch=False)
        self.batch.report(step)
        return step

    def close(self):
        if self.det is not None:
            self.det.close()
            self.det = None
        self.batch.close()
