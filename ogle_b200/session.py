"""Python front end of the C++ host runtime (libogle_rt.so, include/ogle_runtime.h):
FBOSession and Detector with the reference's call shapes
(ogl_runtime/opengl/core/fbo_session.h, examples/ssd/detector.h in kl456123/OGLE).
Everything here is a ctypes call into the native library; there is no fallback.
"""
import ctypes as C
import os

import numpy as np

from . import _lib
from ._lib import OgleError

_vp = C.c_void_p
_cp = C.c_char_p
_fpp = C.POINTER(C.POINTER(C.c_float))
_ipp = C.POINTER(C.POINTER(C.c_int))
_ip = C.POINTER(C.c_int)

RT_SYMBOLS = {
    "ogle_rt_last_error": (_cp, []),
    "ogle_rt_registered_kernels": (_cp, []),
    "ogle_session_create": (_vp, [C.c_int, _vp]),
    "ogle_session_destroy": (None, [_vp]),
    "ogle_session_set_option": (C.c_int, [_vp, _cp, C.c_int]),
    "ogle_session_load_graph_file": (C.c_int, [_vp, _cp]),
    "ogle_session_load_graph_bytes": (C.c_int, [_vp, _vp, C.c_size_t]),
    "ogle_session_run": (C.c_int, [_vp, C.c_int, C.POINTER(_cp), _fpp, _ipp, _ip, _ip]),
    "ogle_session_run_device": (C.c_int, [_vp, C.c_int, C.POINTER(_cp), C.POINTER(_vp)]),
    "ogle_session_synchronize": (C.c_int, [_vp]),
    "ogle_session_tensor_info": (C.c_int, [_vp, _cp, _ip, _ip, _ip, C.POINTER(_vp)]),
    "ogle_session_get_output": (C.c_int, [_vp, _cp, _cp, _vp, C.c_size_t]),
    "ogle_session_num_active_kernels": (C.c_int, [_vp]),
    "ogle_session_num_placed": (C.c_int, [_vp]),
    "ogle_session_num_residuals": (C.c_int, [_vp]),
    "ogle_session_num_branches": (C.c_int, [_vp]),
    "ogle_session_graph_captured": (C.c_int, [_vp]),
    "ogle_session_device_bytes": (C.c_size_t, [_vp]),
    "ogle_session_profile": (C.c_int, [_vp, C.c_int, C.POINTER(_cp), _fpp, _ipp, _ip, _ip, _cp, C.c_size_t]),
    "ogle_detector_create": (_vp, [C.c_int, _vp, _cp, C.c_int, C.c_float, C.c_int, C.c_float, C.c_int, _cp, _cp, _cp, _cp]),
    "ogle_detector_destroy": (None, [_vp]),
    "ogle_detector_detect_async": (C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int]),
    "ogle_detector_detect_device_async": (C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    "ogle_detector_detect_bgr8_async": (C.c_int, [_vp, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int,
                                                  C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "ogle_detector_wait": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "ogle_detector_info": (C.c_int, [_vp, _ip, _ip, _ip, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "ogle_detector_session": (_vp, [_vp]),
    "ogle_rt_plan_streams": (C.c_int, [C.c_int, C.c_int, _ip, C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), _ip, C.c_int,
                                       _ip, C.POINTER(C.c_ubyte)]),
    "ogle_host_alloc_pinned": (_vp, [C.c_size_t]),
    "ogle_host_free_pinned": (None, [_vp]),
    "ogle_host_huge_page_bytes": (C.c_size_t, [_vp]),
    "ogle_host_shared_open": (_vp, [_cp, C.c_size_t, C.c_int, C.c_int]),
    "ogle_host_shared_close": (None, [_vp, C.c_int]),
    "ogle_host_upload_async": (C.c_int, [_vp, _vp, C.c_size_t, _vp]),
    "ogle_detector_use_result_buffers": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "ogle_detector_result_layout": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_size_t), _ip, _ip]),
    "ogle_host_bind_to_device": (C.c_int, [C.c_int, _ip, _ip, _ip]),
    "ogle_host_parse_cpulist": (C.c_int, [_cp, _ip, C.c_int]),
}

_rt = None


def rt_lib():
    global _rt
    if _rt is None:
        _lib.cuda_lib()
        if not os.path.exists(_lib.RT_LIB_PATH):
            raise RuntimeError(f"{_lib.RT_LIB_PATH} is missing: build it with `python -m ogle_b200.build`.")
        lib = C.CDLL(_lib.RT_LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in RT_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _rt = lib
    return _rt


def _check(rc, what):
    if rc != 0:
        raise OgleError(f"{what}: {rt_lib().ogle_rt_last_error().decode()}")


def bind_host_to_device(device):
    """Pins the calling thread to the CPUs of the GPU's NUMA node and makes its later host
    allocations (pinned buffers included) prefer that node. Call before allocating the buffers
    that feed the device. Returns {"numa_node", "cpus_bound", "memory_preferred"}."""
    node, cpus, mem = C.c_int(-1), C.c_int(0), C.c_int(0)
    rt_lib().ogle_host_bind_to_device(int(device), C.byref(node), C.byref(cpus), C.byref(mem))
    return {"numa_node": node.value, "cpus_bound": cpus.value, "memory_preferred": bool(mem.value)}


class PinnedArray:
    """numpy view of pinned host memory from ogle_host_alloc_pinned (2 MB pages where the host grants them).
    Keep the object alive while views of .array are in use; close() (or deletion) releases the memory."""

    def __init__(self, shape, dtype=np.float32):
        self.shape = tuple(int(d) for d in shape)
        self.nbytes = int(np.prod(self.shape)) * np.dtype(dtype).itemsize
        self.ptr = rt_lib().ogle_host_alloc_pinned(self.nbytes)
        if not self.ptr:
            raise OgleError("ogle_host_alloc_pinned(%d) failed" % self.nbytes)
        buf = (C.c_char * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dtype).reshape(self.shape)

    def close(self):
        if getattr(self, "ptr", None):
            self.array = None
            rt_lib().ogle_host_free_pinned(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def plan_streams(nodes, streams):
    """The session's stream planner on its own. nodes: list of (reads, writes), each a list of (lo, hi) spans.
    Returns (lanes, waits, branches): waits[i] = nodes on other streams that node i waits for."""
    n = len(nodes)
    rec = [(i, lo, hi, w) for i, (rd, wr) in enumerate(nodes) for (spans, w) in ((rd, 0), (wr, 1)) for (lo, hi) in spans]
    m = len(rec)
    node = (C.c_int * max(m, 1))(*[r[0] for r in rec])
    lo = (C.c_ulonglong * max(m, 1))(*[r[1] for r in rec])
    hi = (C.c_ulonglong * max(m, 1))(*[r[2] for r in rec])
    wr = (C.c_int * max(m, 1))(*[r[3] for r in rec])
    lane = (C.c_int * max(n, 1))()
    waits = (C.c_ubyte * max(n * n, 1))()
    branches = rt_lib().ogle_rt_plan_streams(n, m, node, lo, hi, wr, streams, lane, waits)
    if branches < 0:
        raise OgleError("plan_streams: bad arguments")
    return list(lane[:n]), [[j for j in range(n) if waits[i * n + j]] for i in range(n)], branches


def parse_cpulist(text):
    buf = (C.c_int * 4096)()
    n = rt_lib().ogle_host_parse_cpulist(text.encode(), buf, 4096)
    return list(buf[:min(n, 4096)])


def registered_kernels():
    return rt_lib().ogle_rt_registered_kernels().decode().split()


_FORMATS = {"NCHW": 0, "NHWC": 1, "NHWC4": 3, "HWN4C4": 4, "ANY": 5, "ANY4": 6}


def _pack_inputs(inputs):
    """inputs: {name: (array, dformat_str)} or {name: array (NHWC)} -> ctypes argument arrays."""
    names, arrays, fmts = [], [], []
    for k, v in inputs.items():
        arr, fmt = v if isinstance(v, tuple) else (v, "NHWC" if np.ndim(v) == 4 else "ANY")
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        names.append(k.encode())
        arrays.append(arr)
        fmts.append(_FORMATS[fmt])
    n = len(names)
    c_names = (_cp * n)(*names)
    c_data = (C.POINTER(C.c_float) * n)(*[a.ctypes.data_as(C.POINTER(C.c_float)) for a in arrays])
    shape_arrays = [(C.c_int * a.ndim)(*a.shape) for a in arrays]
    c_shapes = (C.POINTER(C.c_int) * n)(*[C.cast(s, C.POINTER(C.c_int)) for s in shape_arrays])
    c_ranks = (C.c_int * n)(*[a.ndim for a in arrays])
    c_fmts = (C.c_int * n)(*fmts)
    return n, c_names, c_data, c_shapes, c_ranks, c_fmts, (arrays, shape_arrays)


class FBOSession:
    def __init__(self, device=-1, stream=None, _borrowed=None):
        self._lib = rt_lib()
        self._owned = _borrowed is None
        self._keep = None
        if _borrowed is not None:
            self._h = _borrowed
        else:
            self._h = self._lib.ogle_session_create(device, stream)
            if not self._h:
                raise OgleError("session_create: " + self._lib.ogle_rt_last_error().decode())

    def close(self):
        if self._h and self._owned:
            self._lib.ogle_session_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_option(self, key, value):
        _check(self._lib.ogle_session_set_option(self._h, key.encode(), int(value)), "set_option")

    def LoadGraph(self, model):
        """model: path to a .dlx file, raw bytes, or an ogle_b200.dlx.Model."""
        if isinstance(model, str):
            _check(self._lib.ogle_session_load_graph_file(self._h, model.encode()), "LoadGraph")
        else:
            data = model if isinstance(model, (bytes, bytearray)) else model.encode()
            buf = C.create_string_buffer(bytes(data), len(data))
            _check(self._lib.ogle_session_load_graph_bytes(self._h, buf, len(data)), "LoadGraph")

    def Run(self, inputs):
        n, names, data, shapes, ranks, fmts, keep = _pack_inputs(inputs)
        self._keep = keep   # host buffers stay alive until the next call
        _check(self._lib.ogle_session_run(self._h, n, names, data, shapes, ranks, fmts), "Run")

    def RunDevice(self, inputs):
        """inputs: {name: device pointer (int)} already in the padded device layout."""
        n = len(inputs)
        names = (_cp * n)(*[k.encode() for k in inputs])
        ptrs = (_vp * n)(*[int(v) for v in inputs.values()])
        _check(self._lib.ogle_session_run_device(self._h, n, names, ptrs), "RunDevice")

    def synchronize(self):
        _check(self._lib.ogle_session_synchronize(self._h), "synchronize")

    def tensor_info(self, name):
        shape = (C.c_int * 8)()
        rank, fmt, ptr = C.c_int(), C.c_int(), _vp()
        _check(self._lib.ogle_session_tensor_info(self._h, name.encode(), shape, C.byref(rank), C.byref(fmt), C.byref(ptr)),
               "tensor_info")
        return list(shape[:rank.value]), fmt.value, ptr.value

    def GetOutputs(self, names, dformats):
        outs = []
        for name, f in zip(names, dformats):
            shape, _, _ = self.tensor_info(name)
            if f in ("NHWC4", "ANY4"):
                hshape = shape[:-1] + [(shape[-1] + 3) // 4 * 4]
            else:
                hshape = shape
            n = int(np.prod(hshape, dtype=np.int64))
            buf = np.empty(max((n + 3) // 4 * 4, 4), np.float32)
            _check(self._lib.ogle_session_get_output(self._h, name.encode(), f.encode(), buf.ctypes.data_as(_vp), buf.size),
                   "GetOutputs")
            outs.append(buf[:n].reshape(hshape).copy())
        return outs

    def num_active_kernels(self):
        return self._lib.ogle_session_num_active_kernels(self._h)

    def num_placed(self):
        """Concat inputs written in place by their producers (option "fuse_concats")."""
        return self._lib.ogle_session_num_placed(self._h)

    def num_residuals(self):
        """Residual Adds computed in a convolution's pass (option "fuse_residuals")."""
        return self._lib.ogle_session_num_residuals(self._h)

    def num_branches(self):
        return self._lib.ogle_session_num_branches(self._h)

    def graph_captured(self):
        return bool(self._lib.ogle_session_graph_captured(self._h))

    def device_bytes(self):
        return int(self._lib.ogle_session_device_bytes(self._h))

    def Profile(self, inputs):
        n, names, data, shapes, ranks, fmts, keep = _pack_inputs(inputs)
        buf = C.create_string_buffer(1 << 20)
        _check(self._lib.ogle_session_profile(self._h, n, names, data, shapes, ranks, fmts, buf, len(buf)), "Profile")
        rows = []
        for line in buf.value.decode().splitlines():
            name, type_, kernel, ms = line.split("\t")
            rows.append((name, type_, kernel, float(ms)))
        return rows


class Detector:
    """SSD detector: network + box decode + post-process on the device.
    mode 0 = the reference Detector's rule, mode 1 = per-class top-k."""

    def __init__(self, model_path, mode=0, score_thr=0.3, top_k=100, nms_thr=0.45, math_mode=-1, device=-1, stream=None):
        self._lib = rt_lib()
        self.mode, self.top_k = mode, top_k
        self._h = self._lib.ogle_detector_create(device, stream, model_path.encode(), mode, score_thr, top_k, nms_thr,
                                                 math_mode, None, None, None, None)
        if not self._h:
            raise OgleError("detector_create: " + self._lib.ogle_rt_last_error().decode())
        self._shape = None
        self._in_flight = 0

    def close(self):
        if self._h:
            self._lib.ogle_detector_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def session(self):
        return FBOSession(_borrowed=self._lib.ogle_detector_session(self._h))

    def detect_async(self, images_ptr, N, H, W):
        """images_ptr: address of N*H*W*3 host floats (NHWC, preprocessed); pinned memory makes the copy asynchronous.
        Up to two calls may be in flight; wait() retires the oldest."""
        _check(self._lib.ogle_detector_detect_async(self._h, images_ptr, N, H, W), "detect_async")
        self._shape = N
        self._in_flight += 1

    def in_flight(self):
        return self._in_flight

    def detect_bgr8_async(self, images, H, W, mean_rgb=(123.0, 117.0, 104.0)):
        """images: list of uint8 numpy arrays [h_i, w_i, 3] (BGR, C-contiguous; they must stay alive until
        the wait() that retires the call). Resize and mean-subtraction happen on the device."""
        n = len(images)
        for im in images:
            if im.dtype != np.uint8 or im.ndim != 3 or im.shape[2] != 3 or not im.flags["C_CONTIGUOUS"]:
                raise ValueError("expected C-contiguous uint8 [h, w, 3] images")
        ptrs = (C.c_void_p * n)(*[im.ctypes.data for im in images])
        hs = (C.c_int * n)(*[im.shape[0] for im in images])
        ws = (C.c_int * n)(*[im.shape[1] for im in images])
        mean = (C.c_float * 3)(*mean_rgb)
        _check(self._lib.ogle_detector_detect_bgr8_async(self._h, ptrs, hs, ws, n, H, W, mean), "detect_bgr8_async")
        self._shape = n
        self._in_flight += 1

    def detect_bgr8_frames_async(self, frames_ptr, n, h, w, H, W, mean_rgb=(123.0, 117.0, 104.0)):
        """n equally sized 8-bit BGR frames stored back to back at host address frames_ptr ([n, h, w, 3] bytes;
        pinned memory makes the upload asynchronous): one upload, one preprocessing launch."""
        key = (frames_ptr, n, h, w)
        cache = self.__dict__.setdefault("_frames_args", {})      # callers alternate between a few buffers
        cached = cache.get(key)
        if cached is None:
            if len(cache) > 8:
                cache.clear()
            ptrs = (C.c_void_p * n)(*[frames_ptr + i * h * w * 3 for i in range(n)])
            cached = (key, ptrs, (C.c_int * n)(*([h] * n)), (C.c_int * n)(*([w] * n)))
            cache[key] = cached
        mean = (C.c_float * 3)(*mean_rgb)
        _check(self._lib.ogle_detector_detect_bgr8_async(self._h, cached[1], cached[2], cached[3], n, H, W, mean),
               "detect_bgr8_async")
        self._shape = n
        self._in_flight += 1

    def detect_device_async(self, images_dev_ptr, N, H, W, copy_back=False):
        """images_dev_ptr: device address of [N,H,W,4] floats (padded NHWC4)."""
        _check(self._lib.ogle_detector_detect_device_async(self._h, images_dev_ptr, N, H, W, int(copy_back)),
               "detect_device_async")
        self._shape = N
        self._in_flight += int(bool(copy_back))

    def info(self):
        a, c, r = C.c_int(), C.c_int(), C.c_int()
        h, d = C.c_size_t(), C.c_size_t()
        self._lib.ogle_detector_info(self._h, C.byref(a), C.byref(c), C.byref(r), C.byref(h), C.byref(d))
        return dict(num_anchors=a.value, num_classes=c.value, rows=r.value, h2d_bytes=h.value, d2h_bytes=d.value)

    def wait(self, fetch=True):
        self._in_flight = max(0, self._in_flight - 1)
        if not fetch:
            _check(self._lib.ogle_detector_wait(self._h, None, None, None, None, None), "wait")
            return None
        i = self.info()
        N, rows = self._shape, i["rows"]
        score = np.empty((N, rows), np.float32)
        anchor = np.empty((N, rows), np.int32)
        cls = np.empty((N, rows), np.int32)
        box = np.empty((N, rows, 4), np.float32)
        count = np.empty((N,) if self.mode == 0 else (N, i["num_classes"] - 1), np.int32)
        _check(self._lib.ogle_detector_wait(self._h, score.ctypes.data_as(_vp), anchor.ctypes.data_as(_vp),
                                            cls.ctypes.data_as(_vp), box.ctypes.data_as(_vp), count.ctypes.data_as(_vp)), "wait")
        return dict(score=score, anchor=anchor, cls=cls, box=box, count=count)

    def detect(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        N, H, W, _ = images.shape
        self.detect_async(images.ctypes.data_as(_vp), N, H, W)
        return self.wait()
