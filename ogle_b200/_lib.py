"""ctypes bindings of the C ABI in include/ogle_cuda.h.

The library is the product: if libogle_cuda.so is missing this module raises,
it never falls back to another implementation.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
CUDA_LIB_PATH = os.path.join(_HERE, "libogle_cuda.so")
RT_LIB_PATH = os.path.join(_HERE, "libogle_rt.so")

OGLE_MAX_CONCAT_INPUTS = 16

MATH_FP32, MATH_TF32, MATH_TF32X3 = 0, 1, 2
ACT_NONE, ACT_CLIP, ACT_RELU = 0, 1, 2


class ConvParams(C.Structure):
    _fields_ = [
        ("N", C.c_int), ("in_hwc", C.c_int * 3), ("out_hwc", C.c_int * 3),
        ("kernel", C.c_int), ("stride", C.c_int), ("pad", C.c_int), ("dilation", C.c_int), ("group", C.c_int),
        ("has_bias", C.c_int), ("act", C.c_int), ("min_value", C.c_float), ("max_value", C.c_float),
        ("in_channel_stride", C.c_int), ("out_channel_stride", C.c_int), ("out_channel_offset", C.c_int),
        ("math_mode", C.c_int), ("n_tile", C.c_int), ("split", C.c_int), ("channels_on_m", C.c_int), ("sm_pair", C.c_int),
    ]


class PoolParams(C.Structure):
    _fields_ = [
        ("N", C.c_int), ("in_hwc", C.c_int * 3), ("out_hwc", C.c_int * 3),
        ("kernel", C.c_int), ("stride", C.c_int), ("pad", C.c_int), ("type", C.c_int),
        ("in_channel_stride", C.c_int), ("out_channel_stride", C.c_int),
    ]


class GemmParams(C.Structure):
    _fields_ = [
        ("M", C.c_int), ("K", C.c_int), ("N", C.c_int), ("transB", C.c_int),
        ("alpha", C.c_float), ("beta", C.c_float), ("bias_mode", C.c_int),
        ("lda", C.c_int), ("ldb", C.c_int), ("ldc", C.c_int), ("ldy", C.c_int), ("math_mode", C.c_int),
    ]


class ConcatParams(C.Structure):
    _fields_ = [("n_inputs", C.c_int), ("axis", C.c_int), ("in_shapes", (C.c_int * 4) * OGLE_MAX_CONCAT_INPUTS)]


class DetectParams(C.Structure):
    _fields_ = [
        ("N", C.c_int), ("A", C.c_int), ("C", C.c_int), ("logit_stride", C.c_int), ("mode", C.c_int),
        ("score_thr", C.c_float), ("top_k", C.c_int), ("nms_thr", C.c_float),
        ("image_w", C.c_int), ("image_h", C.c_int), ("frame_sizes", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol include/ogle_cuda.h declares
_vp = C.c_void_p
CUDA_SYMBOLS = {
    "ogle_cuda_status_string": (C.c_char_p, [C.c_int]),
    "ogle_cuda_set_wait_limit": (C.c_int, [C.c_long]),
    "ogle_cuda_build_info": (C.c_char_p, []),
    "ogle_cuda_launch_count": (C.c_uint64, []),
    "ogle_cuda_last_error": (C.c_char_p, []),
    "ogle_cuda_conv2d_infer": (C.c_int, [C.POINTER(ConvParams)]),
    "ogle_cuda_conv2d_filter_bytes": (C.c_size_t, [C.POINTER(ConvParams)]),
    "ogle_cuda_conv2d_prepack": (C.c_int, [C.POINTER(ConvParams), _vp, _vp, _vp]),
    "ogle_cuda_conv2d": (C.c_int, [C.POINTER(ConvParams), _vp, _vp, _vp, _vp, _vp]),
    "ogle_cuda_conv2d_residual_supported": (C.c_int, [C.POINTER(ConvParams)]),
    "ogle_cuda_conv2d_residual": (C.c_int, [C.POINTER(ConvParams), _vp, _vp, _vp, _vp, C.c_int, _vp, _vp]),
    "ogle_cuda_conv2d_workspace_bytes": (C.c_size_t, [C.POINTER(ConvParams)]),
    "ogle_cuda_conv2d_ws": (C.c_int, [C.POINTER(ConvParams), _vp, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "ogle_cuda_conv2d_kernel_name": (C.c_char_p, [C.POINTER(ConvParams)]),
    "ogle_cuda_conv2d_pair_supported": (C.c_int, [C.POINTER(ConvParams)]),
    "ogle_cuda_conv2d_pair": (C.c_int, [C.POINTER(ConvParams), _vp, _vp, _vp, C.c_int, C.c_int, _vp, _vp, _vp]),
    "ogle_cuda_conv2d_pair_workspace_bytes": (C.c_size_t, [C.POINTER(ConvParams), C.c_int, C.c_int]),
    "ogle_cuda_conv2d_pair_ws": (C.c_int, [C.POINTER(ConvParams), _vp, _vp, _vp, C.c_int, C.c_int, _vp, _vp, _vp, C.c_size_t, _vp]),
    "ogle_cuda_pool_infer": (C.c_int, [C.POINTER(PoolParams)]),
    "ogle_cuda_pool": (C.c_int, [C.POINTER(PoolParams), _vp, _vp, _vp]),
    "ogle_cuda_batchnorm": (C.c_int, [_vp] * 6 + [C.c_long, C.c_int, C.c_int, C.c_float, _vp]),
    "ogle_cuda_relu": (C.c_int, [_vp, _vp, C.c_long, _vp]),
    "ogle_cuda_clip": (C.c_int, [_vp, _vp, C.c_long, C.c_float, C.c_float, _vp]),
    "ogle_cuda_add": (C.c_int, [_vp, _vp, _vp, C.c_long, _vp]),
    "ogle_cuda_add_act": (C.c_int, [_vp, _vp, _vp, C.c_long, C.c_int, C.c_float, C.c_float, _vp]),
    "ogle_cuda_gemm": (C.c_int, [C.POINTER(GemmParams), _vp, _vp, _vp, _vp, _vp]),
    "ogle_cuda_gemm_packed_b_bytes": (C.c_size_t, [C.POINTER(GemmParams)]),
    "ogle_cuda_gemm_pack_b": (C.c_int, [C.POINTER(GemmParams), _vp, _vp, _vp]),
    "ogle_cuda_gemm_packed": (C.c_int, [C.POINTER(GemmParams), _vp, _vp, _vp, _vp, _vp]),
    "ogle_cuda_gemm_ws": (C.c_int, [C.POINTER(GemmParams), _vp, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "ogle_cuda_gemm_static_max_bytes": (C.c_size_t, []),
    "ogle_cuda_gemm_static": (C.c_int, [C.POINTER(GemmParams), _vp, _vp, _vp, _vp, _vp]),
    "ogle_cuda_set_overlapped_launches": (C.c_int, [C.c_int]),
    "ogle_cuda_device_status": (C.c_int, []),
    "ogle_cuda_clear_device_status": (C.c_int, []),
    "ogle_cuda_device_status_detail": (C.c_int, []),
    "ogle_cuda_concat": (C.c_int, [C.POINTER(ConcatParams), C.POINTER(_vp), _vp, _vp]),
    "ogle_cuda_pad4": (C.c_int, [_vp, _vp, C.c_long, C.c_int, C.c_int, _vp]),
    "ogle_cuda_unpad4": (C.c_int, [_vp, _vp, C.c_long, C.c_int, C.c_int, _vp]),
    "ogle_cuda_preprocess_bgr8_batch": (C.c_int, [_vp, _vp, C.c_int, _vp, C.c_int, C.c_int, C.POINTER(C.c_float), _vp]),
    "ogle_cuda_preprocess_bgr8": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, _vp, C.c_int, C.c_int, C.POINTER(C.c_float), _vp]),
    "ogle_cuda_nchw_to_nhwc4": (C.c_int, [_vp, _vp] + [C.c_int] * 4 + [_vp]),
    "ogle_cuda_transpose": (C.c_int, [_vp, _vp, C.POINTER(C.c_int), C.POINTER(C.c_int), _vp]),
    "ogle_cuda_reshape": (C.c_int, [_vp, _vp, C.c_long, C.c_int, C.c_int, _vp]),
    "ogle_cuda_reshape_placed": (C.c_int, [_vp, _vp, C.c_long, C.c_int, C.c_int, C.c_long, C.c_long, _vp]),
    "ogle_cuda_ssd_decode": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.POINTER(C.c_float), _vp]),
    "ogle_cuda_ssd_detect": (C.c_int, [C.POINTER(DetectParams)] + [_vp] * 8),
}

_cuda = None


def cuda_lib():
    """Loads libogle_cuda.so (no GPU needed to load it) and types its symbols."""
    global _cuda
    if _cuda is None:
        if not os.path.exists(CUDA_LIB_PATH):
            raise RuntimeError(
                f"{CUDA_LIB_PATH} is missing: build it with `python -m ogle_b200.build` "
                "(nvcc, sm_100a). There is no fallback path.")
        lib = C.CDLL(CUDA_LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in CUDA_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _cuda = lib
    return _cuda


class OgleError(RuntimeError):
    pass


def check(rc, what):
    if rc != 0:
        lib = cuda_lib()
        msg = lib.ogle_cuda_status_string(rc).decode()
        extra = lib.ogle_cuda_last_error().decode()
        raise OgleError(f"{what}: {msg} (status {rc}){' - ' + extra if extra and rc == -3 else ''}")
