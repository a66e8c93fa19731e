"""The C-ABI library loads without a GPU and exports every symbol the headers declare."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header, prefix):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"\w+)\s*\(", text)))


def test_cuda_library_exports_every_declared_symbol():
    from ogle_b200 import _lib
    lib = _lib.cuda_lib()
    names = _declared("ogle_cuda.h", "ogle_cuda_")
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.CUDA_SYMBOLS), set(names) ^ set(_lib.CUDA_SYMBOLS)
    assert b"sm_100a" in lib.ogle_cuda_build_info()
    assert lib.ogle_cuda_status_string(-2).startswith(b"unsupported")


def test_shape_inference_needs_no_gpu():
    """Output-size rule of conv2d.cc:191-194 and pool.cc:93-96."""
    from ogle_b200 import ops
    p = ops.conv_params(1, 300, 300, 3, 32, 3, stride=2, pad=1)
    assert list(p.out_hwc) == [150, 150, 32]
    p = ops.conv_params(1, 19, 19, 512, 24, 3, stride=1, pad=1)
    assert list(p.out_hwc) == [19, 19, 24]
    p = ops.conv_params(1, 10, 10, 8, 8, 3, stride=2, pad=1, dilation=2)
    assert list(p.out_hwc) == [4, 4, 8]
    q = ops.pool_params(32, 76, 76, 256, 3, 2, 1, 0)
    assert list(q.out_hwc) == [38, 38, 256]
    q = ops.pool_params(2, 7, 7, 512, 0, 0, 0, 2)
    assert list(q.out_hwc) == [1, 1, 512] and q.kernel == 7


def test_invalid_arguments_return_status_not_abort():
    from ogle_b200 import _lib
    lib = _lib.cuda_lib()
    p = _lib.ConvParams()
    assert lib.ogle_cuda_conv2d_infer(ctypes.byref(p)) == -1
    assert lib.ogle_cuda_conv2d_filter_bytes(ctypes.byref(p)) == 0
    assert lib.ogle_cuda_relu(None, None, 3, None) == -1      # n not a multiple of 4
    assert lib.ogle_cuda_relu(None, None, 0, None) == 0       # empty input is a no-op
    assert lib.ogle_cuda_pad4(None, None, 0, 5, 0, None) == 0


def test_runtime_library_exports_every_declared_symbol():
    from ogle_b200 import session
    lib = session.rt_lib()
    names = _declared("ogle_runtime.h", "ogle_(?:rt|session|detector|host)_")
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(session.RT_SYMBOLS), set(names) ^ set(session.RT_SYMBOLS)


def test_cpu_list_parser():
    from ogle_b200 import session
    assert session.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert session.parse_cpulist("5") == [5]
    assert session.parse_cpulist("") == []
    assert session.parse_cpulist("2-1,x,7-") == []          # nothing well-formed
    assert session.parse_cpulist("0-1,,4") == [0, 1, 4]


def test_host_binding_is_harmless_without_a_gpu():
    """Unknown topology: nothing is changed and nothing fails."""
    import torch
    from ogle_b200 import session
    if torch.cuda.is_available():
        pytest.skip("covers the no-GPU answer")
    before = os.sched_getaffinity(0)
    r = session.bind_host_to_device(0)
    assert r == {"numa_node": -1, "cpus_bound": 0, "memory_preferred": False}
    assert os.sched_getaffinity(0) == before


def test_pinned_allocation_fails_cleanly_without_a_gpu():
    import torch
    from ogle_b200 import session
    if torch.cuda.is_available():
        pytest.skip("covers the no-GPU answer")
    with pytest.raises(session.OgleError):
        session.PinnedArray((4, 4))
    session.rt_lib().ogle_host_free_pinned(None)          # no-op


def test_ctypes_mirrors_have_the_headers_layout(tmp_path):
    """The Python front end mirrors the parameter structs of include/ogle_cuda.h by hand: a small C program
    compiled against the header prints each struct's size and the offset of its last fields, and they must be
    what ctypes computes for the mirror (a field added on one side only shows up here, not as a corrupted launch)."""
    import subprocess
    from ogle_b200 import _lib
    pairs = [("OgleConvParams", _lib.ConvParams, ["math_mode", "n_tile", "split", "channels_on_m", "sm_pair"]),
             ("OglePoolParams", _lib.PoolParams, ["type", "out_channel_stride"]),
             ("OgleGemmParams", _lib.GemmParams, ["bias_mode"]),
             ("OgleConcatParams", _lib.ConcatParams, ["axis", "in_shapes"]),
             ("OgleDetectParams", _lib.DetectParams, ["top_k", "nms_thr"])]
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "ogle_cuda.h"', 'int main(void) {']
    for cname, _, fields in pairs:
        lines.append('printf("%s %%zu", sizeof(%s));' % (cname, cname))
        for f in fields:
            lines.append('printf(" %%zu", offsetof(%s, %s));' % (cname, f))
        lines.append('printf("\\n");')
    lines += ['return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n")
    for (cname, mirror, fields), line in zip(pairs, out):
        got = line.split()
        assert got[0] == cname
        want = [ctypes.sizeof(mirror)] + [getattr(mirror, f).offset for f in fields]
        assert [int(v) for v in got[1:]] == want, (cname, got[1:], want)
