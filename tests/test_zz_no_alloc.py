"""The allocation-free gemm entry point (scratch in a device array inside the library) must give
exactly what the workspace entry point gives, call after call. Collected last on purpose: it has to
pass both on a fresh process and after every other GPU test has run."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(rng, M, K, N, tb):
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = (rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32) * 0.05).astype(np.float32)
    Cm = rng.standard_normal(N, dtype=np.float32)
    return A, B, Cm


def test_gemm_static_matches_workspace_entry_twice_in_a_row():
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    assert lib.ogle_cuda_gemm_static_max_bytes() == 8 << 20
    rng = np.random.default_rng(77)
    shapes = [(200, 512, 1000, 1), (130, 300, 70, 0)]     # second call uses less of the scratch than the first
    for mode in (ops.MATH_TF32X3, ops.MATH_TF32):
        cases = []
        for (M, K, N, tb) in shapes:
            A, B, Cm = _case(rng, M, K, N, tb)
            A4, B4, C4 = ops.upload(A), ops.upload(B), ops.upload(Cm)
            want = ops.gemm_ws(A4, B4, C4, M, K, N, tb, 0.5, 2.0, 2, mode)
            out = torch.full((M, ops.up4(N)), float("nan"), dtype=torch.float32, device="cuda")
            cases.append((M, K, N, tb, A4, B4, C4, want, out))
        # The first call on a device resolves the scratch address, and the first launch of a kernel may make the
        # driver load its code; neither is an allocation of the entry point, so they happen before the measurement.
        for (M, K, N, tb, A4, B4, C4, want, out) in cases:
            ops.gemm_static(A4, B4, C4, out, M, K, N, tb, 0.5, 2.0, 2, mode)
            out.fill_(float("nan"))
        torch.cuda.synchronize()
        # Free bytes of the DEVICE, as the driver reports them: unlike torch's allocator statistics this also sees a
        # cudaMalloc made inside the library.
        free_before, _ = torch.cuda.mem_get_info()
        for (M, K, N, tb, A4, B4, C4, want, out) in cases:        # two calls in a row, no sync between
            ops.gemm_static(A4, B4, C4, out, M, K, N, tb, 0.5, 2.0, 2, mode)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, f"device free memory changed by {free_before - free_after} bytes across the calls"
        for (M, K, N, tb, A4, B4, C4, want, out) in cases:
            assert torch.equal(out, want), (M, K, N, tb, mode)
        # and once more in the opposite order: the scratch carries nothing from call to call
        for (M, K, N, tb, A4, B4, C4, want, out) in reversed(cases):
            out.fill_(float("nan"))
            ops.gemm_static(A4, B4, C4, out, M, K, N, tb, 0.5, 2.0, 2, mode)
            torch.cuda.synchronize()
            assert torch.equal(out, want), (M, K, N, tb, mode)
    assert lib.ogle_cuda_device_status() == 0


def test_gemm_static_rejects_what_does_not_fit():
    import ctypes as C
    import torch
    from ogle_b200 import _lib, ops
    lib = _lib.cuda_lib()
    M, K, N = 8, 1024, 1152                  # packed B = 2 * 1152 * 1024 * 4 bytes > 8 MiB
    A4 = torch.zeros((M, K), dtype=torch.float32, device="cuda")
    B4 = torch.zeros((K, N), dtype=torch.float32, device="cuda")
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    p = ops._gemm_params(A4, B4, None, M, K, N, 0, 1.0, 1.0, 0, ops.MATH_TF32X3)
    assert lib.ogle_cuda_gemm_packed_b_bytes(C.byref(p)) > lib.ogle_cuda_gemm_static_max_bytes()
    launches = ops.launch_count()
    rc = lib.ogle_cuda_gemm_static(C.byref(p), ops._p(A4), ops._p(B4), None, ops._p(out), ops._stream())
    assert rc == -2                          # OGLE_ERR_UNSUPPORTED
    assert b"static scratch holds" in lib.ogle_cuda_last_error()
    assert ops.launch_count() == launches    # refused before any launch
    # the largest problem that does fit is served
    N = 1024
    B4 = torch.zeros((K, N), dtype=torch.float32, device="cuda")
    out = torch.ones((M, N), dtype=torch.float32, device="cuda")
    ops.gemm_static(A4, B4, None, out, M, K, N)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
