"""GPU test of mgx_cuda_qgemm_static_scratch(), the quant_dot entry point for callers that
cannot allocate device memory (their runtime fixed its memory plan at compile time, or a
cudaMalloc - which synchronises the device - is not acceptable in their serving loop).  Its
scratch is a fixed array inside the library's device image instead of a caller-provided
workspace.  The result must be identical to mgx_cuda_qgemm() with a workspace, on two calls
in a row (the array is shared and keeps the previous call's contents), and a request beyond
the fixed limit must be rejected.  This file sorts last on purpose: a run that stops at the
first failure has then already run every other test."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _desc(capi, M, N, K, out_type, scale_mode=0, act=0):
    return capi.QgemmDesc(M=M, N=N, K=K, batch=1, lda=K, ldb=N, ldd=N, stride_a=M * K,
                          stride_b=K * N, stride_d=M * N, ab_type=capi.I8, out_type=out_type,
                          b_layout=capi.B_KN, scale_mode=scale_mode, act=act, reserved=0)


def test_static_scratch_matches_workspace_entry_point(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    lib = capi.load()
    limit = lib.mgx_cuda_qgemm_static_scratch_limit()
    assert limit == 16 << 20
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(42)
    # two different problems back to back: the second one finds the first one's bytes in the array
    for (M, N, K, fused) in [(200, 1024, 1040, False), (256, 768, 512, True)]:
        a = torch.from_numpy(rng.integers(-128, 128, size=(M, K), dtype=np.int8)).to(cuda_device)
        b = torch.from_numpy(rng.integers(-128, 128, size=(K, N), dtype=np.int8)).to(cuda_device)
        scale = torch.from_numpy(rng.uniform(1e-5, 1e-4, size=N).astype(np.float32)).to(cuda_device)
        bias = torch.from_numpy(rng.normal(0, 0.1, size=N).astype(np.float32)).to(cuda_device)
        if fused:
            d = _desc(capi, M, N, K, capi.F32, capi.SCALE_PER_COL, capi.ACT_RELU)
            odt, sp, bp = torch.float32, scale, bias
        else:
            d = _desc(capi, M, N, K, capi.I32)
            odt, sp, bp = torch.int32, None, None
        want = capi.qgemm(a, b, scale=sp, scale_mode=d.scale_mode, bias=bp,
                          act="relu" if fused else None, out_dtype=odt)
        got = torch.zeros((M, N), dtype=odt, device=cuda_device)
        rc = lib.mgx_cuda_qgemm_static_scratch(ctypes.byref(d), a.data_ptr(), b.data_ptr(),
                                               got.data_ptr(), None if sp is None else sp.data_ptr(),
                                               None if bp is None else bp.data_ptr(), None, stream)
        assert rc == 0, capi.status_string(rc)
        torch.cuda.synchronize()
        assert torch.equal(got, want)  # same kernels, same arithmetic: identical bits
    # beyond the fixed maximum: rejected on the host, nothing is launched
    big = _desc(capi, 128, 8192, 4096, capi.I32)
    assert lib.mgx_cuda_qgemm_workspace(ctypes.byref(big)) > limit
    one = ctypes.c_void_p(256)
    rc = lib.mgx_cuda_qgemm_static_scratch(ctypes.byref(big), one, one, one, None, None, None, stream)
    assert rc == capi.E_TOO_LARGE
