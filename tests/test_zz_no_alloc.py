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
                          b_layout=capi.B_KN, scale_mode=scale_mode, act=act, flags=0)


def test_static_scratch_matches_workspace_entry_point(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    from oracle import mgx_oracle as O
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
        # and against the CPU oracle, not only against the library's other entry point
        acc = O.quant_dot_int8(a.cpu().numpy(), b.cpu().numpy())
        if fused:
            ref = O.qlinear_epilogue(acc, scale.cpu().numpy()[None, :], bias.cpu().numpy(), "relu")
            np.testing.assert_allclose(got.cpu().numpy(), ref, rtol=1e-5, atol=1e-6)
        else:
            assert np.array_equal(got.cpu().numpy(), acc)  # int32 accumulators: bit-exact
    # beyond the fixed maximum: rejected on the host, nothing is launched
    big = _desc(capi, 128, 8192, 4096, capi.I32)
    assert lib.mgx_cuda_qgemm_workspace(ctypes.byref(big)) > limit
    one = ctypes.c_void_p(256)
    rc = lib.mgx_cuda_qgemm_static_scratch(ctypes.byref(big), one, one, one, None, None, None, stream)
    assert rc == capi.E_TOO_LARGE


def test_static_scratch_weight_streaming_route(cuda_device):
    """[N,K] weights and at most 16 rows: the library's workspace for this shape is the
    partial-sum area of the weight-streaming kernel, so the call runs that kernel with its tile
    counters and partial sums inside the shared static array.  Two calls in a row (the second
    one finds the first one's counters and sums there), each checked against the workspace
    entry point and against the CPU oracle."""
    import torch
    from amdmigraphx_b200 import capi
    from oracle import mgx_oracle as O
    lib = capi.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(43)
    for (M, N, K, fused) in [(16, 4096, 4096, True), (1, 2048, 8192, False), (7, 4096, 4096, True)]:
        a = torch.from_numpy(rng.integers(-128, 128, size=(M, K), dtype=np.int8)).to(cuda_device)
        b = torch.from_numpy(rng.integers(-128, 128, size=(N, K), dtype=np.int8)).to(cuda_device)
        scale = torch.from_numpy(rng.uniform(1e-5, 1e-4, size=N).astype(np.float32)).to(cuda_device)
        bias = torch.from_numpy(rng.normal(0, 0.1, size=N).astype(np.float32)).to(cuda_device)
        d = capi.QgemmDesc(M=M, N=N, K=K, batch=1, lda=K, ldb=K, ldd=N, stride_a=M * K, stride_b=N * K,
                           stride_d=M * N, ab_type=capi.I8, out_type=capi.F32 if fused else capi.I32,
                           b_layout=capi.B_NK, scale_mode=capi.SCALE_PER_COL if fused else capi.SCALE_NONE,
                           act=capi.ACT_RELU if fused else capi.ACT_NONE, flags=0)
        need = lib.mgx_cuda_qgemm_workspace(ctypes.byref(d))
        assert 0 < need <= lib.mgx_cuda_qgemm_static_scratch_limit()  # the streaming route is taken
        odt = torch.float32 if fused else torch.int32
        ws = torch.empty(need, dtype=torch.uint8, device=cuda_device)
        want = capi.qgemm(a, b, b_layout=capi.B_NK, scale=scale if fused else None,
                          scale_mode=d.scale_mode, bias=bias if fused else None,
                          act="relu" if fused else None, out_dtype=odt, workspace=ws)
        got = torch.zeros((M, N), dtype=odt, device=cuda_device)
        rc = lib.mgx_cuda_qgemm_static_scratch(ctypes.byref(d), a.data_ptr(), b.data_ptr(), got.data_ptr(),
                                               scale.data_ptr() if fused else None,
                                               bias.data_ptr() if fused else None, None, stream)
        assert rc == 0, capi.status_string(rc)
        torch.cuda.synchronize()
        assert torch.equal(got, want.reshape(M, N))
        acc = O.quant_dot_int8(a.cpu().numpy(), b.cpu().numpy().T)
        if fused:
            ref = O.qlinear_epilogue(acc, scale.cpu().numpy()[None, :], bias.cpu().numpy(), "relu")
            np.testing.assert_allclose(got.cpu().numpy(), ref, rtol=1e-5, atol=1e-6)
        else:
            assert np.array_equal(got.cpu().numpy(), acc)


def test_static_scratch_falls_back_to_tiles_beyond_the_limit(cuda_device):
    """[N,K] weights whose optional partial-sum area would not fit the static array: the call is
    not rejected, it runs the tiled kernel, which needs no scratch."""
    import torch
    from amdmigraphx_b200 import capi
    from oracle import mgx_oracle as O
    lib = capi.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(44)
    M, N, K = 16, 151936, 128
    d = capi.QgemmDesc(M=M, N=N, K=K, batch=1, lda=K, ldb=K, ldd=N, stride_a=M * K, stride_b=N * K,
                       stride_d=M * N, ab_type=capi.I8, out_type=capi.I32, b_layout=capi.B_NK,
                       scale_mode=capi.SCALE_NONE, act=capi.ACT_NONE, flags=0)
    if lib.mgx_cuda_qgemm_workspace(ctypes.byref(d)) <= lib.mgx_cuda_qgemm_static_scratch_limit():
        pytest.skip("this shape's partial sums fit the static array")
    a = torch.from_numpy(rng.integers(-128, 128, size=(M, K), dtype=np.int8)).to(cuda_device)
    b = torch.from_numpy(rng.integers(-128, 128, size=(N, K), dtype=np.int8)).to(cuda_device)
    got = torch.zeros((M, N), dtype=torch.int32, device=cuda_device)
    rc = lib.mgx_cuda_qgemm_static_scratch(ctypes.byref(d), a.data_ptr(), b.data_ptr(), got.data_ptr(),
                                           None, None, None, stream)
    assert rc == 0, capi.status_string(rc)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), O.quant_dot_int8(a.cpu().numpy(), b.cpu().numpy().T))
    # invalid dimensions are an argument error, not a size error
    bad = capi.QgemmDesc(M=-1, N=N, K=K, batch=1, lda=K, ldb=K, ldd=N, ab_type=capi.I8, out_type=capi.I32,
                         b_layout=capi.B_NK)
    one = ctypes.c_void_p(256)
    assert lib.mgx_cuda_qgemm_static_scratch(ctypes.byref(bad), one, one, one, None, None, None, stream) == capi.E_INVALID_ARG
