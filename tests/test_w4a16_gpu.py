"""Weight-only int4 linear (unpack_int4 + group dequantizelinear + dot) on the GPU against
the CPU oracle: fp16 output within rtol 2e-2 / atol 1e-2."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def _case(rng, M, N, K, group, with_zp):
    a = rng.normal(0, 1, size=(M, K)).astype(np.float16)
    bp = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    s = rng.uniform(0.005, 0.02, size=(N, K // group)).astype(np.float16)
    zp = rng.integers(0, 16, size=(N, K // group)).astype(np.uint8) if with_zp else None
    return a, bp, s, zp


@pytest.mark.parametrize("M,N,K,group", [
    (1, 256, 512, 128), (1, 4096, 4096, 128), (16, 512, 1024, 128), (4, 100, 256, 32),
    (3, 64, 11008, 128), (16, 1024, 4096, 128), (2, 40, 64, 64),
    (8, 1000, 2048, 256), (5, 4096, 8192, 128), (12, 130, 640, 128), (9, 20000, 1024, 512),
    (2, 512, 1024, 128), (4, 384, 2048, 128), (7, 3000, 1536, 128), (1, 8192, 28672, 128),
])
@pytest.mark.parametrize("with_zp", [False, True])
def test_w4a16_decode(cuda_device, M, N, K, group, with_zp):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M * 1009 + N * 17 + K + group)
    a, bp, s, zp = _case(rng, M, N, K, group, with_zp)
    ref = O.w4a16_linear(a, bp, s, zp, 8, group).astype(np.float32)
    got = capi.w4a16(_t(a, cuda_device), _t(bp, cuda_device), _t(s, cuda_device),
                     None if zp is None else _t(zp, cuda_device), group=group, which="gemv")
    np.testing.assert_allclose(got.cpu().numpy().astype(np.float32), ref, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K,group,with_zp", [
    (17, 256, 1024, 128, True), (512, 512, 1024, 128, True), (100, 136, 2304, 128, True),
    (300, 1000, 2048, 256, False), (129, 20000, 512, 128, True), (256, 384, 4096, 512, False),
])
def test_w4a16_prefill(cuda_device, M, N, K, group, with_zp):
    """More than 16 rows (prefill phase of the int4 decoder): same tolerance."""
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + N + K)
    a, bp, s, zp = _case(rng, M, N, K, group, with_zp)
    ref = O.w4a16_linear(a, bp, s, zp, 8, group).astype(np.float32)
    got = capi.w4a16(_t(a, cuda_device), _t(bp, cuda_device), _t(s, cuda_device),
                     None if zp is None else _t(zp, cuda_device), group=group, which="gemm")
    np.testing.assert_allclose(got.cpu().numpy().astype(np.float32), ref, rtol=2e-2, atol=1e-2)


def test_w4a16_decode_is_reproducible(cuda_device):
    """Tiles shared between thread blocks add their partial sums in a fixed order: two runs of
    the same problem give identical bits, for every row count the decode kernel specialises on."""
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(5)
    for M in (1, 2, 4, 8, 16):
        a, bp, s, zp = _case(rng, M, 1536, 4096, 128, True)
        args = (_t(a, cuda_device), _t(bp, cuda_device), _t(s, cuda_device), _t(zp, cuda_device))
        first = capi.w4a16(*args, group=128, which="gemv").clone()
        for _ in range(3):
            again = capi.w4a16(*args, group=128, which="gemv")
            assert torch.equal(first, again)


def test_w4a16_decode_unaligned_metadata_falls_back(cuda_device):
    """Scales that are not 4-byte aligned cannot take the tensor-core kernel (it copies aligned
    words); the call still succeeds on the fallback kernels with the same tolerance."""
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(6)
    a, bp, s, zp = _case(rng, 2, 256, 1024, 128, False)
    ref = O.w4a16_linear(a, bp, s, None, 8, 128).astype(np.float32)
    buf = torch.zeros(s.size + 1, dtype=torch.float16, device=cuda_device)
    s_dev = buf[1:].view(s.shape)  # 2 bytes past a 4-byte boundary
    s_dev.copy_(_t(s, cuda_device))
    assert s_dev.data_ptr() % 4 == 2
    got = capi.w4a16(_t(a, cuda_device), _t(bp, cuda_device), s_dev, None, group=128, which="gemv")
    np.testing.assert_allclose(got.cpu().numpy().astype(np.float32), ref, rtol=2e-2, atol=1e-2)


def test_w4a16_rejects_bad_arguments(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    a = torch.zeros((1, 48), dtype=torch.float16, device=cuda_device)
    bp = torch.zeros((8, 24), dtype=torch.uint8, device=cuda_device)
    s = torch.ones((8, 1), dtype=torch.float16, device=cuda_device)
    with pytest.raises(capi.MgxError) as e:
        capi.w4a16(a, bp, s, group=48)
    assert e.value.code == capi.E_UNSUPPORTED


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 4096, 11008), (64, 2048, 4096)])
def test_w4a16_heavy_tailed_activations(cuda_device, M, N, K):
    """Activations with outliers (a few values per row 100x - 1000x the rest, as the outlier
    channels of real decoder activations): the decode kernels quantise activations per row and
    128-k group, so an outlier may only cost the other values of its own group precision.  The
    results are sums of large terms that partly cancel; the absolute tolerance is therefore
    scaled by the row's typical magnitude: |d| <= 1e-2 * max(1, rms(row)) + 2e-2 * |ref|."""
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + N + K)
    a = rng.normal(0, 1, size=(M, K)).astype(np.float16)
    for r in range(M):
        cols = rng.choice(K, size=6, replace=False)
        a[r, cols] = (rng.uniform(100, 1000, size=6) * rng.choice([-1, 1], size=6)).astype(np.float16)
    bp = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    sc = rng.uniform(0.005, 0.02, size=(N, K // 128)).astype(np.float16)
    t = lambda v: torch.from_numpy(v).to(cuda_device)  # noqa: E731
    got = capi.w4a16(t(a), t(bp), t(sc), group=128).cpu().numpy().astype(np.float64)
    torch.cuda.synchronize()
    ref = O.w4a16_linear(a, bp, sc, None, 8, 128).astype(np.float64)
    atol = 1e-2 * np.maximum(1.0, np.sqrt((ref ** 2).mean(axis=1, keepdims=True)))
    assert np.all(np.abs(got - ref) <= atol + 2e-2 * np.abs(ref))
    # the error itself is small against the rows' magnitude
    assert np.sqrt(((got - ref) ** 2).mean()) <= 2e-3 * np.sqrt((ref ** 2).mean())
