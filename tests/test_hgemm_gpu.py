"""dot on fp16 operands through mgx_cuda_qgemm (ab_type MGX_F16): kind::f16 tensor-core tiles with
fp32 accumulation against a float64 product of the same fp16 inputs; the fp16 result is the
truncated fp32 accumulator, so it may sit one fp16 step from the truncated exact value."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def _check(got, a, b, out_half):
    ref = a.astype(np.float64) @ b.astype(np.float64)
    mag = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    err = np.abs(got.astype(np.float64) - ref)
    # accumulation error of fp32 partial sums plus, for fp16 results, one fp16 step of the value
    bound = 4e-6 * mag + (np.abs(ref) * 2.0 ** -10 + 2.0 ** -24 if out_half else 0)
    assert np.all(err <= bound), float((err / np.maximum(bound, 1e-30)).max())


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 136, 264), (1, 64, 8), (300, 520, 1032),
                                   (1024, 768, 768)])
@pytest.mark.parametrize("out_half", [True, False])
def test_f16_dot_nk(cuda_device, M, N, K, out_half):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + N + K)
    a = rng.normal(0, 1, (M, K)).astype(np.float16)
    bt = rng.normal(0, 0.5, (N, K)).astype(np.float16)
    got = capi.qgemm(_t(a, cuda_device), _t(bt, cuda_device), b_layout=capi.B_NK,
                     out_dtype=torch.float16 if out_half else torch.float32)
    _check(got.cpu().numpy().reshape(M, N), a, bt.T, out_half)


@pytest.mark.parametrize("batch,M,N,K", [(1, 72, 50, 96), (3, 72, 50, 100), (8, 64, 64, 32)])
def test_f16_dot_kn_batched(cuda_device, batch, M, N, K):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(batch * 7 + K)
    # A rows padded to a 16-byte multiple, as the tensor maps need
    lda = (K + 7) // 8 * 8
    afull = rng.normal(0, 1, (batch, M, lda)).astype(np.float16)
    a = afull[:, :, :K]
    b = rng.normal(0, 0.5, (batch, K, N)).astype(np.float16)
    at = _t(afull, cuda_device)[:, :, :K]
    got = capi.qgemm(at, _t(b, cuda_device), b_layout=capi.B_KN, out_dtype=torch.float16)
    got = got.cpu().numpy()
    for i in range(batch):
        _check(got[i], a[i], b[i], True)


def test_f16_dot_bias_relu_residual(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(3)
    M, N, K = 256, 192, 128
    a = rng.normal(0, 1, (M, K)).astype(np.float16)
    bt = rng.normal(0, 0.5, (N, K)).astype(np.float16)
    bias = rng.normal(0, 1, N).astype(np.float32)
    res = rng.normal(0, 1, (M, N)).astype(np.float32)
    got = capi.qgemm(_t(a, cuda_device), _t(bt, cuda_device), b_layout=capi.B_NK,
                     bias=_t(bias, cuda_device), act="relu", residual=_t(res, cuda_device),
                     out_dtype=torch.float32).cpu().numpy().reshape(M, N)
    ref = np.maximum(a.astype(np.float64) @ bt.T.astype(np.float64) + bias, 0) + res
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-4)


def test_f16_dot_rejects_unaligned_rows(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    a = torch.zeros((16, 20), dtype=torch.float16, device=cuda_device)
    b = torch.zeros((32, 20), dtype=torch.float16, device=cuda_device)
    with pytest.raises(Exception):
        capi.qgemm(a, b, b_layout=capi.B_NK, out_dtype=torch.float16)
