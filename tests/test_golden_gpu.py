"""GPU tests: the CUDA kernels, called through the C ABI, against outputs of MIGraphX's own
`ref` target committed as fixtures (tests/golden/ref_fixtures.npz)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FX = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_fixtures.npz"))


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def _bits(t):
    import torch
    return t.contiguous().view(torch.uint8).cpu().numpy()


@pytest.mark.parametrize("tag", ["f32", "f16"])
def test_quantizelinear_matches_ref(cuda_device, tag):
    import torch
    from amdmigraphx_b200 import capi
    x, s = _t(FX[f"q_{tag}_x"], cuda_device), _t(FX[f"q_{tag}_scale"], cuda_device)
    np.testing.assert_array_equal(_bits(capi.quantizelinear(x, s, out_dtype=torch.int8)),
                                  FX[f"q_{tag}_i8"].view(np.uint8))
    zp = _t(np.array([128], dtype=np.uint8), cuda_device)
    np.testing.assert_array_equal(_bits(capi.quantizelinear(x, s, zp)), FX[f"q_{tag}_u8_zp128"])
    np.testing.assert_array_equal(_bits(capi.quantizelinear(x, s, out_dtype=torch.float8_e4m3fn)),
                                  FX[f"q_{tag}_fp8"])


def test_quantizelinear_per_channel_matches_ref(cuda_device):
    from amdmigraphx_b200 import capi
    got = capi.quantizelinear(_t(FX["qc_x"], cuda_device), _t(FX["qc_scale"], cuda_device),
                              _t(FX["qc_zp"], cuda_device))
    np.testing.assert_array_equal(got.cpu().numpy(), FX["qc_i8"])


def test_dequantizelinear_matches_ref(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    got = capi.dequantizelinear(_t(FX["dq_i32_x"], cuda_device), _t(FX["dq_i32_scale"], cuda_device))
    np.testing.assert_array_equal(_bits(got), FX["dq_i32_y"].view(np.uint8).reshape(16, -1))
    got = capi.dequantizelinear(_t(FX["dq_u8_x"], cuda_device), _t(FX["dq_u8_scale"], cuda_device),
                                _t(FX["dq_u8_zp"], cuda_device))
    np.testing.assert_array_equal(_bits(got), FX["dq_u8_y"].view(np.uint8).reshape(16, -1))
    got = capi.dequantizelinear(_t(FX["dq_fp8_x"], cuda_device).view(torch.float8_e4m3fn),
                                _t(FX["dq_i32_scale"], cuda_device))
    np.testing.assert_array_equal(_bits(got), FX["dq_fp8_y"].view(np.uint8).reshape(16, -1))


def test_int4_matches_ref(cuda_device):
    from amdmigraphx_b200 import capi
    np.testing.assert_array_equal(capi.unpack_int4(_t(FX["u4_packed"], cuda_device)).cpu().numpy(),
                                  FX["u4_unpacked_u8"])
    np.testing.assert_array_equal(
        capi.unpack_int4(_t(FX["u4_packed"].view(np.int8), cuda_device)).cpu().numpy(),
        FX["u4_unpacked_i8"])
    np.testing.assert_array_equal(capi.pack_int4(_t(FX["p4_values_i8"], cuda_device)).cpu().numpy(),
                                  FX["p4_packed_i8"])
    np.testing.assert_array_equal(
        capi.pack_int4(_t(FX["p4_values_i8"].astype(np.uint8), cuda_device)).cpu().numpy(),
        FX["p4_packed_u8"])


def test_quant_dot_matches_ref(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    got = capi.qgemm(_t(FX["qd_i8_a"], cuda_device), _t(FX["qd_i8_b"], cuda_device))
    np.testing.assert_array_equal(got.cpu().numpy(), FX["qd_i8_c"])  # int32: bit-exact
    got = capi.qgemm(_t(FX["qd_fp8_a"], cuda_device).view(torch.float8_e4m3fn),
                     _t(FX["qd_fp8_b"], cuda_device).view(torch.float8_e4m3fn),
                     out_dtype=torch.float32).cpu().numpy()
    ref = FX["qd_fp8_c"]
    assert np.max(np.abs(got - ref)) <= 2e-6 * np.abs(ref).max()


def test_qdq_block_matches_ref(cuda_device):
    """quantizelinear -> quant_dot -> dequantizelinear -> add -> relu / gelu, config-1 form."""
    import torch
    from amdmigraphx_b200 import capi
    xq = capi.quantizelinear(_t(FX["blk_x"], cuda_device), _t(FX["blk_xscale"], cuda_device),
                             out_dtype=torch.int8)
    np.testing.assert_array_equal(xq.cpu().numpy(), FX["blk_xq"])
    w = _t(FX["blk_w"], cuda_device)
    np.testing.assert_array_equal(capi.qgemm(xq, w).cpu().numpy(), FX["blk_acc"])
    scale, bias = _t(FX["blk_scale"], cuda_device), _t(FX["blk_bias"], cuda_device)
    for act, key in ((None, "blk_none"), ("relu", "blk_relu")):
        got = capi.qgemm(xq, w, scale=scale, bias=bias, act=act, out_dtype=torch.float32)
        np.testing.assert_array_equal(got.cpu().numpy(), FX[key])  # same ops, same roundings
    got = capi.qgemm(xq, w, scale=scale, bias=bias, act="gelu_erf", out_dtype=torch.float32)
    np.testing.assert_allclose(got.cpu().numpy(), FX["blk_gelu"], rtol=1e-5, atol=3e-6)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_w4a16_matches_ref(cuda_device, tag):
    from amdmigraphx_b200 import capi
    g = int(FX[f"w4{tag}_group"][0])
    a, bp, s, zp = (_t(FX[f"w4{tag}_{k}"], cuda_device) for k in ("a", "bp", "scales", "zp"))
    got = capi.w4a16(a, bp, s, None, group=g).cpu().numpy().astype(np.float32)
    np.testing.assert_allclose(got, FX[f"w4{tag}_y_zp8"].astype(np.float32), rtol=2e-2, atol=1e-2)
    got = capi.w4a16(a, bp, s, zp, group=g).cpu().numpy().astype(np.float32)
    np.testing.assert_allclose(got, FX[f"w4{tag}_y_zp"].astype(np.float32), rtol=2e-2, atol=1e-2)
