"""quantizelinear / dequantizelinear / int4 pack-unpack / transpose on the GPU against
the CPU oracle, through the C ABI.  Integer and byte results are bit-exact."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


@pytest.mark.parametrize("rows,cols", [(256, 1024), (3, 7), (1, 4096), (3072, 768), (33, 100)])
@pytest.mark.parametrize("out", ["int8", "uint8", "fp8e4m3fn"])
@pytest.mark.parametrize("xdtype", [np.float32, np.float16])
def test_quantizelinear_per_tensor(cuda_device, rows, cols, out, xdtype):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(rows * 131 + cols)
    x = (rng.normal(0, 1, size=(rows, cols)) * 3).astype(xdtype)
    # exact ties and saturation
    x.flat[: min(8, x.size)] = np.array([0.01, 0.03, -0.01, -0.03, 1000, -1000, 0.05, -0.05],
                                        dtype=xdtype)[: min(8, x.size)]
    scale = np.array([0.02], dtype=xdtype)
    tdt = {"int8": torch.int8, "uint8": torch.uint8, "fp8e4m3fn": torch.float8_e4m3fn}[out]
    zp = None
    zp_t = None
    if out == "uint8":
        zp = np.array([128], dtype=np.uint8)
        zp_t = _t(zp, cuda_device)
    ref = O.quantizelinear(x, scale, zp, out)
    got = capi.quantizelinear(_t(x, cuda_device), _t(scale, cuda_device), zp_t, out_dtype=tdt)
    np.testing.assert_array_equal(got.view(torch.uint8).cpu().numpy(), ref.view(np.uint8))


@pytest.mark.parametrize("axis", [0, 1])
def test_quantizelinear_per_channel_and_zero_point(cuda_device, axis):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(3)
    rows, cols = 96, 160
    x = rng.normal(0, 2, size=(rows, cols)).astype(np.float32)
    n = rows if axis == 0 else cols
    s = rng.uniform(0.01, 0.05, size=n).astype(np.float32)
    z = rng.integers(-20, 20, size=n).astype(np.int8)
    sv = s[:, None] if axis == 0 else s[None, :]
    zv = z[:, None] if axis == 0 else z[None, :]
    ref = O.quantizelinear(x, sv, zv, "int8")
    got = capi.quantizelinear(_t(x, cuda_device), _t(sv, cuda_device), _t(zv, cuda_device))
    np.testing.assert_array_equal(got.cpu().numpy(), ref)


def test_quantizelinear_full_shape_operands(cuda_device):
    """scale and zero point given as dense tensors of x's shape (the op's own form)."""
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(4)
    x = rng.normal(0, 50, size=(18, 20)).astype(np.float32)
    s = rng.uniform(0.5, 6, size=x.shape).astype(np.float32)
    z = rng.integers(-5, 5, size=x.shape).astype(np.int8)
    ref = O.quantizelinear(x, s, z, "int8")
    got = capi.quantizelinear(_t(x, cuda_device), _t(s, cuda_device), _t(z, cuda_device))
    np.testing.assert_array_equal(got.cpu().numpy(), ref)


def test_quantizelinear_empty(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    x = torch.empty((0, 16), dtype=torch.float32, device=cuda_device)
    s = torch.ones(1, dtype=torch.float32, device=cuda_device)
    assert capi.quantizelinear(x, s, out_dtype=torch.int8).shape == (0, 16)


@pytest.mark.parametrize("xt", ["int8", "uint8", "int32", "fp8"])
@pytest.mark.parametrize("st", [np.float32, np.float16])
def test_dequantizelinear(cuda_device, xt, st):
    import torch
    from amdmigraphx_b200 import capi
    if xt == "int32" and st == np.float16:
        pytest.skip("int32 input with an fp16 scale and no zero point is undefined in the reference")
    rng = np.random.default_rng(9)
    rows, cols = 64, 200
    if xt == "int8":
        x = rng.integers(-128, 128, size=(rows, cols)).astype(np.int8)
        zp = rng.integers(-10, 10, size=cols).astype(np.int8)[None, :]
    elif xt == "uint8":
        x = rng.integers(0, 256, size=(rows, cols)).astype(np.uint8)
        zp = rng.integers(0, 16, size=cols).astype(np.uint8)[None, :]
    elif xt == "int32":
        x = rng.integers(-2 ** 24, 2 ** 24, size=(rows, cols)).astype(np.int32)
        zp = None
    else:
        x = rng.integers(0, 0x7F, size=(rows, cols)).astype(np.uint8)
        x |= (rng.integers(0, 2, size=x.shape).astype(np.uint8) << 7)
        zp = None
    s = rng.uniform(0.001, 0.02, size=cols).astype(st)[None, :]
    ref = O.dequantizelinear(x, s, zp, x_is_fp8=(xt == "fp8"))
    xt_t = _t(x, cuda_device)
    if xt == "fp8":
        xt_t = xt_t.view(torch.float8_e4m3fn)
    got = capi.dequantizelinear(xt_t, _t(s, cuda_device), None if zp is None else _t(zp, cuda_device))
    np.testing.assert_array_equal(got.cpu().numpy(), ref)


@pytest.mark.parametrize("signed", [False, True])
def test_int4_pack_unpack(cuda_device, signed):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(1)
    packed = rng.integers(0, 256, size=(37, 64), dtype=np.uint8)
    if signed:
        packed = packed.view(np.int8)
    un = capi.unpack_int4(_t(packed, cuda_device))
    np.testing.assert_array_equal(un.cpu().numpy(), O.unpack_int4(packed, signed))
    # pack clips out-of-range values first
    vals = rng.integers(-20, 30, size=(37, 128)).astype(np.int8 if signed else np.uint8)
    pk = capi.pack_int4(_t(vals, cuda_device))
    np.testing.assert_array_equal(pk.cpu().numpy(), O.pack_int4(vals, signed))
    # round trip
    rt = capi.pack_int4(un)
    np.testing.assert_array_equal(rt.cpu().numpy(), packed)


@pytest.mark.parametrize("shape", [(64, 64), (1000, 130), (3, 7), (2, 96, 257)])
def test_transpose_8bit(cuda_device, shape):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(2)
    x = rng.integers(-128, 128, size=shape).astype(np.int8)
    got = capi.transpose_8bit(_t(x, cuda_device)).cpu().numpy()
    np.testing.assert_array_equal(got, np.swapaxes(x, -1, -2))
