"""Reductions over the innermost axis and softmax through the C ABI against numpy restatements
of the reference's semantics: accumulation in double (reduce_op.hpp:180-203, accumulator_type),
softmax with the exponentials stored in the output type before the sum (ref_softmax,
src/targets/ref/lowering.cpp:253-320); fp16 results by truncating conversion."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def _ref_reduce(x, op):
    xd = x.astype(np.float64)
    r = {"sum": xd.sum(1), "mean": xd.sum(1) / x.shape[1], "max": xd.max(1), "min": xd.min(1)}[op]
    return r.reshape(-1, 1)


def _ref_softmax(x, half):
    xd = x.astype(np.float64)
    e = np.exp(xd - xd.max(1, keepdims=True))
    e = O.half_trunc(e.astype(np.float32)).astype(np.float64) if half else e.astype(np.float32).astype(np.float64)
    y = e / e.sum(1, keepdims=True)
    return O.half_trunc(y.astype(np.float32)).astype(np.float32) if half else y.astype(np.float32)


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min"])
@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 33), (300, 768), (5, 20000), (2000, 129)])
def test_reduce_f32(cuda_device, op, rows, cols):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(rows * 131 + cols)
    x = rng.normal(0.3, 2.0, (rows, cols)).astype(np.float32)
    got = capi.reduce_rows(_t(x, cuda_device), op).cpu().numpy()
    ref = _ref_reduce(x, op)
    if op in ("max", "min"):
        assert np.array_equal(got, ref.astype(np.float32))
    else:
        # fp32 tree against double: error far below sqrt(cols) * eps * sum|x|
        bound = 1e-6 * np.abs(x).astype(np.float64).sum(1, keepdims=True) / (cols if op == "mean" else 1)
        assert np.all(np.abs(got - ref) <= bound + 1e-30)


@pytest.mark.parametrize("op", ["sum", "mean", "max", "min"])
def test_reduce_f16_strided_rows(cuda_device, op):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(5)
    full = rng.normal(0, 1.0, (64, 1024)).astype(np.float16)
    x = full[:, :700]
    xt = _t(full, cuda_device)[:, :700]
    assert xt.stride(0) == 1024
    got = capi.reduce_rows(xt, op).cpu().numpy().astype(np.float32)
    ref = _ref_reduce(x.astype(np.float32), op)
    if op in ("max", "min"):
        assert np.array_equal(got, ref.astype(np.float32))
    else:
        # the truncated result may fall one fp16 step below the reference's when the fp32 sum
        # lands on the other side of a representable value
        reft = O.half_trunc(ref.astype(np.float32)).astype(np.float32)
        ulp = np.maximum(np.abs(reft) * 2.0 ** -10, 2.0 ** -24)
        assert np.all(np.abs(got - reft) <= ulp)
        assert np.mean(got == reft) > 0.9


@pytest.mark.parametrize("op", ["sum", "max"])
@pytest.mark.parametrize("cols", [704, 8192])
def test_reduce_f16_vector_path_strided_rows(cuda_device, op, cols):
    """Rows whose pitch and length allow 16-byte loads (a warp per row, a block per long row)."""
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(cols)
    full = rng.normal(0, 1.0, (37, cols + 64)).astype(np.float16)
    xt = _t(full, cuda_device)[:, :cols]
    got = capi.reduce_rows(xt, op).cpu().numpy().astype(np.float32)
    ref = _ref_reduce(full[:, :cols].astype(np.float32), op)
    if op == "max":
        assert np.array_equal(got, ref.astype(np.float32))
    else:
        reft = O.half_trunc(ref.astype(np.float32)).astype(np.float32)
        ulp = np.maximum(np.abs(reft) * 2.0 ** -10, 2.0 ** -24)
        assert np.all(np.abs(got - reft) <= ulp)


def test_softmax_strided_rows_vector_path(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(8)
    full = rng.normal(0, 3.0, (50, 512)).astype(np.float32)
    xt = _t(full, cuda_device)[:, :384]
    got = capi.softmax(xt).cpu().numpy()
    np.testing.assert_allclose(got, _ref_softmax(full[:, :384], False), rtol=1e-5, atol=1e-10)


@pytest.mark.parametrize("rows,cols", [(3, 5), (128, 384), (40, 1500), (9, 4096), (4, 8192), (3, 10000)])
def test_softmax_f32(cuda_device, rows, cols):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(cols)
    x = rng.normal(0, 4.0, (rows, cols)).astype(np.float32)
    got = capi.softmax(_t(x, cuda_device)).cpu().numpy()
    ref = _ref_softmax(x, False)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-10)
    np.testing.assert_allclose(got.astype(np.float64).sum(1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("rows,cols", [(16, 64), (77, 1000), (5, 5000), (2, 9000)])
def test_softmax_f16(cuda_device, rows, cols):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(cols + 1)
    x = rng.normal(0, 3.0, (rows, cols)).astype(np.float16)
    got = capi.softmax(_t(x, cuda_device)).cpu().numpy().astype(np.float32)
    ref = _ref_softmax(x.astype(np.float32), True)
    # one fp16 step: libm / CUDA exp differ in the last fp32 place before truncation
    np.testing.assert_allclose(got, ref, rtol=2.0 ** -9, atol=2.0 ** -24)
    assert np.mean(got == ref) > 0.9


def test_softmax_extreme_values(cuda_device):
    """Large magnitudes and a constant row: no overflow, a uniform row gives 1/cols exactly."""
    from amdmigraphx_b200 import capi
    x = np.zeros((3, 256), np.float32)
    x[0] = 1e30
    x[1, 7] = 1e4
    x[2] = -1e30
    got = capi.softmax(_t(x, cuda_device)).cpu().numpy()
    assert np.array_equal(got[0], np.full(256, 1 / 256, np.float32))
    assert got[1, 7] == 1.0 and got[1].sum() == 1.0
    assert np.array_equal(got[2], np.full(256, 1 / 256, np.float32))


def test_reduce_rejects_bad_arguments(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    x = torch.zeros((4, 8), dtype=torch.int32, device=cuda_device)
    with pytest.raises(Exception):
        capi.reduce_rows(x, "sum")
