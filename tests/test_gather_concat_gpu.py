"""gather and concat through the C ABI against numpy (op::gather / op::concat semantics:
src/include/migraphx/op/gather.hpp:107-150, concat.hpp:147-163)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


@pytest.mark.parametrize("shape,axis,idx_shape,dtype,itype", [
    ((500, 128), 0, (2, 24), np.float16, np.int64),     # embedding rows, 16-byte units
    ((37, 5, 3), 0, (11,), np.float32, np.int32),       # 4-byte units
    ((6, 50, 7), 1, (3, 4), np.int8, np.int64),         # odd row length: single bytes
    ((4, 9, 10), 2, (5,), np.float16, np.int32),        # innermost axis: one element per row
    ((3, 8), 1, (1,), np.float32, np.int64),
])
def test_gather_matches_numpy(cuda_device, shape, axis, idx_shape, dtype, itype):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(sum(shape) + axis)
    data = (rng.normal(0, 10, shape)).astype(dtype)
    idx = rng.integers(-shape[axis], shape[axis], idx_shape).astype(itype)  # negative: from the end
    got = capi.gather(_t(data, cuda_device), _t(idx, cuda_device), axis).cpu().numpy()
    ref = np.take(data, idx, axis=axis)
    assert got.shape == ref.shape and np.array_equal(got, ref)


def test_gather_out_of_range_index_gives_zeros(cuda_device):
    from amdmigraphx_b200 import capi
    data = np.arange(1, 41, dtype=np.float32).reshape(10, 4)
    idx = np.array([0, 10, -11, 9], dtype=np.int64)
    got = capi.gather(_t(data, cuda_device), _t(idx, cuda_device), 0).cpu().numpy()
    assert np.array_equal(got[0], data[0]) and np.array_equal(got[3], data[9])
    assert not got[1].any() and not got[2].any()


@pytest.mark.parametrize("lens,axis,dtype", [
    ([(2, 40, 128), (2, 24, 128)], 1, np.float16),
    ([(2, 24, 64), (2, 24, 64)], 2, np.float16),
    ([(3, 5), (4, 5), (1, 5)], 0, np.float32),
    ([(7, 3), (7, 2), (7, 11)], 1, np.int8),
    ([(1, 2, 3, 5), (1, 2, 3, 1)], -1, np.int32),
])
def test_concat_matches_numpy(cuda_device, lens, axis, dtype):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(len(lens) + axis)
    xs = [rng.integers(-100, 100, l).astype(dtype) for l in lens]
    got = capi.concat([_t(x, cuda_device) for x in xs], axis).cpu().numpy()
    assert np.array_equal(got, np.concatenate(xs, axis=axis))


def test_empty_gather_and_bad_index_type(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    data = torch.zeros((4, 4), dtype=torch.float32, device=cuda_device)
    idx = torch.zeros((0,), dtype=torch.int64, device=cuda_device)
    assert capi.gather(data, idx, 0).shape == (0, 4)
    with pytest.raises(Exception):
        capi.gather(data, torch.zeros((2,), dtype=torch.int8, device=cuda_device), 0)
