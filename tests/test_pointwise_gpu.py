"""The generic element-wise kernel through the C ABI against a numpy restatement of the reference's
per-operator semantics: every result takes its instruction's type before it is used again (fp16:
truncating conversion, like migraphx::half)."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def _as_type(v, code):
    from amdmigraphx_b200 import capi
    v = np.asarray(v, dtype=np.float32)
    if code == capi.F16:
        return O.half_trunc(v).astype(np.float32)
    if code == capi.I8:
        return v.astype(np.int32).astype(np.int8).astype(np.float32)
    if code == capi.I32:
        return v.astype(np.int32).astype(np.float32)
    return v


def _numpy_program(inputs, program):
    vals = [np.asarray(i, dtype=np.float32) for i in inputs]
    f32 = np.float32
    fn = {
        "add": lambda x, y, z: x + y, "sub": lambda x, y, z: x - y, "mul": lambda x, y, z: x * y,
        "div": lambda x, y, z: x / y, "min": lambda x, y, z: np.where(y < x, y, x),
        "max": lambda x, y, z: np.where(x < y, y, x), "neg": lambda x, y, z: -x,
        "abs": lambda x, y, z: np.abs(x), "sqrt": lambda x, y, z: np.sqrt(x),
        "rsqrt": lambda x, y, z: f32(1) / np.sqrt(x), "recip": lambda x, y, z: f32(1) / x,
        "relu": lambda x, y, z: np.where(x < 0, f32(0), x), "floor": lambda x, y, z: np.floor(x),
        "ceil": lambda x, y, z: np.ceil(x), "nearbyint": lambda x, y, z: np.rint(x),
        "convert": lambda x, y, z: x, "where": lambda x, y, z: np.where(x != 0, y, z),
        "clip": lambda x, y, z: np.minimum(np.maximum(x, y), z),
        "equal": lambda x, y, z: (x == y).astype(f32), "greater": lambda x, y, z: (x > y).astype(f32),
        "less": lambda x, y, z: (x < y).astype(f32), "identity": lambda x, y, z: x,
    }
    for (op, ty, src, imm) in program:
        s = list(src) + [0] * (3 - len(src))
        if op == "const":
            v = np.full_like(vals[0], imm, dtype=np.float32)
        elif op == "leaky_relu":
            v = np.where(vals[s[0]] > 0, vals[s[0]], vals[s[0]] * f32(imm))
        else:
            with np.errstate(all="ignore"):
                v = fn[op](vals[s[0]], vals[s[1]], vals[s[2]]).astype(np.float32)
        vals.append(_as_type(v, ty))
    return vals[-1]


def test_pointwise_fp16_chain_bit_exact(cuda_device):
    """bias add, scale, clip, residual in fp16: exactly rounded operators, truncation after each."""
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(0)
    r, c = 70, 200
    x = rng.normal(0, 2, size=(r, c)).astype(np.float16)
    res = rng.normal(0, 1, size=(r, c)).astype(np.float16)
    bias = rng.normal(0, 0.5, size=(c,)).astype(np.float16)
    h = capi.F16
    prog = [("add", h, (0, 1), 0.0), ("const", h, (), 0.7071), ("mul", h, (3, 4), 0.0),
            ("const", h, (), -1.5), ("const", h, (), 2.25), ("clip", h, (5, 6, 7), 0.0),
            ("abs", h, (8,), 0.0), ("sqrt", h, (9,), 0.0), ("add", h, (10, 2), 0.0),
            ("leaky_relu", h, (11,), 0.1)]
    xt, rt = _t(x, cuda_device), _t(res, cuda_device)
    bt = _t(bias, cuda_device)[None, :].expand(r, c)
    got = capi.pointwise([xt, bt, rt], prog, (r, c)).cpu().numpy()
    ref = _numpy_program([x, np.broadcast_to(bias, (r, c)), res], prog)
    np.testing.assert_array_equal(got.astype(np.float32), ref)


def test_pointwise_fp32_broadcast_where_and_convert(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(1)
    shape = (3, 17, 5, 33)
    x = rng.normal(0, 3, size=shape).astype(np.float32)
    y = rng.normal(0, 3, size=shape).astype(np.float32)
    s = rng.uniform(0.5, 2.0, size=(shape[1], 1, 1)).astype(np.float32)
    f, i8 = capi.F32, capi.I8
    prog = [("div", f, (0, 2), 0.0), ("greater", f, (0, 1), 0.0), ("min", f, (0, 1), 0.0),
            ("where", f, (4, 3, 5), 0.0), ("nearbyint", f, (6,), 0.0), ("const", f, (), -128.0),
            ("const", f, (), 127.0), ("clip", f, (7, 8, 9), 0.0), ("convert", i8, (10,), 0.0)]
    st = _t(s, cuda_device)[None].expand(*shape)
    got = capi.pointwise([_t(x, cuda_device), _t(y, cuda_device), st], prog, shape)
    assert got.dtype == torch.int8
    ref = _numpy_program([x, y, np.broadcast_to(s[None], shape)], prog)
    np.testing.assert_array_equal(got.cpu().numpy().astype(np.float32), ref)


def test_pointwise_transcendentals_close_to_libm(cuda_device):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(2)
    x = rng.normal(0, 1.5, size=(64, 128)).astype(np.float32)
    f = capi.F32
    prog = [("tanh", f, (0,), 0.0), ("sigmoid", f, (0,), 0.0), ("exp", f, (1,), 0.0), ("add", f, (3, 2), 0.0),
            ("log", f, (4,), 0.0), ("erf", f, (0,), 0.0), ("mul", f, (5, 6), 0.0)]
    got = capi.pointwise([_t(x, cuda_device)], prog, x.shape).cpu().numpy()
    xd = x.astype(np.float64)
    import math
    erf = np.vectorize(math.erf)
    ref = np.log(np.exp(np.tanh(xd)) + 1.0 / (1.0 + np.exp(-xd))) * erf(xd)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


def test_pointwise_rejects_bad_programs(cuda_device):
    from amdmigraphx_b200 import capi
    import torch
    x = torch.zeros((4, 4), device=cuda_device)
    with pytest.raises(capi.MgxError) as e:
        capi.pointwise([x], [("add", capi.F32, (0, 3), 0.0)], (4, 4))  # operand 3 does not exist
    assert e.value.code == capi.E_INVALID_ARG


@pytest.mark.parametrize("rows,cols,strided", [(1, 4096, False), (16, 11008, True), (3, 64, True), (5, 264, False)])
def test_fixed_fp16_forms_match_the_register_machine(cuda_device, rows, cols, strided):
    """A residual add / sub / mul and the SwiGLU gate take a fixed-function kernel when their fp16
    operands have contiguous, 16-byte aligned rows.  The same programs behind a leading identity
    (which changes no value) go through the register machine: the bits must agree, values in the
    fp16 subnormal range and zeros included; add / sub / mul also against numpy."""
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(rows * 1000 + cols)
    h = capi.F16
    both = rng.normal(0, 2, size=(rows, 2 * cols)).astype(np.float16)
    both[:, ::7] *= np.float16(1e-3)
    both[0, :8] = [0.0, -0.0, 6e-8, -6e-8, 6.1e-5, -6.1e-5, 30000.0, -30000.0]
    both[0, cols:cols + 8] = [1.0, 0.0, 3e-4, 1e-4, 1e-3, 6e-5, 2.0, 2.0]
    if strided:  # two column slices of one packed buffer, like gate and up of a fused linear
        packed = _t(both, cuda_device)
        xt, yt = packed[:, :cols], packed[:, cols:]
    else:
        xt, yt = _t(both[:, :cols], cuda_device), _t(both[:, cols:], cuda_device)
    x, y = both[:, :cols], both[:, cols:]
    for op in ("add", "sub", "mul"):
        fast = capi.pointwise([xt, yt], [(op, h, (0, 1), 0.0)], (rows, cols))
        slow = capi.pointwise([xt, yt], [("identity", h, (0,), 0.0), (op, h, (2, 1), 0.0)], (rows, cols))
        assert torch.equal(fast.view(torch.int16), slow.view(torch.int16)), op
        ref = _numpy_program([x, y], [(op, h, (0, 1), 0.0)])
        np.testing.assert_array_equal(fast.cpu().numpy().astype(np.float32), ref)
    swiglu = [("sigmoid", h, (0,), 0.0), ("mul", h, (0, 2), 0.0), ("mul", h, (3, 1), 0.0)]
    behind = [("identity", h, (0,), 0.0), ("sigmoid", h, (2,), 0.0), ("mul", h, (2, 3), 0.0), ("mul", h, (4, 1), 0.0)]
    fast = capi.pointwise([xt, yt], swiglu, (rows, cols))
    slow = capi.pointwise([xt, yt], behind, (rows, cols))
    assert torch.equal(fast.view(torch.int16), slow.view(torch.int16))
    # the gate as the second input
    fast2 = capi.pointwise([yt, xt], [("sigmoid", h, (1,), 0.0), ("mul", h, (2, 1), 0.0), ("mul", h, (0, 3), 0.0)],
                           (rows, cols))
    assert torch.equal(fast2.view(torch.int16), slow.view(torch.int16))
    assert capi.device_status() == 0
