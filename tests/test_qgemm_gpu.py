"""Parity of the CUDA quant_dot (+ fused epilogue) against the CPU oracle, through
the C ABI.  int32 accumulators must be bit-exact; the dequantised fp32 output must be
within rtol 1e-5 (it is bit-exact for relu / no activation by construction); fp8 and
fp16 outputs within rtol 2e-2 / atol 1e-2."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


def _t(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def _rand_i8(rng, shape):
    return rng.integers(-127, 128, size=shape, dtype=np.int8)


INT8_SHAPES = [
    (128, 128, 128), (128, 256, 128), (256, 1024, 1024), (64, 96, 128), (1, 64, 32),
    (130, 72, 272), (300, 520, 1040), (129, 257, 4096), (512, 768, 3072),
]


@pytest.mark.parametrize("M,N,K", INT8_SHAPES)
@pytest.mark.parametrize("layout", ["kn", "nk"])
def test_quant_dot_int8_bit_exact(cuda_device, M, N, K, layout):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M * 7919 + N * 31 + K)
    a = _rand_i8(rng, (M, K))
    b = _rand_i8(rng, (K, N))
    ref = O.quant_dot_int8(a, b)
    if layout == "kn":
        got = capi.qgemm(_t(a, cuda_device), _t(b, cuda_device), b_layout=capi.B_KN)
    else:
        got = capi.qgemm(_t(a, cuda_device), _t(b.T, cuda_device), b_layout=capi.B_NK)
    assert got.dtype == torch.int32
    np.testing.assert_array_equal(got.cpu().numpy(), ref)


def test_quant_dot_int8_extremes(cuda_device):
    from amdmigraphx_b200 import capi
    M, N, K = 128, 128, 2048
    a = np.full((M, K), -128, dtype=np.int8)
    b = np.full((K, N), -128, dtype=np.int8)
    b[:, ::2] = 127
    got = capi.qgemm(_t(a, cuda_device), _t(b, cuda_device))
    np.testing.assert_array_equal(got.cpu().numpy(), O.quant_dot_int8(a, b))


def test_quant_dot_int8_batched(cuda_device):
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(5)
    a = _rand_i8(rng, (3, 200, 160))
    b = _rand_i8(rng, (3, 160, 144))
    got = capi.qgemm(_t(a, cuda_device), _t(b, cuda_device))
    np.testing.assert_array_equal(got.cpu().numpy(), O.quant_dot_int8(a, b))


@pytest.mark.parametrize("act", [None, "relu", "gelu_erf"])
@pytest.mark.parametrize("scale_kind", ["tensor", "col", "row"])
def test_qlinear_int8_fused_epilogue(cuda_device, act, scale_kind):
    """config-1 shaped block: quant_dot -> dequantizelinear -> add(bias) -> act."""
    import torch
    from amdmigraphx_b200 import capi
    M, N, K = 256, 1024, 1024
    rng = np.random.default_rng(0)
    a = _rand_i8(rng, (M, K))
    b = _rand_i8(rng, (K, N))
    x_scale = np.float32(0.02)
    if scale_kind == "tensor":
        scale = np.array([x_scale * np.float32(0.005)], dtype=np.float32)
        sview = scale
    elif scale_kind == "col":
        scale = (x_scale * rng.uniform(0.001, 0.01, size=N).astype(np.float32)).astype(np.float32)
        sview = scale[None, :]
    else:
        scale = (x_scale * rng.uniform(0.001, 0.01, size=M).astype(np.float32)).astype(np.float32)
        sview = scale[:, None]
    bias = rng.normal(0, 0.1, size=N).astype(np.float32)
    acc = O.quant_dot_int8(a, b)
    ref = O.qlinear_epilogue(acc, sview, bias, act)
    mode = {"tensor": capi.SCALE_PER_TENSOR, "col": capi.SCALE_PER_COL, "row": capi.SCALE_PER_ROW}[scale_kind]
    got = capi.qgemm(_t(a, cuda_device), _t(b, cuda_device), scale=_t(scale, cuda_device),
                     scale_mode=mode, bias=_t(bias, cuda_device), act=act,
                     out_dtype=torch.float32).cpu().numpy()
    if act in (None, "relu"):
        np.testing.assert_array_equal(got, ref)  # same operations, same roundings
    else:
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=3e-6)


def test_qlinear_int8_residual_fp16_out(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    M, N, K = 384, 768, 768
    rng = np.random.default_rng(11)
    a = _rand_i8(rng, (M, K))
    b = _rand_i8(rng, (K, N))
    scale = rng.uniform(1e-5, 1e-4, size=N).astype(np.float32)
    bias = rng.normal(0, 0.1, size=N).astype(np.float32)
    res = rng.normal(0, 1, size=(M, N)).astype(np.float16)
    ref = O.qlinear_epilogue(O.quant_dot_int8(a, b), scale[None, :], bias, None, res, np.float16)
    got = capi.qgemm(_t(a, cuda_device), _t(b, cuda_device), scale=_t(scale, cuda_device),
                     bias=_t(bias, cuda_device), residual=_t(res, cuda_device),
                     out_dtype=torch.float16).cpu().numpy()
    np.testing.assert_allclose(got.astype(np.float32), ref.astype(np.float32), rtol=2e-2, atol=1e-2)
    # same fp32 chain and the reference's truncating half conversions: identical bits
    np.testing.assert_array_equal(got, ref)


FP8_SHAPES = [(128, 128, 128), (16, 4096, 4096), (1, 512, 256), (200, 328, 1040), (1024, 512, 4096)]


@pytest.mark.parametrize("M,N,K", FP8_SHAPES)
def test_quant_dot_fp8(cuda_device, M, N, K):
    """config-3 shaped: fp8 e4m3fn operands, fp32 accumulate, DQ + bias + gelu."""
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    af = rng.normal(0, 1, size=(M, K)).astype(np.float32)
    bf = rng.normal(0, 1, size=(K, N)).astype(np.float32)
    sa = np.float32(np.abs(af).max() / 448.0)
    sb = np.float32(np.abs(bf).max() / 448.0)
    aq = O.quantizelinear(af, sa, None, "fp8e4m3fn")
    bq = O.quantizelinear(bf, sb, None, "fp8e4m3fn")
    bias = rng.normal(0, 0.1, size=N).astype(np.float32)
    acc = O.quant_dot_fp8(aq, bq)
    scale = np.array([sa * sb], dtype=np.float32)
    ref = O.qlinear_epilogue(acc, scale, bias, "gelu_erf")
    a_t = _t(aq, cuda_device).view(torch.float8_e4m3fn)
    b_t = _t(bq, cuda_device).view(torch.float8_e4m3fn)
    raw = capi.qgemm(a_t, b_t, out_dtype=torch.float32).cpu().numpy()
    # un-dequantised accumulators are O(1e5..1e6) here: fp32 accumulation of exact
    # products differs from the oracle's double accumulation only by summation rounding
    assert np.max(np.abs(raw - acc)) <= 2e-6 * np.abs(acc).max()
    got = capi.qgemm(a_t, b_t, scale=_t(scale, cuda_device), bias=_t(bias, cuda_device),
                     act="gelu_erf", out_dtype=torch.float32).cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=2e-2, atol=1e-2)


def test_qgemm_rejects_bad_arguments(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    a = torch.zeros((16, 24), dtype=torch.int8, device=cuda_device)  # K % 16 != 0
    b = torch.zeros((24, 16), dtype=torch.int8, device=cuda_device)
    with pytest.raises(capi.MgxError) as e:
        capi.qgemm(a, b)
    assert e.value.code == capi.E_ALIGNMENT
    a = torch.zeros((16, 32), dtype=torch.int8, device=cuda_device)
    b = torch.zeros((32, 16), dtype=torch.int8, device=cuda_device)
    with pytest.raises(capi.MgxError) as e:
        capi.qgemm(a, b, workspace=torch.empty(8, dtype=torch.uint8, device=cuda_device))
    assert e.value.code == capi.E_WORKSPACE


@pytest.mark.parametrize("out", ["f16", "f32"])
@pytest.mark.parametrize("qtype", ["int8", "fp8e4m3fn"])
@pytest.mark.parametrize("write_d", [True, False])
def test_qlinear_fused_output_quantizelinear(cuda_device, out, qtype, write_d):
    """dequantizelinear -> add -> relu -> quantizelinear in one epilogue: the quantised tensor is
    bit-identical to quantizelinear applied to the stored result."""
    import torch
    from amdmigraphx_b200 import capi
    M, N, K = 200, 328, 512
    rng = np.random.default_rng(21)
    a = _rand_i8(rng, (M, K))
    b = _rand_i8(rng, (K, N))
    scale = rng.uniform(1e-5, 1e-4, size=N).astype(np.float32)
    bias = rng.normal(0, 0.1, size=N).astype(np.float32)
    odt_np, odt = (np.float16, torch.float16) if out == "f16" else (np.float32, torch.float32)
    y_ref = O.qlinear_epilogue(O.quant_dot_int8(a, b), scale[None, :], bias, "relu", None, odt_np)
    q_scale = odt_np(0.0125)
    q_ref = O.quantizelinear(y_ref, np.array([q_scale], dtype=odt_np), None, qtype)
    qdt = torch.int8 if qtype == "int8" else torch.float8_e4m3fn
    q = torch.zeros((M, N), dtype=qdt, device=cuda_device)
    y = torch.full((M, N), 7.0, dtype=odt, device=cuda_device)
    capi.qgemm(_t(a, cuda_device), _t(b, cuda_device), scale=_t(scale, cuda_device),
               bias=_t(bias, cuda_device), act="relu", out=y, q_out=q, q_scale=float(q_scale),
               write_d=write_d)
    np.testing.assert_array_equal(q.view(torch.uint8).cpu().numpy(), q_ref.view(np.uint8))
    if write_d:
        np.testing.assert_array_equal(y.cpu().numpy(), y_ref)
    else:
        assert float(y.min()) == 7.0 and float(y.max()) == 7.0  # untouched


# ---------------------------------------------------------------- at most 16 rows: weight-streaming kernel
SKINNY = [(1, 256, 512), (5, 1000, 2064), (16, 4096, 4096), (3, 130, 48), (16, 20000, 1024), (2, 384, 11008)]


@pytest.mark.parametrize("M,N,K", SKINNY)
def test_skinny_quant_dot_int8_bit_exact(cuda_device, M, N, K):
    """[N,K] weights, decode-sized M: split-K partial sums are integers, the result is exact."""
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + N + K)
    a = _rand_i8(rng, (M, K))
    w = _rand_i8(rng, (N, K))
    got = capi.qgemm(_t(a, cuda_device), _t(w, cuda_device), b_layout=capi.B_NK)
    assert got.dtype == torch.int32
    np.testing.assert_array_equal(got.cpu().numpy(), O.quant_dot_int8(a, w.T))


@pytest.mark.parametrize("act", [None, "relu", "gelu_erf"])
@pytest.mark.parametrize("scale_kind,out", [("tensor", "f32"), ("col", "f32"), ("col", "f16")])
def test_skinny_qlinear_int8_fused_epilogue(cuda_device, act, scale_kind, out):
    import torch
    from amdmigraphx_b200 import capi
    M, N, K = 8, 3072, 768
    rng = np.random.default_rng(3)
    a = _rand_i8(rng, (M, K))
    w = _rand_i8(rng, (N, K))
    if scale_kind == "tensor":
        scale = np.array([1e-4], dtype=np.float32)
        sview, mode = scale, capi.SCALE_PER_TENSOR
    else:
        scale = rng.uniform(2e-5, 2e-4, size=N).astype(np.float32)
        sview, mode = scale[None, :], capi.SCALE_PER_COL
    bias = rng.normal(0, 0.1, size=N).astype(np.float32)
    odt = np.float32 if out == "f32" else np.float16
    ref = O.qlinear_epilogue(O.quant_dot_int8(a, w.T), sview, bias, act, None, odt)
    got = capi.qgemm(_t(a, cuda_device), _t(w, cuda_device), b_layout=capi.B_NK,
                     scale=_t(scale, cuda_device), scale_mode=mode, bias=_t(bias, cuda_device), act=act,
                     out_dtype=torch.float32 if out == "f32" else torch.float16).cpu().numpy()
    if act in (None, "relu"):
        np.testing.assert_array_equal(got, ref)
    elif out == "f32":
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=3e-6)
    else:
        np.testing.assert_allclose(got.astype(np.float32), ref.astype(np.float32), rtol=2e-3, atol=1e-3)


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 1536, 8192), (7, 200, 336)])
def test_skinny_quant_dot_fp8(cuda_device, M, N, K):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    af = rng.normal(0, 1, size=(M, K)).astype(np.float32)
    wf = rng.normal(0, 1, size=(N, K)).astype(np.float32)
    sa = np.float32(np.abs(af).max() / 448.0)
    sw = np.float32(np.abs(wf).max() / 448.0)
    aq = O.quantizelinear(af, sa, None, "fp8e4m3fn")
    wq = O.quantizelinear(wf, sw, None, "fp8e4m3fn")
    bias = rng.normal(0, 0.1, size=N).astype(np.float32)
    acc = O.quant_dot_fp8(aq, np.ascontiguousarray(wq.T))
    scale = np.array([sa * sw], dtype=np.float32)
    ref = O.qlinear_epilogue(acc, scale, bias, "gelu_erf")
    a_t = _t(aq, cuda_device).view(torch.float8_e4m3fn)
    w_t = _t(wq, cuda_device).view(torch.float8_e4m3fn)
    raw = capi.qgemm(a_t, w_t, b_layout=capi.B_NK, out_dtype=torch.float32).cpu().numpy()
    assert np.max(np.abs(raw - acc)) <= 2e-6 * np.abs(acc).max()
    got = capi.qgemm(a_t, w_t, b_layout=capi.B_NK, scale=_t(scale, cuda_device),
                     scale_mode=capi.SCALE_PER_TENSOR, bias=_t(bias, cuda_device), act="gelu_erf",
                     out_dtype=torch.float32).cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=2e-2, atol=1e-2)


def test_skinny_without_workspace_runs_as_tiles(cuda_device):
    """The workspace is optional for [N,K] weights: without it the tiled kernel takes the call."""
    import ctypes
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(9)
    a = _rand_i8(rng, (4, 256))
    w = _rand_i8(rng, (384, 256))
    lib = capi.load()
    at, wt = _t(a, cuda_device), _t(w, cuda_device)
    d = torch.empty((4, 384), dtype=torch.int32, device=cuda_device)
    desc = capi.QgemmDesc(M=4, N=384, K=256, batch=1, lda=256, ldb=256, ldd=384, stride_a=0, stride_b=0,
                          stride_d=0, ab_type=capi.I8, out_type=capi.I32, b_layout=capi.B_NK,
                          scale_mode=capi.SCALE_NONE, act=0, flags=0)
    assert lib.mgx_cuda_qgemm_workspace(ctypes.byref(desc)) > 0
    capi.check(lib.mgx_cuda_qgemm(ctypes.byref(desc), capi._ptr(at), capi._ptr(wt), capi._ptr(d), None,
                                  None, None, None, 0, capi._stream()), "mgx_cuda_qgemm")
    np.testing.assert_array_equal(d.cpu().numpy(), O.quant_dot_int8(a, w.T))


@pytest.mark.parametrize("act", [None, "relu"])
def test_qlinear_int8_fp16_tiny_outputs_bit_exact(cuda_device, act):
    """fp16 outputs in the subnormal range of a half (and exact zeros from relu), with a residual
    and a fused quantizelinear so that every truncation site of the epilogue sees them."""
    import torch
    from amdmigraphx_b200 import capi
    M, N, K = 256, 512, 256
    rng = np.random.default_rng(21)
    a = _rand_i8(rng, (M, K))
    w = _rand_i8(rng, (N, K))
    # accumulators ~1e5 x scales 1e-11..1e-9 -> |values| from 1e-8 to 1e-4
    scale = (10.0 ** rng.uniform(-11, -9, size=N)).astype(np.float32)
    bias = (rng.normal(0, 1, size=N) * 1e-6).astype(np.float32)
    res = (rng.normal(0, 1, size=(M, N)) * 3e-6).astype(np.float16)
    acc = O.quant_dot_int8(a, w.T)
    ref = O.qlinear_epilogue(acc, scale[None, :], bias, act, res, np.float16)
    got = capi.qgemm(_t(a, cuda_device), _t(w, cuda_device), b_layout=capi.B_NK, scale=_t(scale, cuda_device),
                     bias=_t(bias, cuda_device), act=act, residual=_t(res, cuda_device),
                     out_dtype=torch.float16).cpu().numpy()
    assert np.count_nonzero(np.abs(ref.astype(np.float32)) < 6.1e-5) > ref.size // 2
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("M,N,K,act,res", [(384, 3072, 768, "gelu_erf", False), (256, 768, 3072, None, True),
                                           (130, 200, 96, "gelu_erf", True), (384, 768, 768, "relu", False)])
def test_int8_half_math_epilogue_matches_half_operator_chain(cuda_device, M, N, K, act, res):
    """fp16 model: after dequantizelinear the value is converted to half and bias add, erf-GELU and
    residual add are half operators, each rounding (truncating) to half.  With MGX_QGEMM_HALF_MATH
    the fused epilogue makes the same roundings: identical bits except where the kernel's erf and
    its multiplication by 1 / half(sqrt 2) land in the neighbouring half (< 0.1 % of the elements,
    one half step)."""
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + N)
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    scale = (0.03 * rng.uniform(0.4, 1.2, size=N) / (127.0 * np.sqrt(K))).astype(np.float32)
    bias = rng.normal(0, 0.2, size=N).astype(np.float16)
    resid = rng.normal(0, 1, size=(M, N)).astype(np.float16) if res else None
    t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(cuda_device)  # noqa: E731
    got = capi.qgemm(t(a), t(b), b_layout=capi.B_NK, scale=t(scale), bias=t(bias.astype(np.float32)), act=act,
                     residual=None if resid is None else t(resid), out_dtype=torch.float16, half_math=True)
    torch.cuda.synchronize()
    ref = O.qlinear_epilogue_half_chain(O.quant_dot_int8(a, b.T), scale[None, :], bias, act, resid)
    g, r = got.cpu().numpy(), ref
    diff = g.view(np.uint16) != r.view(np.uint16)
    if act == "gelu_erf":
        assert diff.mean() < 1e-3
        np.testing.assert_allclose(g.astype(np.float32), r.astype(np.float32), rtol=2e-3, atol=1e-6)
    else:
        assert not diff.any()


@pytest.mark.parametrize("M,N,K,act", [(256, 320, 256, "gelu_erf"), (128, 64, 768, "relu"), (384, 3072, 768, "gelu_erf"),
                                         (128, 128, 2048, "gelu_erf")])
def test_int8_lut_epilogue_is_the_half_operator_chain(cuda_device, M, N, K, act):
    """fp16 model whose linear feeds only the next quantizelinear: activation + quantizelinear of the
    half the chain holds after the bias is one look-up in a 65536-entry table (MGX_QOUT_LUT).  With a
    table made by the reference's arithmetic the int8 tensor is the operator chain's bit for bit; the
    arithmetic epilogue differs from it only where its erf lands in the neighbouring half."""
    import warnings
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(M + N + 1)
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    b = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    scale = (2.0 * rng.uniform(0.4, 1.2, size=N) / (127.0 * np.sqrt(K))).astype(np.float32)
    bias = rng.normal(0, 0.2, size=N).astype(np.float16)
    q_scale = np.float16(0.03)
    halves = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    with warnings.catch_warnings(), np.errstate(all="ignore"):
        warnings.simplefilter("ignore")
        acted = O.qlinear_epilogue_half_chain(halves.astype(np.float32), np.float32(1.0), None, act)
        table = O.quantizelinear(acted, np.array([q_scale]), None, "int8")
    t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(cuda_device)  # noqa: E731
    outs = []
    for lut in (None, t(table)):
        q = torch.empty((M, N), dtype=torch.int8, device=cuda_device)
        capi.qgemm(t(a), t(b), b_layout=capi.B_NK, scale=t(scale), bias=t(bias.astype(np.float32)), act=act,
                   out_dtype=torch.float16, half_math=True, q_out=q, q_scale=float(q_scale), write_d=False, lut=lut)
        torch.cuda.synchronize()
        outs.append(q.cpu().numpy())
    v = O.qlinear_epilogue_half_chain(O.quant_dot_int8(a, b.T), scale[None, :], bias, act)
    ref = O.quantizelinear(v, np.array([q_scale]), None, "int8")
    np.testing.assert_array_equal(outs[1], ref)
    d = np.abs(outs[0].astype(np.int32) - ref.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 2e-3
    assert capi.device_status() == 0
