"""CPU restatement (numpy) of MIGraphX's quantized-GEMM arithmetic.

TEST INFRASTRUCTURE ONLY.  Nothing in the product imports this module: it is the
checker used by tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline
leg.  Every function restates one operator of the reference and cites the lines it
follows (paths relative to the MIGraphX source tree).  The restatement is pinned
bit for bit against MIGraphX's own `ref` target built from the reference sources
(oracle/_ref, see oracle/build_ref.py): live in tests/test_oracle_vs_ref_target.py and
tests/test_oracle_chains_vs_ref_target.py, and through the committed fixtures
tests/golden/ref_fixtures.npz (made by tests/golden/make_golden.py).  The reference's
own golden tests (test/ref/*.cpp) run against that build in
tests/test_reference_golden_tests.py, and the known answers of its MatMulNBits tests
(test/onnx/verify/matmulnbits_tests.cpp, extracted into tests/golden/matmulnbits_goldens.json)
pin the int4 operators in tests/test_oracle_golden.py.
"""
import numpy as np

# ----------------------------------------------------------------------------- fp8 e4m3fn
# Format: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinities; 0x7F / 0xFF are NaN;
# largest finite value 448 (src/include/migraphx/float8.hpp:83-112,
# src/include/migraphx/float8_impl.hpp:38-245).


def _e4m3fn_table():
    vals = np.zeros(256, dtype=np.float64)
    for code in range(256):
        s = -1.0 if code & 0x80 else 1.0
        e = (code >> 3) & 0xF
        m = code & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        vals[code] = v
    return vals


E4M3FN_VALUES = _e4m3fn_table()
_POS = E4M3FN_VALUES[:0x7F]  # codes 0x00..0x7E: 0 .. 448, increasing
_MID = (_POS[:-1] + _POS[1:]) / 2.0


def fp8e4m3fn_decode(codes):
    """uint8 bit patterns -> float32 values."""
    return E4M3FN_VALUES[np.asarray(codes, dtype=np.uint8)].astype(np.float32)


def fp8e4m3fn_encode(x):
    """float -> uint8 bit patterns, round-to-nearest-even, for |x| <= 448
    (the cast of float8_impl.hpp:195-245 without clipping or stochastic rounding).
    NaN -> 0x7F with the sign bit kept."""
    x = np.asarray(x, dtype=np.float64)
    ax = np.abs(x)
    idx = np.searchsorted(_MID, ax, side="left")  # first midpoint >= |x|
    idx = np.minimum(idx, len(_POS) - 1)
    # exact tie with the midpoint above code idx: take the even code
    tie = (idx < len(_MID)) & (ax == _MID[np.minimum(idx, len(_MID) - 1)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)
    code = idx.astype(np.uint8)
    code = np.where(np.isnan(x), np.uint8(0x7F), code)
    sign = np.signbit(x).astype(np.uint8) << 7
    return (code | sign).astype(np.uint8)


# ----------------------------------------------------------------------------- fp16
def half_trunc(x):
    """float -> float16 the way migraphx::half does it: the float32 mantissa is shifted
    right, i.e. rounded TOWARD ZERO, not to nearest; float exponents beyond the half range
    give infinity (src/include/migraphx/generic_float.hpp:180-230).  A double is first
    converted to float32 (round to nearest) by the language."""
    x = np.asarray(x).astype(np.float32)
    with np.errstate(over="ignore"):
        h = x.astype(np.float16)  # round to nearest even
    hf = h.astype(np.float32)
    over = (np.abs(hf) > np.abs(x)) & (np.abs(x) < 65536.0)
    bits = h.view(np.uint16).copy()
    bits[over] -= 1  # one step toward zero on the sign-magnitude pattern
    return bits.view(np.float16).reshape(x.shape)


# ----------------------------------------------------------------------------- quantizelinear
def quantizelinear(x, scale, zp=None, out_type="int8"):
    """src/include/migraphx/op/quantizelinear.hpp:71-108.

    Integer targets: nearbyint(x / scale) with the division in the INPUT type and
    round-half-even, + zero point in double, clamp to the type's range.
    fp8 target: double(x)/double(scale) + zp, clamp to +-448, one RNE cast.
    `scale` / `zp` broadcast against x like MIGraphX's broadcast views.
    out_type: 'int8' | 'uint8' | 'fp8e4m3fn' (returned as uint8 bit patterns)."""
    x = np.asarray(x)
    scale = np.broadcast_to(np.asarray(scale, dtype=x.dtype), x.shape)
    if out_type in ("int8", "uint8"):
        lo, hi = (-128.0, 127.0) if out_type == "int8" else (0.0, 255.0)
        z = np.zeros(x.shape) if zp is None else np.broadcast_to(np.asarray(zp), x.shape).astype(np.float64)
        with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
            if x.dtype == np.float16:
                # half / half = half(float(a) / float(b)) with the truncating conversion
                # (generic_float.hpp:321-329)
                q = half_trunc(x.astype(np.float32) / scale.astype(np.float32))
            else:
                q = x / scale
        q = np.rint(q.astype(np.float64)) + z
        # std::max(min, std::min(max, q)) : a NaN q ends up at max
        q = np.where(np.isnan(q), hi, q)
        q = np.maximum(lo, np.minimum(hi, q))
        return q.astype(np.int8 if out_type == "int8" else np.uint8)
    if out_type == "fp8e4m3fn":
        z = 0.0 if zp is None else fp8e4m3fn_decode(np.broadcast_to(np.asarray(zp), x.shape)).astype(np.float64)
        with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
            q = x.astype(np.float64) / scale.astype(np.float64) + z
        q = np.where(np.isnan(q), 448.0, q)
        q = np.maximum(-448.0, np.minimum(448.0, q))
        # double -> float -> fp8: the float step is exact enough not to matter for a
        # 3-bit mantissa except on ties, which the float rounding preserves
        return fp8e4m3fn_encode(q.astype(np.float32))
    raise ValueError(out_type)


# ----------------------------------------------------------------------------- dequantizelinear
def dequantizelinear(x, scale, zp=None, x_is_fp8=False):
    """src/include/migraphx/op/dequantizelinear.hpp:60-82:
    y = (double(x) - double(zp)) * scale, stored in scale's type."""
    scale = np.asarray(scale)
    xv = fp8e4m3fn_decode(x).astype(np.float64) if x_is_fp8 else np.asarray(x).astype(np.float64)
    if zp is None:
        zv = 0.0
    else:
        zv = fp8e4m3fn_decode(zp).astype(np.float64) if x_is_fp8 else np.asarray(zp).astype(np.float64)
    s = np.broadcast_to(scale, xv.shape).astype(np.float64)
    y = (xv - zv) * s
    if scale.dtype == np.float16:
        return half_trunc(y)  # double -> float (nearest) -> half (toward zero)
    return y.astype(scale.dtype)


# ----------------------------------------------------------------------------- int4
def unpack_int4(packed, signed=False):
    """src/include/migraphx/op/unpack_int4.hpp:75-120, last axis:
    out[..., 2i] = low nibble, out[..., 2i+1] = high nibble; int8 sign-extends."""
    b = np.asarray(packed).astype(np.uint8)
    lo = b & 0xF
    hi = b >> 4
    out = np.stack([lo, hi], axis=-1).reshape(b.shape[:-1] + (b.shape[-1] * 2,))
    if signed:
        out = ((out.astype(np.int16) ^ 8) - 8).astype(np.int8)
    return out


def pack_int4(x, signed=False):
    """src/include/migraphx/op/pack_int4.hpp:79-123: clip to the 4-bit range, then
    out[..., i] = (x[..., 2i+1] << 4) | (x[..., 2i] & 0xF)."""
    x = np.asarray(x)
    if signed:
        c = np.clip(x.astype(np.int16), -8, 7).astype(np.int8).view(np.uint8)
    else:
        c = np.minimum(x.astype(np.uint8), 15)
    lo = c[..., 0::2] & 0xF
    hi = c[..., 1::2]
    out = ((hi.astype(np.uint16) << 4) | lo).astype(np.uint8)
    return out.view(np.int8) if signed else out


# ----------------------------------------------------------------------------- quant_dot
def quant_dot_int8(a, b):
    """ref_quant_gemm -> gemm_naive (src/targets/ref/lowering.cpp:205-249,
    src/gemm.cpp:43-63) for int8 operands: exact sum of products, stored as int32.
    a [..., M, K], b [..., K, N]."""
    a = np.asarray(a)
    b = np.asarray(b)
    # float64 matmul is exact here: |sum| <= 128*128*K < 2^53
    c = np.matmul(a.astype(np.float64), b.astype(np.float64))
    return c.astype(np.int64).astype(np.int32)


def quant_dot_fp8(a_codes, b_codes):
    """Same routine for fp8 e4m3fn operands (bit patterns in, float32 out):
    double accumulate, one rounding to float (src/gemm.cpp:55-61)."""
    a = fp8e4m3fn_decode(a_codes).astype(np.float64)
    b = fp8e4m3fn_decode(b_codes).astype(np.float64)
    return np.matmul(a, b).astype(np.float32)


# ----------------------------------------------------------------------------- pointwise pieces
_LIBM = None


def _erff(x):
    """erf evaluated by the C library's single-precision erff, which is what the erf
    operator's std::erf(float) resolves to on the ref target
    (src/include/migraphx/op/erf.hpp); it is not correctly rounded, so a double-precision
    erf rounded to float would differ in the last bit for some inputs."""
    global _LIBM
    import ctypes
    import ctypes.util
    if _LIBM is None:
        _LIBM = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
        _LIBM.erff.restype = ctypes.c_float
        _LIBM.erff.argtypes = [ctypes.c_float]
    x = np.asarray(x, dtype=np.float32)
    f = _LIBM.erff
    return np.fromiter((f(float(v)) for v in x.ravel()), dtype=np.float32, count=x.size).reshape(x.shape)


def gelu_erf(x):
    """(x*0.5) * (erf(x / sqrt(2)) + 1) evaluated op by op in float32
    (src/op/builder/gelu.cpp:58-74)."""
    x = np.asarray(x, dtype=np.float32)
    half = (x * np.float32(0.5)).astype(np.float32)
    d = (x / np.float32(np.sqrt(2.0))).astype(np.float32)
    e = _erff(d)
    return (half * (e + np.float32(1.0)).astype(np.float32)).astype(np.float32)


def apply_act(x, act):
    if act in (None, "none"):
        return x
    if act == "relu":
        return np.maximum(x, x.dtype.type(0))
    if act == "gelu_erf":
        return gelu_erf(x)
    if act == "gelu_tanh":
        x64 = x.astype(np.float64)
        return (0.5 * x64 * (1.0 + np.tanh(0.7978845608028654 * (x64 + 0.044715 * x64 ** 3)))).astype(x.dtype)
    if act == "silu":
        x64 = x.astype(np.float64)
        return (x64 / (1.0 + np.exp(-x64))).astype(x.dtype)
    raise ValueError(act)


def qlinear_epilogue(acc, scale=None, bias=None, act=None, residual=None, out_dtype=np.float32):
    """The instruction chain simplify_qdq + the model leave after quant_dot
    (src/simplify_qdq.cpp:243-287): dequantizelinear(acc, scale) -> add(bias) ->
    activation -> add(residual), each a separate fp32 operation; a final convert
    when the model runs in fp16."""
    acc = np.asarray(acc)
    if scale is None:
        v = acc.astype(np.float32)
    else:
        v = dequantizelinear(acc, np.asarray(scale, dtype=np.float32))
    if bias is not None:
        v = (v + np.asarray(bias, dtype=np.float32)).astype(np.float32)
    v = apply_act(v, act)
    if np.dtype(out_dtype) == np.float16:
        # fp16 model: convert (truncating, see half_trunc) and then add in half arithmetic
        v = half_trunc(v)
        if residual is not None:
            v = half_trunc(v.astype(np.float32) + np.asarray(residual).astype(np.float32))
        return v
    if residual is not None:
        v = (v + np.asarray(residual).astype(np.float32)).astype(np.float32)
    return v.astype(out_dtype)


# ----------------------------------------------------------------------------- weight-only int4
def w4a16_dequant_weights(bp, scales, zp=None, zp_const=8, group=128):
    """unpack_int4 + dequantizelinear to fp16 as src/onnx/parse_matmulnbits.cpp:85-158
    builds them: W[n,k] = half((q[n,k] - zp[n,k/group]) * s[n,k/group]), with MIGraphX's
    truncating float -> half conversion."""
    q = unpack_int4(bp).astype(np.float64)  # [N, K]
    n, k = q.shape
    s = np.repeat(np.asarray(scales, dtype=np.float16).reshape(n, k // group), group, axis=1)
    if zp is None:
        z = float(zp_const)
    else:
        z = np.repeat(np.asarray(zp).reshape(n, k // group), group, axis=1).astype(np.float64)
    return half_trunc((q - z) * s.astype(np.float64))


def w4a16_linear(a, bp, scales, zp=None, zp_const=8, group=128, act=None):
    """dot(A_fp16[M,K], transpose(W_fp16[N,K])) with gemm_naive's double accumulation
    and one (truncating) conversion to half (src/gemm.cpp:55-61)."""
    w = w4a16_dequant_weights(bp, scales, zp, zp_const, group)
    acc = np.matmul(np.asarray(a, dtype=np.float16).astype(np.float64), w.astype(np.float64).T)
    if act not in (None, "none"):
        acc = apply_act(acc.astype(np.float32), act).astype(np.float64)
    return half_trunc(acc)


# ----------------------------------------------------------------------------- LayerNorm / attention chains
def _as_type(x, dtype):
    """A double result stored in the operator's output type (half: truncating)."""
    return half_trunc(x) if np.dtype(dtype) == np.float16 else np.asarray(x).astype(dtype)


def layernorm_chain(x, gamma=None, beta=None, eps=1e-5):
    """The instruction chain the ONNX parser emits for LayerNormalization over the last axis
    (src/onnx/parse_layernorm.cpp:100-140), operator by operator in x's type: reduce_mean sums in
    double and stores in x's type (src/include/migraphx/op/reduce_op.hpp:180-203), every
    element-wise operator computes in fp32 / double and stores in x's type (fp16: truncating)."""
    x = np.asarray(x)
    dt = x.dtype
    f = lambda a: np.asarray(a).astype(np.float64)  # noqa: E731
    n = x.shape[-1]
    mean = _as_type(f(x).sum(axis=-1, keepdims=True) / n, dt)
    d = _as_type(f(x).astype(np.float32) - f(mean).astype(np.float32), dt)
    dd = _as_type(f(d).astype(np.float32) * f(d).astype(np.float32), dt)
    var = _as_type(f(dd).sum(axis=-1, keepdims=True) / n, dt)
    ve = _as_type(f(var).astype(np.float32) + np.float32(_as_type(np.float64(eps), dt)), dt)
    rs = _as_type(np.float32(1.0) / np.sqrt(f(ve).astype(np.float32)), dt)
    y = _as_type(f(d).astype(np.float32) * f(rs).astype(np.float32), dt)
    if gamma is not None:
        y = _as_type(f(y).astype(np.float32) * f(gamma).astype(np.float32), dt)
    if beta is not None:
        y = _as_type(f(y).astype(np.float32) + f(beta).astype(np.float32), dt)
    return y


def attention_chain(q, k, v, batch, seq, heads, scale):
    """reshape -> transpose -> dot -> mul(scale) -> softmax -> dot -> transpose -> reshape on fp16
    [batch*seq, heads*d] matrices, every operator storing half (truncating): dot accumulates in
    double (src/gemm.cpp:55-61), softmax as ref_softmax (src/targets/ref/lowering.cpp:253-320:
    exp(x - max) stored in half, summed in fp32, divided in half arithmetic)."""
    q, k, v = (np.asarray(a, dtype=np.float16) for a in (q, k, v))
    d = q.shape[1] // heads
    hd = lambda a: a.reshape(batch, seq, heads, d).transpose(0, 2, 1, 3).astype(np.float64)  # noqa: E731
    qh, kh, vh = hd(q), hd(k), hd(v)
    sc = half_trunc(np.matmul(qh, kh.transpose(0, 1, 3, 2)))
    ss = half_trunc(sc.astype(np.float32) * np.float32(np.float16(scale)))
    mx = ss.astype(np.float32).max(axis=-1, keepdims=True)
    e = half_trunc(np.exp((ss.astype(np.float32) - mx).astype(np.float32)))
    tot = e.astype(np.float32).sum(axis=-1, keepdims=True, dtype=np.float32)
    p = half_trunc(e.astype(np.float32) / tot)
    o = half_trunc(np.matmul(p.astype(np.float64), vh))
    return np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(batch * seq, heads * d)


def concat_past_present(present, seqlens, past):
    """op::concat_past_present::compute (src/include/migraphx/op/concat_past_present.hpp:84-155): the
    chunk of `seq` rows of every (batch entry, KV head) goes to row seqlens[b] of the cache when seq == 1,
    to row 0 otherwise; returns the updated cache."""
    out = np.array(past, copy=True)
    batch, kvh, seq, _ = present.shape
    for b in range(batch):
        pos = int(np.asarray(seqlens).reshape(-1)[b]) if seq == 1 else 0
        out[b, :, pos:pos + seq, :] = present[b]
    return out


def gqa_rotary_embedding(qkv, seqlens, cos_cache, sin_cache, heads, kv_heads, interleaved=False):
    """op::gqa_rotary_embedding::compute (src/include/migraphx/op/gqa_rotary_embedding.hpp:72-221) on
    packed fp16 [batch, heads + 2 kv_heads, seq, head]: x * cos is a half product (truncated),
    sign * x' * sin stays fp32, the sum is stored as half; V heads pass through."""
    qkv = np.asarray(qkv, dtype=np.float16)
    out = qkv.copy()
    batch, _, seq, head = qkv.shape
    rot = 2 * cos_cache.shape[1]
    half = rot // 2
    i = np.arange(rot)
    if interleaved:
        ci, sign, j = (i // 2) % half, np.where(i % 2 == 0, -1.0, 1.0), np.where(i % 2 == 0, i + 1, i - 1)
    else:
        ci, sign, j = i % half, np.where(i < half, -1.0, 1.0), (i + half) % rot
    for b in range(batch):
        for s_ in range(seq):
            pos = int(np.asarray(seqlens).reshape(-1)[b]) if seq == 1 else s_
            c = cos_cache[pos, ci].astype(np.float32)
            sn = sin_cache[pos, ci].astype(np.float32)
            x = qkv[b, :heads + kv_heads, s_, :rot].astype(np.float32)
            t1 = half_trunc(x * c).astype(np.float32)
            t2 = (sign.astype(np.float32) * x[:, j]) * sn
            out[b, :heads + kv_heads, s_, :rot] = half_trunc(t1 + t2)
    return out


def rotary_builder_chain(x, positions, cos_cache, sin_cache):
    """The rotary_embedding builder's rotation (src/op/builder/rotary_embedding.cpp:60-230,
    non-interleaved) on fp16 x [batch, heads, seq, head]: cos / sin rows gathered at positions
    [batch, seq] and doubled; mul(x, cos), mul(signs, sin), mul(rotate_half(x), .), add - every
    operator stores half (truncating)."""
    x = np.asarray(x, dtype=np.float16)
    half = x.shape[3] // 2
    pos = np.asarray(positions).reshape(x.shape[0], x.shape[2])
    c = np.concatenate([cos_cache[pos], cos_cache[pos]], axis=-1)[:, None, :, :].astype(np.float32)
    sn = np.concatenate([sin_cache[pos], sin_cache[pos]], axis=-1)[:, None, :, :].astype(np.float32)
    signs = np.concatenate([-np.ones(half, np.float32), np.ones(half, np.float32)])
    rot = np.concatenate([x[..., half:], x[..., :half]], axis=-1).astype(np.float32)
    t1 = half_trunc(x.astype(np.float32) * c).astype(np.float32)
    ms = half_trunc(signs * sn).astype(np.float32)
    t2 = half_trunc(rot * ms).astype(np.float32)
    return half_trunc(t1 + t2)


def rmsnorm_chain(x, gamma, eps):
    """SimplifiedLayerNormalization as the parser decomposes it
    (src/onnx/parse_simplified_layer_normalization.cpp:91-106) on fp16 rows: squares and their mean in
    fp32 (reduce_mean accumulates in double), the mean, mean + eps, rsqrt and the two products stored
    in half (truncating)."""
    x = np.asarray(x, dtype=np.float16)
    fx = x.astype(np.float32)
    ms = half_trunc(((fx * fx).astype(np.float64).sum(axis=-1, keepdims=True) / x.shape[-1]).astype(np.float32))
    ve = half_trunc(ms.astype(np.float32) + np.float32(np.float16(half_trunc(np.float32(eps)))))
    rr = half_trunc(np.float32(1.0) / np.sqrt(ve.astype(np.float32)))
    y = half_trunc(fx * rr.astype(np.float32))
    return half_trunc(y.astype(np.float32) * np.asarray(gamma, dtype=np.float16).astype(np.float32))


def gqa_decode_chain(q, k_cache, v_cache, seqlens, scale):
    """The decode step of GroupQueryAttention as the parser decomposes it
    (src/onnx/parse_group_query_attention.cpp:184-262) on fp16: q [batch, heads, head] against caches
    [batch, kv_heads, T, head]; positions beyond seqlens[b] masked with -inf; every operator stores
    half (truncating); returns [batch, heads * head]."""
    q = np.asarray(q, dtype=np.float16)
    batch, heads, head = q.shape
    kvh, t = k_cache.shape[1], k_cache.shape[2]
    rep = heads // kvh
    out = np.zeros((batch, heads * head), dtype=np.float16)
    for b in range(batch):
        n = int(np.asarray(seqlens).reshape(-1)[b]) + 1
        for h in range(heads):
            kk = k_cache[b, h // rep, :n].astype(np.float64)
            vv = v_cache[b, h // rep, :n].astype(np.float64)
            sc = half_trunc(kk @ q[b, h].astype(np.float64))
            ss = half_trunc(sc.astype(np.float32) * np.float32(np.float16(scale))).astype(np.float32)
            e = half_trunc(np.exp((ss - ss.max()).astype(np.float32)))
            tot = e.astype(np.float32).sum(dtype=np.float32)
            p = half_trunc(e.astype(np.float32) / tot)
            out[b, h * head:(h + 1) * head] = half_trunc(p.astype(np.float64) @ vv)
    return out


def qlinear_epilogue_half_chain(acc, scale, bias=None, act=None, residual=None):
    """The operators after quant_dot in an fp16 model (src/simplify_qdq.cpp:283-287):
    dequantizelinear in fp32, convert to half, then add(bias), the erf-GELU chain of
    src/op/builder/gelu.cpp:58-74 and add(residual) as HALF operators - every one computes in fp32
    and stores half (truncating)."""
    f32 = lambda a: np.asarray(a).astype(np.float32)  # noqa: E731
    v = half_trunc(dequantizelinear(np.asarray(acc), np.asarray(scale, dtype=np.float32)))
    if bias is not None:
        v = half_trunc(f32(v) + f32(np.asarray(bias, dtype=np.float16)))
    if act == "gelu_erf":
        mh = half_trunc(f32(v) * np.float32(0.5))
        dv = half_trunc(f32(v) / f32(half_trunc(np.float32(np.sqrt(2.0)))))
        er = half_trunc(_erff(f32(dv)))
        e1 = half_trunc(f32(er) + np.float32(1.0))
        v = half_trunc(f32(mh) * f32(e1))
    elif act == "relu":
        v = np.maximum(v, np.float16(0))
    elif act not in (None, "none"):
        raise ValueError(act)
    if residual is not None:
        v = half_trunc(f32(v) + f32(residual))
    return v
