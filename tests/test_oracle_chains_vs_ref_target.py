"""CPU tests: the numpy restatements of the fp16 operator CHAINS (fused epilogue of an fp16 model,
LayerNorm, RMSNorm, encoder attention, rotary embedding, KV-cache append, decode attention) against
MIGraphX's own `ref` target evaluating the same operators one by one through
oracle/_ref/lib/libmgx_ref_oracle.so.  Data movement between the operators (reshape, transpose,
slice, concat, gather, mask selection) is done in numpy; every arithmetic operator runs on ref.
Skipped where that build is not present."""
import numpy as np
import pytest

from oracle import mgx_oracle as O
from oracle import ref_target as R

pytestmark = pytest.mark.skipif(not R.available(), reason="oracle/_ref is not built here")

H = "half_type"


def _eq(a, b):
    np.testing.assert_array_equal(np.ascontiguousarray(a).view(np.uint8), np.ascontiguousarray(b).view(np.uint8))


# shape::type_t as the convert operator serialises it (src/include/migraphx/shape.hpp: bool, half, float, ...)
_TYPE_ID = {"half_type": 1, "float_type": 2}


def _convert(x, np_type, name):
    return R.run_op("convert", [np.ascontiguousarray(x)], x.shape, name, {"target_type": _TYPE_ID[name]})


def _reduce_mean_last(x):
    x = np.ascontiguousarray(x)
    t = "half_type" if x.dtype == np.float16 else "float_type"
    return R.run_op("reduce_mean", [x], x.shape[:-1] + (1,), t, {"axes": [x.ndim - 1]})


def _bin(name, a, b):
    a = np.ascontiguousarray(a)
    return R.binary(name, a, np.broadcast_to(np.asarray(b, dtype=a.dtype), a.shape))


@pytest.mark.parametrize("act,res", [(None, False), ("gelu_erf", False), ("relu", True), ("gelu_erf", True)])
def test_half_epilogue_chain(act, res):
    rng = np.random.default_rng(7)
    acc = rng.integers(-2 ** 20, 2 ** 20, size=(10, 40)).astype(np.int32)
    scale = rng.uniform(1e-6, 4e-6, size=(1, 40)).astype(np.float32)
    bias = rng.normal(0, 0.2, size=40).astype(np.float16)
    resid = rng.normal(0, 1, size=(10, 40)).astype(np.float16) if res else None
    v = R.dequantizelinear(acc, np.broadcast_to(scale, acc.shape))
    v = _convert(v, np.float16, H)
    v = _bin("add", v, bias)
    if act == "gelu_erf":
        v = R.gelu_erf(v)
    elif act == "relu":
        v = R.unary("relu", v)
    if res:
        v = _bin("add", v, resid)
    _eq(O.qlinear_epilogue_half_chain(acc, scale, bias, act, resid), v)


def test_layernorm_chain():
    rng = np.random.default_rng(8)
    x = (rng.normal(size=(6, 96)) * 2 + 0.5).astype(np.float16)
    g = rng.uniform(0.5, 1.5, size=96).astype(np.float16)
    b = rng.normal(0, 0.2, size=96).astype(np.float16)
    mean = _reduce_mean_last(x)
    d = _bin("sub", x, mean)
    var = _reduce_mean_last(_bin("mul", d, d))
    rs = R.unary("rsqrt", _bin("add", var, np.float16(1e-5)))
    y = _bin("add", _bin("mul", _bin("mul", d, rs), g), b)
    _eq(O.layernorm_chain(x, g, b, float(np.float16(1e-5))), y)


def test_rmsnorm_chain():
    rng = np.random.default_rng(9)
    x = (rng.normal(size=(5, 128)) * 1.7).astype(np.float16)
    g = rng.uniform(0.5, 1.5, size=128).astype(np.float16)
    fx = _convert(x, np.float32, "float_type")
    ms = _convert(_reduce_mean_last(_bin("mul", fx, fx)), np.float16, H)
    rr = R.unary("rsqrt", _bin("add", ms, np.float16(1e-5)))
    y = _bin("mul", _bin("mul", x, rr), g)
    _eq(O.rmsnorm_chain(x, g, 1e-5), y)


def _softmax_last(x):
    x = np.ascontiguousarray(x)
    return R.run_op("softmax", [x], x.shape, H, {"axis": x.ndim - 1})


def test_attention_chain():
    rng = np.random.default_rng(10)
    batch, seq, heads, d = 2, 24, 2, 16
    q, k, v = (rng.normal(size=(batch * seq, heads * d)).astype(np.float16) for _ in range(3))
    hd = lambda a: np.ascontiguousarray(a.reshape(batch, seq, heads, d).transpose(0, 2, 1, 3))  # noqa: E731
    sc = R.dot(hd(q), np.ascontiguousarray(hd(k).transpose(0, 1, 3, 2)))
    p = _softmax_last(_bin("mul", sc, np.float16(0.25)))
    o = R.dot(p, hd(v))
    ref = np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(batch * seq, heads * d)
    _eq(O.attention_chain(q, k, v, batch, seq, heads, 0.25), ref)


def test_rotary_builder_chain():
    rng = np.random.default_rng(11)
    batch, heads, seq, head, max_pos = 2, 3, 4, 16, 32
    x = rng.normal(size=(batch, heads, seq, head)).astype(np.float16)
    ang = np.arange(max_pos)[:, None] * (10000.0 ** (-2.0 * np.arange(head // 2) / head))[None, :]
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    pos = rng.integers(0, max_pos, size=(batch, seq))
    c = np.broadcast_to(np.concatenate([cos[pos], cos[pos]], -1)[:, None], x.shape)
    s = np.broadcast_to(np.concatenate([sin[pos], sin[pos]], -1)[:, None], x.shape)
    signs = np.broadcast_to(np.concatenate([-np.ones(head // 2), np.ones(head // 2)]).astype(np.float16), x.shape)
    rot = np.concatenate([x[..., head // 2:], x[..., :head // 2]], -1)
    y = _bin("add", _bin("mul", x, c), _bin("mul", rot, _bin("mul", signs, s)))
    _eq(O.rotary_builder_chain(x, pos, cos, sin), y)


def test_gqa_decode_chain():
    rng = np.random.default_rng(12)
    batch, heads, kvh, head, t = 2, 4, 2, 16, 40
    q = rng.normal(size=(batch, heads, head)).astype(np.float16)
    kc = rng.normal(size=(batch, kvh, t, head)).astype(np.float16)
    vc = rng.normal(size=(batch, kvh, t, head)).astype(np.float16)
    lens = np.array([[17], [39]], dtype=np.int32)
    scale = np.float16(0.25)
    kk = np.repeat(kc, heads // kvh, axis=1)
    vv = np.repeat(vc, heads // kvh, axis=1)
    sc = R.dot(np.ascontiguousarray(q[:, :, None, :]), np.ascontiguousarray(kk.transpose(0, 1, 3, 2)))
    sc = _bin("mul", sc, scale)
    mask = np.arange(t)[None, None, None, :] > lens[:, :, None, None]
    sc = np.where(np.broadcast_to(mask, sc.shape), np.float16(-np.inf), sc)  # `where` selects, it computes nothing
    o = R.dot(_softmax_last(sc), vv)
    ref = np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(batch, heads * head)
    _eq(O.gqa_decode_chain(q, kc, vc, lens, float(scale)), ref)


def test_cache_append_and_rotary_operators():
    rng = np.random.default_rng(13)
    batch, heads, kvh, head, t = 2, 4, 2, 16, 24
    # op::concat_past_present at a decode step
    present = rng.normal(size=(batch, kvh, 1, head)).astype(np.float16)
    past = rng.normal(size=(batch, kvh, t, head)).astype(np.float16)
    lens = np.array([[5], [23]], dtype=np.int32)
    got = R.run_op("concat_past_present", [present, lens, past.copy()], past.shape, H, {"kv_num_heads": kvh})
    _eq(O.concat_past_present(present, lens, past), got)
    # op::gqa_rotary_embedding on packed QKV
    qkv = rng.normal(size=(batch, heads + 2 * kvh, 1, head)).astype(np.float16)
    ang = np.arange(t)[:, None] * (10000.0 ** (-2.0 * np.arange(head // 2) / head))[None, :]
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    got = R.run_op("gqa_rotary_embedding", [qkv, lens, cos, sin], qkv.shape, H,
                   {"num_heads": heads, "kv_num_heads": kvh, "interleaved": False})
    _eq(O.gqa_rotary_embedding(qkv, lens, cos, sin, heads, kvh, False), got)
