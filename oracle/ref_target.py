"""ctypes binding of oracle/_ref/lib/libmgx_ref_oracle.so: single MIGraphX operators run on
the unmodified `ref` target built from the reference sources (oracle/build_ref.py).

TEST INFRASTRUCTURE ONLY (tests/, bench.py's CPU-baseline legs, fixture generation).
"""
import ctypes
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "lib", "libmgx_ref_oracle.so")

_TYPE_NAMES = {
    np.dtype(np.float32): "float_type", np.dtype(np.float16): "half_type",
    np.dtype(np.float64): "double_type", np.dtype(np.int8): "int8_type",
    np.dtype(np.uint8): "uint8_type", np.dtype(np.int32): "int32_type",
    np.dtype(np.int64): "int64_type", np.dtype(np.bool_): "bool_type",
}
_NP_OF = {v: k for k, v in _TYPE_NAMES.items()}
_NP_OF["fp8e4m3fn_type"] = np.dtype(np.uint8)  # carried as bit patterns


class _Tensor(ctypes.Structure):
    _fields_ = [("type", ctypes.c_char_p), ("ndim", ctypes.c_int),
                ("lens", ctypes.POINTER(ctypes.c_int64)),
                ("strides", ctypes.POINTER(ctypes.c_int64)), ("data", ctypes.c_void_p)]


_lib = None


def available():
    return os.path.exists(LIB_PATH)


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(LIB_PATH)
        lib.ref_last_error.restype = ctypes.c_char_p
        lib.ref_run_op.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int,
                                   ctypes.POINTER(_Tensor), ctypes.POINTER(_Tensor),
                                   ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
        lib.ref_time_bert.argtypes = [ctypes.c_int64] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double),
                                                            ctypes.POINTER(ctypes.c_double)]
        _lib = lib
    return _lib


def time_bert_encoder(batch, seq, layers, hidden=768, heads=12, ffn=3072, vocab=30522, warmup=0, repeat=1):
    """Total seconds of `repeat` eval() calls (after `warmup` untimed ones) of the benchmark's
    BERT-shaped int8 encoder program on the ref target (all host threads MIGraphX's par_for uses)
    and the 2*M*N*K of its QDQ linears per eval()."""
    secs, ops = ctypes.c_double(0), ctypes.c_double(0)
    rc = load().ref_time_bert(batch, seq, layers, hidden, heads, ffn, vocab, warmup, repeat,
                              ctypes.byref(secs), ctypes.byref(ops))
    if rc != 0:
        raise RuntimeError("ref_time_bert: " + load().ref_last_error().decode())
    return secs.value, ops.value


def hardware_threads():
    return load().ref_hardware_threads()


class Fp8(object):
    """Marks a uint8 array as fp8e4m3fn bit patterns."""

    def __init__(self, codes):
        self.codes = np.ascontiguousarray(codes, dtype=np.uint8)


def _mk(arr, keep):
    if isinstance(arr, Fp8):
        a, tname = arr.codes, "fp8e4m3fn_type"
    else:
        a = np.ascontiguousarray(arr)
        tname = _TYPE_NAMES[a.dtype]
    lens = (ctypes.c_int64 * a.ndim)(*a.shape)
    keep.extend([a, lens])
    return _Tensor(tname.encode(), a.ndim, lens, None, a.ctypes.data_as(ctypes.c_void_p))


def run_op(name, inputs, out_shape, out_type, attrs=None, repeat=1, want_seconds=False):
    """Evaluate one MIGraphX operator on the ref target.
    inputs: numpy arrays (or Fp8); out_type: MIGraphX type name, e.g. 'int32_type'."""
    lib = load()
    keep = []
    ins = (_Tensor * len(inputs))(*[_mk(x, keep) for x in inputs])
    out = np.empty(out_shape, dtype=_NP_OF[out_type])
    olens = (ctypes.c_int64 * out.ndim)(*out.shape)
    ot = _Tensor(out_type.encode(), out.ndim, olens, None, out.ctypes.data_as(ctypes.c_void_p))
    secs = ctypes.c_double(0)
    rc = lib.ref_run_op(name.encode(), json.dumps(attrs or {}).encode(), len(inputs), ins,
                        ctypes.byref(ot), repeat, ctypes.byref(secs))
    if rc != 0:
        raise RuntimeError(f"ref {name}: {lib.ref_last_error().decode()}")
    return (out, secs.value) if want_seconds else out


# ---- the operators of the quantized path, with MIGraphX's calling conventions ----------
def _full(v, shape, dtype=None):
    a = np.broadcast_to(np.asarray(v, dtype=dtype), shape)
    return np.ascontiguousarray(a)


def quantizelinear(x, scale, zp=None, out_type="int8"):
    x = np.asarray(x)
    s = _full(scale, x.shape, x.dtype)
    tname = {"int8": "int8_type", "uint8": "uint8_type", "fp8e4m3fn": "fp8e4m3fn_type"}[out_type]
    if zp is None and out_type == "uint8":
        return run_op("quantizelinear", [x, s], x.shape, tname)
    if zp is None:
        z = np.zeros(x.shape, dtype=np.int8 if out_type == "int8" else np.uint8)
    else:
        z = _full(zp, x.shape)
    zin = Fp8(z) if out_type == "fp8e4m3fn" else z
    return run_op("quantizelinear", [x, s, zin], x.shape, tname)


def dequantizelinear(x, scale, zp=None, x_is_fp8=False):
    x = np.asarray(x)
    scale = np.asarray(scale)
    s = _full(scale, x.shape)
    ins = [Fp8(x) if x_is_fp8 else x, s]
    if zp is not None:
        z = _full(zp, x.shape, x.dtype)
        ins.append(Fp8(z) if x_is_fp8 else z)
    return run_op("dequantizelinear", ins, x.shape, _TYPE_NAMES[scale.dtype])


def quant_dot(a, b, fp8=False, repeat=1, want_seconds=False):
    a = np.asarray(a)
    b = np.asarray(b)
    shape = a.shape[:-1] + (b.shape[-1],)
    ins = [Fp8(a), Fp8(b)] if fp8 else [a, b]
    return run_op("quant_dot", ins, shape, "float_type" if fp8 else "int32_type",
                  repeat=repeat, want_seconds=want_seconds)


def dot(a, b):
    a = np.asarray(a)
    b = np.asarray(b)
    return run_op("dot", [a, b], a.shape[:-1] + (b.shape[-1],), _TYPE_NAMES[a.dtype])


def unpack_int4(x):
    x = np.asarray(x)
    return run_op("unpack_int4", [x], x.shape[:-1] + (x.shape[-1] * 2,), _TYPE_NAMES[x.dtype])


def pack_int4(x):
    x = np.asarray(x)
    return run_op("pack_int4", [x], x.shape[:-1] + (x.shape[-1] // 2,), _TYPE_NAMES[x.dtype])


def binary(name, a, b):
    a = np.asarray(a)
    return run_op(name, [a, _full(b, a.shape, a.dtype)], a.shape, _TYPE_NAMES[a.dtype])


def unary(name, a):
    a = np.asarray(a)
    return run_op(name, [a], a.shape, _TYPE_NAMES[a.dtype])


def gelu_erf(x):
    """The instruction sequence of src/op/builder/gelu.cpp:58-74 on ref."""
    x = np.asarray(x)
    t = x.dtype.type
    mul_half = binary("mul", x, t(0.5))
    div = binary("div", x, t(np.float32(np.sqrt(2.0))))
    erf = unary("erf", div)
    add_one = binary("add", erf, t(1.0))
    return binary("mul", mul_half, add_one)


def qlinear_epilogue(acc, scale, bias=None, act=None, residual=None):
    v = dequantizelinear(acc, np.asarray(scale, dtype=np.float32))
    if bias is not None:
        v = binary("add", v, np.asarray(bias, dtype=np.float32))
    if act == "relu":
        v = unary("relu", v)
    elif act == "gelu_erf":
        v = gelu_erf(v)
    elif act not in (None, "none"):
        raise ValueError(act)
    if residual is not None:
        v = binary("add", v, np.asarray(residual, dtype=np.float32))
    return v


def w4a16_linear(a, bp, scales, zp=None, zp_const=8, group=128):
    """unpack_int4 -> dequantizelinear (fp16) -> transpose -> dot, the IR of
    src/onnx/parse_matmulnbits.cpp:85-158."""
    q = unpack_int4(np.asarray(bp, dtype=np.uint8))
    n, k = q.shape
    s = np.repeat(np.asarray(scales, dtype=np.float16).reshape(n, k // group), group, axis=1)
    if zp is None:
        z = np.full(q.shape, zp_const, dtype=np.uint8)
    else:
        z = np.repeat(np.asarray(zp, dtype=np.uint8).reshape(n, k // group), group, axis=1)
    w = dequantizelinear(q, s, z)
    return dot(np.asarray(a, dtype=np.float16), np.ascontiguousarray(w.T))
