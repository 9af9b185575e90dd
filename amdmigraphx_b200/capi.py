"""ctypes binding of lib/libmgx_cuda_kernels.so (the C ABI of include/mgx_cuda.h).

Used by the tests and the benchmark to drive the kernels with torch tensors as
device buffers; the MIGraphX plug-in (libmigraphx_cuda.so) calls the same entry
points from C++.  There is no fallback: if the library is missing, loading raises.
"""
import ctypes
import os
import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB_PATH = os.path.join(_PKG, "lib", "libmgx_cuda_kernels.so")

# mgx_dtype
F32, F16, I8, U8, I32, FP8_E4M3FN, I64 = 0, 1, 2, 3, 4, 5, 6
# mgx_scale_mode
SCALE_NONE, SCALE_PER_TENSOR, SCALE_PER_COL, SCALE_PER_ROW = 0, 1, 2, 3
# mgx_act
ACT_NONE, ACT_RELU, ACT_GELU_ERF, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3, 4
ACT_BY_NAME = {None: 0, "none": 0, "relu": 1, "gelu_erf": 2, "gelu_tanh": 3, "silu": 4}
# mgx_b_layout
B_KN, B_NK = 0, 1

E_INVALID_ARG, E_UNSUPPORTED, E_ALIGNMENT, E_WORKSPACE, E_TOO_LARGE = -1, -2, -3, -4, -5

EXPORTED_SYMBOLS = [
    "mgx_cuda_quantizelinear", "mgx_cuda_dequantizelinear", "mgx_cuda_unpack_int4",
    "mgx_cuda_pack_int4", "mgx_cuda_pointwise", "mgx_cuda_reduce", "mgx_cuda_softmax", "mgx_cuda_layernorm", "mgx_cuda_layernorm_ex", "mgx_cuda_layernorm_supported", "mgx_cuda_attention", "mgx_cuda_concat_past_present", "mgx_cuda_gqa_rotary_embedding", "mgx_cuda_rotary_embedding", "mgx_cuda_gqa_decode_attention", "mgx_cuda_gqa_decode_supported", "mgx_cuda_gather", "mgx_cuda_copy_rows", "mgx_cuda_qgemm_workspace", "mgx_cuda_qgemm", "mgx_cuda_qgemm_ex",
    "mgx_cuda_qgemm_static_scratch_limit", "mgx_cuda_qgemm_static_scratch",
    "mgx_cuda_transpose_8bit", "mgx_cuda_w4a16_workspace", "mgx_cuda_w4a16_gemv",
    "mgx_cuda_w4a16_gemm", "mgx_cuda_w4a16", "mgx_cuda_device_status",
    "mgx_cuda_status_string", "mgx_cuda_version", "mgx_cuda_selftest_bounded_wait",
    "mgx_cuda_comm_unique_id", "mgx_cuda_comm_create", "mgx_cuda_comm_destroy",
    "mgx_cuda_comm_set_default", "mgx_cuda_comm_default", "mgx_cuda_all_reduce",
]


class QgemmDesc(ctypes.Structure):
    _fields_ = [("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
                ("batch", ctypes.c_int64),
                ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldd", ctypes.c_int64),
                ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64),
                ("stride_d", ctypes.c_int64),
                ("ab_type", ctypes.c_int32), ("out_type", ctypes.c_int32),
                ("b_layout", ctypes.c_int32), ("scale_mode", ctypes.c_int32),
                ("act", ctypes.c_int32), ("flags", ctypes.c_int32)]


QGEMM_HALF_MATH = 1


class QgemmQout(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("ldq", ctypes.c_int64), ("stride_q", ctypes.c_int64),
                ("q_type", ctypes.c_int32), ("scale", ctypes.c_float),
                ("zero_point", ctypes.c_float), ("flags", ctypes.c_int32), ("lut", ctypes.c_void_p)]


QOUT_LUT = 1


class W4Desc(ctypes.Structure):
    _fields_ = [("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
                ("lda", ctypes.c_int64), ("ldd", ctypes.c_int64),
                ("group", ctypes.c_int32), ("zp_const", ctypes.c_int32),
                ("act", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class MgxError(RuntimeError):
    def __init__(self, code, what):
        super().__init__(f"{what}: status {code} ({status_string(code)})")
        self.code = code


_lib = None


def load():
    """Load the kernel library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(KERNEL_LIB_PATH):
        raise RuntimeError(
            f"{KERNEL_LIB_PATH} is missing: build it with `python -m amdmigraphx_b200.build` "
            "(there is no CPU fallback)")
    lib = ctypes.CDLL(KERNEL_LIB_PATH)
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    p64 = ctypes.POINTER(ctypes.c_int64)
    lib.mgx_cuda_quantizelinear.argtypes = [vp, i32, i64, vp, p64, vp, p64, vp, i32, i64, i64, i64, vp]
    lib.mgx_cuda_dequantizelinear.argtypes = [vp, i32, i64, vp, i32, p64, vp, p64, vp, i64, i64, i64, vp]
    lib.mgx_cuda_unpack_int4.argtypes = [vp, vp, i32, i64, i64, vp]
    lib.mgx_cuda_pack_int4.argtypes = [vp, vp, i32, i64, i64, vp]
    lib.mgx_cuda_qgemm_workspace.argtypes = [ctypes.POINTER(QgemmDesc)]
    lib.mgx_cuda_qgemm_workspace.restype = sz
    lib.mgx_cuda_qgemm.argtypes = [ctypes.POINTER(QgemmDesc), vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.mgx_cuda_qgemm_ex.argtypes = [ctypes.POINTER(QgemmDesc), vp, vp, vp, vp, vp, vp,
                                      ctypes.POINTER(QgemmQout), vp, sz, vp]
    lib.mgx_cuda_selftest_bounded_wait.argtypes = [ctypes.c_uint64, vp, vp]
    lib.mgx_cuda_qgemm_static_scratch_limit.restype = sz
    lib.mgx_cuda_qgemm_static_scratch.argtypes = [ctypes.POINTER(QgemmDesc), vp, vp, vp, vp, vp, vp, vp]
    lib.mgx_cuda_transpose_8bit.argtypes = [vp, vp, i64, i64, i64, vp]
    lib.mgx_cuda_w4a16_workspace.argtypes = [ctypes.POINTER(W4Desc)]
    lib.mgx_cuda_w4a16_workspace.restype = sz
    for name in ("mgx_cuda_w4a16_gemv", "mgx_cuda_w4a16_gemm", "mgx_cuda_w4a16"):
        getattr(lib, name).argtypes = [ctypes.POINTER(W4Desc), vp, vp, vp, vp, vp, vp, sz, vp]
    lib.mgx_cuda_comm_unique_id.argtypes = [vp]
    lib.mgx_cuda_comm_create.argtypes = [vp, i32, i32, ctypes.POINTER(vp)]
    lib.mgx_cuda_comm_destroy.argtypes = [vp]
    lib.mgx_cuda_comm_set_default.argtypes = [vp]
    lib.mgx_cuda_comm_set_default.restype = None
    lib.mgx_cuda_comm_default.restype = vp
    lib.mgx_cuda_all_reduce.argtypes = [vp, sz, i32, vp, vp]
    lib.mgx_cuda_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    lib.mgx_cuda_status_string.argtypes = [i32]
    lib.mgx_cuda_status_string.restype = ctypes.c_char_p
    lib.mgx_cuda_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def status_string(code):
    return load().mgx_cuda_status_string(int(code)).decode()


def check(code, what):
    if code != 0:
        raise MgxError(code, what)


def device_status():
    """Synchronise the device, return and clear the kernels' status word."""
    s = ctypes.c_int(0)
    check(load().mgx_cuda_device_status(ctypes.byref(s)), "mgx_cuda_device_status")
    return s.value


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype_code(t):
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.int8: I8, torch.uint8: U8,
            torch.int32: I32, torch.float8_e4m3fn: FP8_E4M3FN}[t.dtype]


def _strides2(view, rows, cols):
    """Strides (elements) of a tensor broadcastable to [rows, cols], as MIGraphX
    would pass it: 0 along broadcast dimensions."""
    if view.dim() == 0 or view.numel() == 1:
        return (ctypes.c_int64 * 2)(0, 0)
    if view.dim() == 1:
        if view.shape[0] == cols:
            return (ctypes.c_int64 * 2)(0, view.stride(0))
        raise ValueError("1-D scale must have `cols` elements")
    s0 = 0 if view.shape[0] == 1 else view.stride(0)
    s1 = 0 if view.shape[1] == 1 else view.stride(1)
    return (ctypes.c_int64 * 2)(s0, s1)


# ------------------------------------------------------------------ wrappers
def quantizelinear(x, scale, zp=None, out_dtype=None):
    """x [rows, cols] fp32/fp16 (row stride allowed); scale / zp broadcastable."""
    import torch
    lib = load()
    rows, cols = x.shape
    if out_dtype is None:
        out_dtype = zp.dtype if zp is not None else torch.uint8
    y = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
    code = lib.mgx_cuda_quantizelinear(
        _ptr(x), _dtype_code(x), x.stride(0) if rows > 1 else cols, _ptr(scale),
        _strides2(scale, rows, cols), _ptr(zp),
        _strides2(zp, rows, cols) if zp is not None else None, _ptr(y), _dtype_code(y), cols,
        rows, cols, _stream())
    check(code, "mgx_cuda_quantizelinear")
    return y


def dequantizelinear(x, scale, zp=None):
    import torch
    lib = load()
    rows, cols = x.shape
    y = torch.empty((rows, cols), dtype=scale.dtype, device=x.device)
    code = lib.mgx_cuda_dequantizelinear(
        _ptr(x), _dtype_code(x), x.stride(0) if rows > 1 else cols, _ptr(scale),
        _dtype_code(scale), _strides2(scale, rows, cols), _ptr(zp),
        _strides2(zp, rows, cols) if zp is not None else None, _ptr(y), cols, rows, cols,
        _stream())
    check(code, "mgx_cuda_dequantizelinear")
    return y


def unpack_int4(packed):
    import torch
    rows, pc = packed.shape
    out = torch.empty((rows, pc * 2), dtype=packed.dtype, device=packed.device)
    check(load().mgx_cuda_unpack_int4(_ptr(packed), _ptr(out), _dtype_code(packed), rows, pc,
                                      _stream()), "mgx_cuda_unpack_int4")
    return out


def pack_int4(x):
    import torch
    rows, c = x.shape
    out = torch.empty((rows, c // 2), dtype=x.dtype, device=x.device)
    check(load().mgx_cuda_pack_int4(_ptr(x), _ptr(out), _dtype_code(x), rows, c // 2, _stream()),
          "mgx_cuda_pack_int4")
    return out


def transpose_8bit(src):
    """[batch, rows, cols] or [rows, cols] bytes -> transposed, dense."""
    import torch
    s3 = src if src.dim() == 3 else src.unsqueeze(0)
    b, r, c = s3.shape
    dst = torch.empty((b, c, r), dtype=src.dtype, device=src.device)
    check(load().mgx_cuda_transpose_8bit(_ptr(s3), _ptr(dst), r, c, b, _stream()),
          "mgx_cuda_transpose_8bit")
    return dst if src.dim() == 3 else dst[0]


def qgemm(a, b, *, b_layout=B_KN, scale=None, scale_mode=None, bias=None, act=None,
          residual=None, out_dtype=None, out=None, workspace=None, q_out=None, q_scale=None,
          q_zero_point=0.0, write_d=True, half_math=False, lut=None):
    """quant_dot with the fused epilogue.  a: [M,K] or [B,M,K] int8 / float8_e4m3fn;
    b: [K,N] (B_KN) or [N,K] (B_NK), optionally batched.  q_out (int8 / float8 tensor of the
    output's shape) additionally receives quantizelinear(result, q_scale, q_zero_point);
    write_d=False skips the un-quantised result."""
    import torch
    lib = load()
    a3 = a if a.dim() == 3 else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    batch, M, K = a3.shape
    N = b3.shape[2] if b_layout == B_KN else b3.shape[1]
    is_int = a.dtype == torch.int8
    if out_dtype is None:
        out_dtype = torch.int32 if (is_int and scale is None and bias is None and act is None) \
            else torch.float32
    d = out if out is not None else torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
    d3 = d if d.dim() == 3 else d.unsqueeze(0)
    if scale_mode is None:
        if scale is None:
            scale_mode = SCALE_NONE
        elif scale.numel() == 1:
            scale_mode = SCALE_PER_TENSOR
        elif scale.numel() == N:
            scale_mode = SCALE_PER_COL
        else:
            scale_mode = SCALE_PER_ROW
    desc = QgemmDesc(M=M, N=N, K=K, batch=batch, lda=a3.stride(1), ldb=b3.stride(1),
                     ldd=d3.stride(1), stride_a=a3.stride(0), stride_b=b3.stride(0),
                     stride_d=d3.stride(0), ab_type=_dtype_code(a), out_type=_dtype_code(d),
                     b_layout=b_layout, scale_mode=scale_mode, act=ACT_BY_NAME[act],
                     flags=QGEMM_HALF_MATH if half_math else 0)
    need = lib.mgx_cuda_qgemm_workspace(ctypes.byref(desc))
    if need and workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    if q_out is None:
        code = lib.mgx_cuda_qgemm(ctypes.byref(desc), _ptr(a3), _ptr(b3), _ptr(d3), _ptr(scale),
                                  _ptr(bias), _ptr(residual), _ptr(workspace),
                                  0 if workspace is None else workspace.numel(), _stream())
    else:
        q3 = q_out if q_out.dim() == 3 else q_out.unsqueeze(0)
        qd = QgemmQout(q=q3.data_ptr(), ldq=q3.stride(1), stride_q=q3.stride(0),
                       q_type=_dtype_code(q3), scale=float(q_scale), zero_point=float(q_zero_point),
                       flags=QOUT_LUT if lut is not None else 0, lut=_ptr(lut))
        code = lib.mgx_cuda_qgemm_ex(ctypes.byref(desc), _ptr(a3), _ptr(b3),
                                     _ptr(d3) if write_d else None, _ptr(scale), _ptr(bias),
                                     _ptr(residual), ctypes.byref(qd), _ptr(workspace),
                                     0 if workspace is None else workspace.numel(), _stream())
    check(code, "mgx_cuda_qgemm")
    if out is not None:
        return out
    return d if a.dim() == 3 else d[0]


def w4a16(a, bp, scales, zp=None, *, zp_const=8, group=128, act=None, which="auto",
          workspace=None):
    """a [M,K] fp16, bp [N,K/2] uint8, scales [N,K/group] fp16 -> [M,N] fp16."""
    import torch
    lib = load()
    M, K = a.shape
    N = bp.shape[0]
    d = torch.empty((M, N), dtype=torch.float16, device=a.device)
    desc = W4Desc(M=M, N=N, K=K, lda=a.stride(0), ldd=N, group=group, zp_const=zp_const,
                  act=ACT_BY_NAME[act], reserved=0)
    need = lib.mgx_cuda_w4a16_workspace(ctypes.byref(desc))
    if need and workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    fn = {"auto": lib.mgx_cuda_w4a16, "gemv": lib.mgx_cuda_w4a16_gemv,
          "gemm": lib.mgx_cuda_w4a16_gemm}[which]
    code = fn(ctypes.byref(desc), _ptr(a), _ptr(bp), _ptr(scales), _ptr(zp), _ptr(d),
              _ptr(workspace), 0 if workspace is None else workspace.numel(), _stream())
    check(code, f"mgx_cuda_w4a16[{which}]")
    return d


# ------------------------------------------------------------------ element-wise
PW_MAXDIMS, PW_MAXIN, PW_MAXINSN = 5, 8, 32
PW_OPS = ["add", "sub", "mul", "div", "min", "max", "pow", "neg", "abs", "exp", "log", "sqrt", "rsqrt",
          "recip", "tanh", "sigmoid", "erf", "relu", "sin", "cos", "floor", "ceil", "round", "nearbyint",
          "convert", "where", "clip", "equal", "greater", "less", "leaky_relu", "const", "identity"]


class LayernormDesc(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("cols", ctypes.c_int64), ("ldx", ctypes.c_int64),
                ("ldy", ctypes.c_int64), ("ldq", ctypes.c_int64), ("type", ctypes.c_int32),
                ("eps", ctypes.c_float), ("q_type", ctypes.c_int32), ("q_scale", ctypes.c_float),
                ("q_zero_point", ctypes.c_float), ("flags", ctypes.c_int32)]


def layernorm(x, gamma=None, beta=None, eps=1e-5, q_scale=None, q_zero_point=0.0, write_y=True, dq_scale=None,
              rms=False):
    """LayerNorm over the last axis of a 2-D tensor; returns (y or None, q or None) where q is the
    int8 quantizelinear(y, q_scale, q_zero_point) written by the same launch; with dq_scale a third
    tensor, dequantizelinear(q, dq_scale, q_zero_point) in x's type, is returned too."""
    import torch
    lib = load()
    rows, cols = x.shape
    y = torch.empty_like(x) if write_y else None
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device) if q_scale is not None else None
    d = LayernormDesc(rows=rows, cols=cols, ldx=x.stride(0), ldy=cols, ldq=cols, type=_dtype_code(x), eps=eps,
                      q_type=I8, q_scale=float(q_scale or 1.0), q_zero_point=float(q_zero_point), flags=1 if rms else 0)
    if dq_scale is not None:
        dq = torch.empty_like(x)
        lib.mgx_cuda_layernorm_ex.argtypes = [ctypes.POINTER(LayernormDesc)] + [ctypes.c_void_p] * 6 + \
            [ctypes.c_int64, ctypes.c_float, ctypes.c_void_p]
        check(lib.mgx_cuda_layernorm_ex(ctypes.byref(d), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(q), _ptr(dq),
                                        cols, float(dq_scale), _stream()), "mgx_cuda_layernorm_ex")
        return y, q, dq
    lib.mgx_cuda_layernorm.argtypes = [ctypes.POINTER(LayernormDesc)] + [ctypes.c_void_p] * 6
    check(lib.mgx_cuda_layernorm(ctypes.byref(d), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(q), _stream()),
          "mgx_cuda_layernorm")
    return y, q


class GqaDecodeDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("batch", "heads", "kv_heads", "head", "cache_seq", "q_batch_stride",
                                              "q_head_stride")] + \
               [("scale", ctypes.c_float), ("seqlens_type", ctypes.c_int32)]


def concat_past_present(present, seqlens, past):
    """Appends present [batch, kv_heads, seq, head] (rows contiguous) to the cache past
    [batch, kv_heads, cache_seq, head] in place: at row seqlens[b] when seq == 1, at row 0 otherwise."""
    import torch
    lib = load()
    batch, kv_heads, seq, head = present.shape
    es = present.element_size()
    strides = (ctypes.c_int64 * 3)(present.stride(0) * es, present.stride(1) * es, present.stride(2) * es)
    lib.mgx_cuda_concat_past_present.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)] + \
        [ctypes.c_int64] * 4 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    check(lib.mgx_cuda_concat_past_present(_ptr(present), strides, batch, kv_heads, seq, head * es, _ptr(seqlens),
                                           I64 if seqlens.dtype == torch.int64 else I32, _ptr(past), past.shape[2],
                                           _stream()), "mgx_cuda_concat_past_present")
    return past


def gqa_rotary_embedding(qkv, seqlens, cos_cache, sin_cache, heads, kv_heads, interleaved=False):
    """Rotary embedding of the Q and K heads of packed [batch, heads + 2 kv_heads, seq, head]."""
    import torch
    lib = load()
    batch, _, seq, head = qkv.shape
    out = torch.empty_like(qkv)
    lib.mgx_cuda_gqa_rotary_embedding.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_int64] * 5 + \
        [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
         ctypes.c_void_p, ctypes.c_void_p]
    check(lib.mgx_cuda_gqa_rotary_embedding(_ptr(qkv), _dtype_code(qkv), batch, heads, kv_heads, seq, head,
                                            _ptr(cos_cache), _ptr(sin_cache), cos_cache.shape[0],
                                            cos_cache.shape[1] * 2, _ptr(seqlens),
                                            I64 if seqlens.dtype == torch.int64 else I32, 1 if interleaved else 0,
                                            _ptr(out), _stream()), "mgx_cuda_gqa_rotary_embedding")
    return out


def rotary_embedding(x, positions, cos_cache, sin_cache):
    """The rotary_embedding builder's rotation of x [batch, heads, seq, head] (rows contiguous, any other
    strides) at positions [batch, seq]; returns a packed tensor."""
    import torch
    lib = load()
    batch, heads, seq, head = x.shape
    out = torch.empty((batch, heads, seq, head), dtype=x.dtype, device=x.device)
    strides = (ctypes.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))
    lib.mgx_cuda_rotary_embedding.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int64)] + \
        [ctypes.c_int64] * 4 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                ctypes.c_void_p, ctypes.c_void_p]
    check(lib.mgx_cuda_rotary_embedding(_ptr(x), _dtype_code(x), strides, batch, heads, seq, head, _ptr(positions),
                                        I64 if positions.dtype == torch.int64 else I32, _ptr(cos_cache),
                                        _ptr(sin_cache), cos_cache.shape[0], _ptr(out), _stream()),
          "mgx_cuda_rotary_embedding")
    return out


def gqa_decode_supported(batch, heads, kv_heads, head, cache_seq):
    lib = load()
    lib.mgx_cuda_gqa_decode_supported.argtypes = [ctypes.c_int64] * 5
    return bool(lib.mgx_cuda_gqa_decode_supported(batch, heads, kv_heads, head, cache_seq))


def gqa_decode_attention(q, k_cache, v_cache, seqlens, scale):
    """softmax(scale * q K^T) V over cache positions 0 .. seqlens[b] for q [batch, heads, head] (rows
    contiguous) against caches [batch, kv_heads, cache_seq, head]; returns [batch, heads * head]."""
    import torch
    lib = load()
    batch, heads, head = q.shape
    out = torch.empty((batch, heads * head), dtype=torch.float16, device=q.device)
    d = GqaDecodeDesc(batch=batch, heads=heads, kv_heads=k_cache.shape[1], head=head, cache_seq=k_cache.shape[2],
                      q_batch_stride=q.stride(0), q_head_stride=q.stride(1), scale=float(scale),
                      seqlens_type=I64 if seqlens.dtype == torch.int64 else I32)
    lib.mgx_cuda_gqa_decode_attention.argtypes = [ctypes.POINTER(GqaDecodeDesc)] + [ctypes.c_void_p] * 6
    check(lib.mgx_cuda_gqa_decode_attention(ctypes.byref(d), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seqlens),
                                            _ptr(out), _stream()), "mgx_cuda_gqa_decode_attention")
    return out


class AttentionDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("batch", "seq", "heads", "head_dim", "ldq", "ldk", "ldv", "ldo", "ldoq")] + \
               [("scale", ctypes.c_float), ("q_scale", ctypes.c_float), ("q_zero_point", ctypes.c_float),
                ("flags", ctypes.c_int32)]


def attention(q, k, v, batch, seq, heads, scale, q_scale=None, q_zero_point=0.0, write_o=True, fp32_softmax=False,
              three_pass=False):
    """softmax(scale * Q K^T) V per batch entry and head on [batch*seq, heads*64] fp16 matrices (row
    strided views allowed); returns (o or None, oq or None)."""
    import torch
    lib = load()
    width = heads * 64
    o = torch.empty((batch * seq, width), dtype=torch.float16, device=q.device) if write_o else None
    oq = torch.empty((batch * seq, width), dtype=torch.int8, device=q.device) if q_scale is not None else None
    d = AttentionDesc(batch=batch, seq=seq, heads=heads, head_dim=64, ldq=q.stride(0), ldk=k.stride(0),
                      ldv=v.stride(0), ldo=width, ldoq=width, scale=float(scale), q_scale=float(q_scale or 1.0),
                      q_zero_point=float(q_zero_point), flags=(1 if fp32_softmax else 0) | (2 if three_pass else 0))
    lib.mgx_cuda_attention.argtypes = [ctypes.POINTER(AttentionDesc)] + [ctypes.c_void_p] * 6
    check(lib.mgx_cuda_attention(ctypes.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(oq), _stream()),
          "mgx_cuda_attention")
    return o, oq


class PwInsn(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("type", ctypes.c_int32), ("src", ctypes.c_int32 * 3),
                ("imm", ctypes.c_float)]


class PwDesc(ctypes.Structure):
    _fields_ = [("ndim", ctypes.c_int32), ("ninputs", ctypes.c_int32), ("ninsns", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("lens", ctypes.c_int64 * PW_MAXDIMS),
                ("in_type", ctypes.c_int32 * PW_MAXIN),
                ("in_strides", (ctypes.c_int64 * PW_MAXDIMS) * PW_MAXIN),
                ("insn", PwInsn * PW_MAXINSN)]


def pointwise(inputs, program, lens):
    """inputs: tensors viewed (expanded) to `lens`; program: list of (op name, result dtype code,
    (src0, src1, src2), imm).  Returns the packed result of the last instruction."""
    import torch
    lib = load()
    d = PwDesc()
    d.ndim, d.ninputs, d.ninsns = len(lens), len(inputs), len(program)
    for k, n in enumerate(lens):
        d.lens[k] = n
    for i, t in enumerate(inputs):
        assert tuple(t.shape) == tuple(lens)
        d.in_type[i] = _dtype_code(t)
        for k in range(len(lens)):
            d.in_strides[i][k] = t.stride(k)
    for n, (op, ty, src, imm) in enumerate(program):
        d.insn[n].op, d.insn[n].type, d.insn[n].imm = PW_OPS.index(op), ty, imm
        for j in range(3):
            d.insn[n].src[j] = src[j] if j < len(src) else 0
    tdt = {F32: torch.float32, F16: torch.float16, I8: torch.int8, U8: torch.uint8, I32: torch.int32}
    out = torch.empty(tuple(lens), dtype=tdt[program[-1][1]], device=inputs[0].device)
    ptrs = (ctypes.c_void_p * max(1, len(inputs)))(*[t.data_ptr() for t in inputs])
    lib.mgx_cuda_pointwise.restype = ctypes.c_int
    check(lib.mgx_cuda_pointwise(ctypes.byref(d), ptrs, ctypes.c_void_p(out.data_ptr()), _stream()),
          "mgx_cuda_pointwise")
    return out


REDUCE_OPS = ["sum", "mean", "max", "min"]


def reduce_rows(x, op):
    """reduce_sum / reduce_mean / reduce_max / reduce_min over the last axis of a 2-D tensor
    (rows may be strided); returns [rows, 1] of x's type."""
    import torch
    lib = load()
    assert x.dim() == 2 and x.stride(1) == 1
    out = torch.empty((x.shape[0], 1), dtype=x.dtype, device=x.device)
    lib.mgx_cuda_reduce.restype = ctypes.c_int
    check(lib.mgx_cuda_reduce(ctypes.c_void_p(x.data_ptr()), _dtype_code(x), ctypes.c_int64(x.stride(0)),
                              ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]),
                              REDUCE_OPS.index(op), ctypes.c_void_p(out.data_ptr()), _stream()),
          "mgx_cuda_reduce")
    return out


def softmax(x):
    """softmax over the last axis of a 2-D tensor (rows may be strided)."""
    import torch
    lib = load()
    assert x.dim() == 2 and x.stride(1) == 1
    out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    lib.mgx_cuda_softmax.restype = ctypes.c_int
    check(lib.mgx_cuda_softmax(ctypes.c_void_p(x.data_ptr()), _dtype_code(x), ctypes.c_int64(x.stride(0)),
                               ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(out.stride(0)),
                               ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]), _stream()),
          "mgx_cuda_softmax")
    return out


def gather(data, indices, axis):
    """op::gather on a packed tensor; indices int32 / int64 of any shape."""
    import torch
    lib = load()
    assert data.is_contiguous() and indices.is_contiguous()
    axis = axis % data.dim()
    outer = int(np.prod(data.shape[:axis], dtype=np.int64))
    inner = int(np.prod(data.shape[axis + 1:], dtype=np.int64)) * data.element_size()
    out = torch.empty(tuple(data.shape[:axis]) + tuple(indices.shape) + tuple(data.shape[axis + 1:]),
                      dtype=data.dtype, device=data.device)
    code = {torch.int32: I32, torch.int64: 6}[indices.dtype]
    lib.mgx_cuda_gather.restype = ctypes.c_int
    check(lib.mgx_cuda_gather(ctypes.c_void_p(data.data_ptr()), ctypes.c_int64(outer),
                              ctypes.c_int64(data.shape[axis]), ctypes.c_int64(inner),
                              ctypes.c_void_p(indices.data_ptr()), code, ctypes.c_int64(indices.numel()),
                              ctypes.c_void_p(out.data_ptr()), _stream()), "mgx_cuda_gather")
    return out


def concat(tensors, axis):
    """op::concat of packed tensors along `axis`: one row copy per input."""
    import torch
    lib = load()
    axis = axis % tensors[0].dim()
    lens = list(tensors[0].shape)
    lens[axis] = sum(t.shape[axis] for t in tensors)
    out = torch.empty(tuple(lens), dtype=tensors[0].dtype, device=tensors[0].device)
    es = out.element_size()
    outer = int(np.prod(lens[:axis], dtype=np.int64))
    inner = int(np.prod(lens[axis + 1:], dtype=np.int64)) * es
    lib.mgx_cuda_copy_rows.restype = ctypes.c_int
    off = 0
    for t in tensors:
        assert t.is_contiguous()
        rb = t.shape[axis] * inner
        check(lib.mgx_cuda_copy_rows(ctypes.c_void_p(t.data_ptr()), ctypes.c_int64(rb),
                                     ctypes.c_void_p(out.data_ptr() + off), ctypes.c_int64(lens[axis] * inner),
                                     ctypes.c_int64(outer), ctypes.c_int64(rb), _stream()), "mgx_cuda_copy_rows")
        off += rb
    return out


# ------------------------------------------------------------------ tensor parallel
class Communicator(object):
    """One NCCL communicator per process, created from a 128-byte id that rank 0 makes and the
    caller distributes (here: through torch.distributed's store / broadcast)."""

    def __init__(self, unique_id_bytes, nranks, rank):
        lib = load()
        self.handle = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(bytes(unique_id_bytes), 128)
        check(lib.mgx_cuda_comm_create(buf, nranks, rank, ctypes.byref(self.handle)),
              "mgx_cuda_comm_create")
        self.nranks, self.rank = nranks, rank

    @staticmethod
    def make_unique_id():
        buf = ctypes.create_string_buffer(128)
        check(load().mgx_cuda_comm_unique_id(buf), "mgx_cuda_comm_unique_id")
        return buf.raw

    def all_reduce_(self, t):
        check(load().mgx_cuda_all_reduce(_ptr(t), t.numel(), _dtype_code(t), self.handle, _stream()),
              "mgx_cuda_all_reduce")
        return t

    def destroy(self):
        if self.handle:
            load().mgx_cuda_comm_destroy(self.handle)
            self.handle = ctypes.c_void_p()
