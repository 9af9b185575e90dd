"""CPU test: the kernel library loads without a GPU and exports every entry point that
include/mgx_cuda.h declares (no compute calls are made here)."""
import ctypes
import os
import re

from amdmigraphx_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "mgx_cuda.h")).read()
    return sorted(set(re.findall(r"MGX_API\s+[\w\s\*]+?\b(mgx_cuda_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared() == sorted(capi.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(capi.KERNEL_LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), name


def test_status_strings_and_argument_checks_without_gpu():
    lib = capi.load()
    assert lib.mgx_cuda_version().decode().startswith("mgx_cuda sm_100a")
    assert capi.status_string(0) == "ok"
    assert "workspace" in capi.status_string(capi.E_WORKSPACE)
    # host-side validation happens before any CUDA call
    d = capi.QgemmDesc(M=0, N=8, K=16, batch=1)
    one = ctypes.c_void_p(16)
    assert lib.mgx_cuda_qgemm(ctypes.byref(d), one, one, one, None, None, None, None, 0, None) == capi.E_INVALID_ARG
    assert lib.mgx_cuda_qgemm(None, one, one, one, None, None, None, None, 0, None) == capi.E_INVALID_ARG
    w = capi.W4Desc(M=1, N=8, K=48, lda=48, ldd=8, group=48, zp_const=8)
    assert lib.mgx_cuda_w4a16(ctypes.byref(w), one, one, one, None, one, None, 0, None) == capi.E_UNSUPPORTED
    assert lib.mgx_cuda_qgemm_workspace(None) == 0


def test_decode_attention_host_answers_without_gpu():
    """mgx_cuda_gqa_decode_supported is host arithmetic (heads per KV head, head size, the share of the
    cache a CTA keeps in shared memory), and mgx_cuda_gqa_decode_attention validates its descriptor
    before any CUDA call."""
    assert capi.gqa_decode_supported(1, 32, 32, 128, 2048)      # Llama-2-7B decode
    assert capi.gqa_decode_supported(16, 8, 1, 128, 4096)       # one of eight shards of Llama-2-70B
    assert capi.gqa_decode_supported(16, 32, 8, 64, 2048)
    assert capi.gqa_decode_supported(300, 2, 1, 64, 130)
    assert not capi.gqa_decode_supported(1, 32, 32, 96, 2048)   # head size
    assert not capi.gqa_decode_supported(1, 12, 4, 128, 2048)   # three query heads per KV head
    assert not capi.gqa_decode_supported(1, 32, 5, 128, 2048)   # heads not a multiple of KV heads
    assert not capi.gqa_decode_supported(0, 32, 32, 128, 2048)
    assert not capi.gqa_decode_supported(1, 8, 1, 128, 1 << 20)  # an eighth of the scores: 2 MB of shared memory
    assert capi.gqa_decode_supported(1, 8, 1, 128, 65536)        # 8 heads x 8192 halves = 128 KB + partials

    lib = capi.load()
    lib.mgx_cuda_gqa_decode_attention.argtypes = [ctypes.POINTER(capi.GqaDecodeDesc)] + [ctypes.c_void_p] * 6
    lib.mgx_cuda_gqa_decode_attention.restype = ctypes.c_int
    one, odd = ctypes.c_void_p(4096), ctypes.c_void_p(4104)

    def call(d, q=one, k=one, v=one, s=one, o=one):
        return lib.mgx_cuda_gqa_decode_attention(ctypes.byref(d), q, k, v, s, o, None)

    def desc(**kw):
        base = dict(batch=1, heads=8, kv_heads=2, head=128, cache_seq=256, q_batch_stride=1024, q_head_stride=128,
                    scale=0.088, seqlens_type=capi.I32)
        base.update(kw)
        return capi.GqaDecodeDesc(**base)

    assert call(desc(), q=None) == capi.E_INVALID_ARG
    assert call(desc(heads=7)) == capi.E_INVALID_ARG
    assert call(desc(batch=0)) == capi.E_INVALID_ARG
    assert call(desc(seqlens_type=capi.F16)) == capi.E_UNSUPPORTED
    assert call(desc(head=96)) == capi.E_UNSUPPORTED
    assert call(desc(heads=6)) == capi.E_UNSUPPORTED
    assert call(desc(batch=70000)) == capi.E_TOO_LARGE
    assert call(desc(), k=odd) == capi.E_ALIGNMENT


def test_decoder_byte_movers_and_pointwise_validate_before_any_cuda_call():
    lib = capi.load()
    one = ctypes.c_void_p(4096)
    i64 = ctypes.c_int64
    st3 = (i64 * 3)(1024, 128, 128)

    rot = lib.mgx_cuda_rotary_embedding
    rot.restype = ctypes.c_int
    rot.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(i64), i64, i64, i64, i64, ctypes.c_void_p,
                    ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, i64, ctypes.c_void_p, ctypes.c_void_p]
    assert rot(None, capi.F16, st3, 1, 8, 1, 128, one, capi.I64, one, one, 2048, one, None) == capi.E_INVALID_ARG
    assert rot(one, capi.F16, st3, 1, 8, 1, 127, one, capi.I64, one, one, 2048, one, None) == capi.E_INVALID_ARG
    assert rot(one, capi.I8, st3, 1, 8, 1, 128, one, capi.I64, one, one, 2048, one, None) == capi.E_UNSUPPORTED
    assert rot(one, capi.F16, st3, 1, 8, 1, 128, one, capi.F32, one, one, 2048, one, None) == capi.E_UNSUPPORTED

    cpp = lib.mgx_cuda_concat_past_present
    cpp.restype = ctypes.c_int
    cpp.argtypes = [ctypes.c_void_p, ctypes.POINTER(i64), i64, i64, i64, i64, ctypes.c_void_p, ctypes.c_int,
                    ctypes.c_void_p, i64, ctypes.c_void_p]
    assert cpp(one, st3, 1, 8, 1, 256, None, capi.I32, one, 2048, None) == capi.E_INVALID_ARG  # a decode step needs seqlens
    assert cpp(one, st3, 1, 8, 1, 256, one, capi.F32, one, 2048, None) == capi.E_UNSUPPORTED
    assert cpp(one, st3, 1, 8, 0, 256, one, capi.I32, one, 2048, None) == capi.E_INVALID_ARG
    assert cpp(one, st3, 4096, 32, 1, 256, one, capi.I32, one, 2048, None) == capi.E_TOO_LARGE

    pw = lib.mgx_cuda_pointwise
    pw.restype = ctypes.c_int
    pw.argtypes = [ctypes.POINTER(capi.PwDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    ptrs = (ctypes.c_void_p * 2)(4096, 8192)

    def prog(ndim=1, ninputs=2, lens=(64,), insns=((capi.PW_OPS.index("add"), capi.F16, (0, 1, 0)),)):
        d = capi.PwDesc()
        d.ndim, d.ninputs, d.ninsns = ndim, ninputs, len(insns)
        for k, n in enumerate(lens):
            d.lens[k] = n
        for i in range(ninputs):
            d.in_type[i] = capi.F16
            d.in_strides[i][ndim - 1 if ndim > 0 else 0] = 1
        for n, (op, ty, src) in enumerate(insns):
            d.insn[n].op, d.insn[n].type = op, ty
            for j in range(3):
                d.insn[n].src[j] = src[j]
        return d

    assert pw(None, ptrs, one, None) == capi.E_INVALID_ARG
    assert pw(ctypes.byref(prog(ndim=0)), ptrs, one, None) == capi.E_UNSUPPORTED
    assert pw(ctypes.byref(prog(insns=())), ptrs, one, None) == capi.E_UNSUPPORTED
    assert pw(ctypes.byref(prog(insns=((999, capi.F16, (0, 1, 0)),))), ptrs, one, None) == capi.E_UNSUPPORTED
    # an instruction may only read the inputs and earlier results
    assert pw(ctypes.byref(prog(insns=((0, capi.F16, (0, 2, 0)),))), ptrs, one, None) == capi.E_INVALID_ARG
    assert pw(ctypes.byref(prog(lens=(-1,))), ptrs, one, None) == capi.E_INVALID_ARG
    # nothing to do: no launch, no error
    assert pw(ctypes.byref(prog(lens=(0,))), ptrs, one, None) == 0
