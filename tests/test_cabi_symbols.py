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
