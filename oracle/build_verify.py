#!/usr/bin/env python3
"""Build oracle/_ref/bin/test_verify_cuda: the reference's own cross-target verify harness
(test/verify/run_verify.cpp, verify_program.cpp, auto_print.cpp) and its verify programs for the
quantized path (test/verify/test_quant_dot_3args_*.cpp, test_batch_quant_dot_*.cpp,
test_unpack_int4.cpp, test_quantizelinear*.cpp, test_dequantizelinear.cpp, test_gemm_pointwise.cpp,
test_add_gelu*.cpp, ...), compiled where they lie and linked with the `cuda` plug-in, MIGraphX's
ref target and oracle/verify_cuda_main.cpp.  Nothing is copied.

Usage: python oracle/build_verify.py [--ref <MIGraphX source tree>]
"""
import argparse
import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import build_ref  # noqa: E402

# verify programs of the path this repository covers (globs under test/verify)
PROGRAMS = ["test_quant_dot_3args_*.cpp", "test_batch_quant_dot_*.cpp", "test_unpack_int4.cpp",
            "test_quantizelinear.cpp", "test_quantizelinear_int32.cpp", "test_dequantizelinear.cpp",
            "test_gemm_pointwise.cpp", "test_add_gelu.cpp", "test_add_gelu_half.cpp",
            "test_gemm_half.cpp", "test_softmax*.cpp", "test_layernorm.cpp", "test_gather.cpp",
            "test_concat_axis_0.cpp", "test_concat_axis_1.cpp", "test_reduce_op_large.cpp",
            "test_gemm_softmax_gemm_relu.cpp"]
HARNESS = ["run_verify.cpp", "verify_program.cpp", "auto_print.cpp"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=build_ref.reference_dir())
    a = ap.parse_args()
    vdir = os.path.join(a.ref, "test", "verify")
    if not os.path.isdir(vdir):
        print(f"[build_verify] {vdir} not found; keeping prebuilt files")
        return 0
    root = build_ref.ROOT
    obj = os.path.join(HERE, "_ref", "obj")
    bindir = os.path.join(HERE, "_ref", "bin")
    os.makedirs(obj, exist_ok=True)
    os.makedirs(bindir, exist_ok=True)
    gen = os.path.join(build_ref.HOST, "gen", "include")
    hostlib = os.path.join(build_ref.HOST, "lib")
    reflib = os.path.join(HERE, "_ref", "lib")
    pluglib = os.path.join(root, "amdmigraphx_b200", "lib")
    flags = ["-std=c++17", "-O1", "-w", "-pthread", "-DMIGRAPHX_USE_EIGEN=0", f"-I{gen}",
             f"-I{a.ref}/src/include", f"-I{a.ref}/test/include", f"-I{vdir}"]
    sources = [os.path.join(vdir, f) for f in HARNESS]
    for pat in PROGRAMS:
        sources += sorted(glob.glob(os.path.join(vdir, pat)))
    sources.append(os.path.join(HERE, "verify_cuda_main.cpp"))

    def cc(src):
        o = os.path.join(obj, "verify_" + os.path.basename(src)[:-4] + ".o")
        if not os.path.exists(o) or os.path.getmtime(o) < os.path.getmtime(src):
            r = subprocess.run(["g++", "-c", src, "-o", o] + flags, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed for {src}:\n{r.stderr[-4000:]}")
        return o

    with cf.ThreadPoolExecutor(max(1, min(8, os.cpu_count() or 1))) as ex:
        objs = list(ex.map(cc, sources))
    exe = os.path.join(bindir, "test_verify_cuda")
    cuda_lib = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/lib64"
    subprocess.check_call(["g++", "-o", exe] + objs + [
        f"-L{pluglib}", f"-L{reflib}", f"-L{hostlib}", "-Wl,--no-as-needed", "-lmigraphx_cuda", "-lmigraphx_ref",
        "-lmigraphx", "-lmgx_cuda_kernels", f"-L{cuda_lib}", "-lcudart", "-lpthread",
        "-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath,$ORIGIN/../../../baseline/_ref/lib",
        "-Wl,-rpath,$ORIGIN/../../../amdmigraphx_b200/lib", f"-Wl,-rpath,{cuda_lib}"])
    print(f"[build_verify] {len(sources)} translation units -> {exe}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
