"""In-tree build of the native libraries.

  lib/libmgx_cuda_kernels.so  - sm_100a kernels behind the C ABI of include/mgx_cuda.h
                                (nvcc, cross-compiles without a GPU)
  lib/libmigraphx_cuda.so     - the MIGraphX `cuda` target plug-in (C++17 host code
                                compiled against the MIGraphX headers and linked to
                                libmigraphx.so); built only when those are available.

Run:  python -m amdmigraphx_b200.build [--verbose] [--force]
"""
import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
OBJ = os.path.join(PKG, "build")

KERNEL_SOURCES = ["runtime.cu", "quantize.cu", "qgemm.cu", "qgemv.cu", "pointwise.cu", "reduce.cu", "layernorm.cu", "attention.cu", "kvcache.cu", "gqa_decode.cu", "gather.cu", "w4a16.cu", "w4a16_tc.cu", "w4a16_prefill.cu", "comm.cu"]
KERNEL_LIB = os.path.join(LIB, "libmgx_cuda_kernels.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def nvcc_path():
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return p


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    hs.append(os.path.join(ROOT, "include", "mgx_cuda.h"))
    return hs


def _compile(args):
    src, obj, verbose, force = args
    if not force and not _newer(obj, [src] + _headers()):
        return src, 0, ""
    cmd = [nvcc_path(), "-c", src, "-o", obj] + NVCC_FLAGS
    if verbose:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, (r.stdout + r.stderr)


def build_kernels(verbose=False, force=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    jobs = [(os.path.join(CSRC, s), os.path.join(OBJ, s[:-3] + ".o"), verbose, force)
            for s in KERNEL_SOURCES]
    with cf.ThreadPoolExecutor(len(jobs)) as ex:
        for src, rc, out in ex.map(_compile, jobs):
            if verbose and out:
                print(out)
            if rc != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{out}")
    objs = [j[1] for j in jobs]
    if force or _newer(KERNEL_LIB, objs):
        cmd = [nvcc_path(), "-shared", "-o", KERNEL_LIB] + objs + [
            "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return KERNEL_LIB


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_kernels(a.verbose, a.force))
    try:
        from . import build_target
    except ImportError:
        build_target = None
    if build_target is not None:
        print(build_target.build_target(verbose=a.verbose, force=a.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
