"""Build lib/libmigraphx_cuda.so, the MIGraphX `cuda` target plug-in, and the C++ parity
driver bin/cuda_target_check.

The plug-in is host C++17 compiled against MIGraphX's headers and linked to libmigraphx.so
and to the kernel library.  MIGraphX itself is not part of this repository: the headers
are taken from a MIGraphX source tree (MIGRAPHX_SOURCE_DIR, default: a directory named
`reference` next to this repository) and the library from MIGRAPHX_LIB_DIR (default
baseline/_ref/lib, where oracle/build_ref.py puts its build of the unmodified sources; the
parity driver also links MIGraphX's CPU `ref` target from oracle/_ref/lib).  When the headers are absent (for example on a GPU
box that only received the prebuilt files) the existing binaries are kept.
"""
import concurrent.futures as cf
import os
import subprocess
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
SRC = os.path.join(PKG, "csrc", "target")
LIB = os.path.join(PKG, "lib")
BIN = os.path.join(PKG, "bin")
OBJ = os.path.join(PKG, "build")
TARGET_LIB = os.path.join(LIB, "libmigraphx_cuda.so")
CHECK_BIN = os.path.join(BIN, "cuda_target_check")
RUNNER_LIB = os.path.join(LIB, "libmgx_cuda_runner.so")
DLOPEN_BIN = os.path.join(BIN, "cuda_dlopen_check")
SOURCES = ["runtime.cpp", "ops_compute.cpp", "lowering.cpp", "target.cpp"]


def _paths():
    mgx_src = os.environ.get("MIGRAPHX_SOURCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    mgx_lib = os.environ.get("MIGRAPHX_LIB_DIR", os.path.join(ROOT, "baseline", "_ref", "lib"))
    gen = os.environ.get("MIGRAPHX_GENERATED_INCLUDE", os.path.join(ROOT, "baseline", "_ref", "gen", "include"))
    return mgx_src, mgx_lib, gen


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build_target(verbose=False, force=False):
    mgx_src, mgx_lib, gen = _paths()
    inc = os.path.join(mgx_src, "src", "include")
    if not os.path.isdir(inc) or not os.path.exists(os.path.join(mgx_lib, "libmigraphx.so")):
        return TARGET_LIB if os.path.exists(TARGET_LIB) else None
    for d in (LIB, BIN, OBJ):
        os.makedirs(d, exist_ok=True)
    cuda_inc = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
    cuda_lib = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/lib64"
    flags = ["-std=c++17", "-O2", "-DNDEBUG", "-fPIC", "-w", "-pthread", "-fvisibility=hidden",
             "-DMIGRAPHX_USE_EIGEN=0", f"-I{gen}", f"-I{inc}",
             f"-I{os.path.join(mgx_src, 'src', 'op', 'builder', 'include')}", f"-I{cuda_inc}"]
    headers = [os.path.join(SRC, f) for f in os.listdir(SRC) if f.endswith(".hpp")]
    headers.append(os.path.join(ROOT, "include", "mgx_cuda.h"))

    def cc(name):
        src = os.path.join(SRC, name)
        obj = os.path.join(OBJ, "target_" + name[:-4] + ".o")
        if force or _newer(obj, [src] + headers):
            r = subprocess.run(["g++", "-c", src, "-o", obj] + flags, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed for {src}:\n{r.stderr[-6000:]}")
        return obj

    with cf.ThreadPoolExecutor(4) as ex:
        objs = list(ex.map(cc, SOURCES))
    if force or _newer(TARGET_LIB, objs):
        cmd = ["g++", "-shared", "-o", TARGET_LIB] + objs + [
            f"-L{LIB}", "-lmgx_cuda_kernels", f"-L{mgx_lib}", "-lmigraphx",
            f"-L{cuda_lib}", "-lcudart",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../baseline/_ref/lib", f"-Wl,-rpath,{cuda_lib}"]
        subprocess.check_call(cmd)
        # register_target.cpp:61-79 looks for libmigraphx_<name>.so.<SOMAJOR> first
        link = TARGET_LIB + ".2016000"
        if os.path.lexists(link):
            os.unlink(link)
        os.symlink(os.path.basename(TARGET_LIB), link)
    # the benchmark's window onto program::compile / program::eval (links the plug-in only)
    runner_src = os.path.join(SRC, "runner.cpp")
    if os.path.exists(runner_src) and (force or _newer(RUNNER_LIB, [runner_src, TARGET_LIB] + headers)):
        cmd = ["g++", "-shared", runner_src, "-o", RUNNER_LIB] + flags + [
            f"-L{LIB}", f"-L{mgx_lib}", "-Wl,--no-as-needed", "-lmigraphx_cuda", "-lmigraphx",
            f"-L{cuda_lib}", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../baseline/_ref/lib",
            f"-Wl,-rpath,{cuda_lib}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed for {runner_src}:\n{r.stderr[-6000:]}")
    check_src = os.path.join(SRC, "check_main.cpp")
    if os.path.exists(check_src) and (force or _newer(CHECK_BIN, [check_src, TARGET_LIB] + headers)):
        ref_lib = os.path.join(ROOT, "oracle", "_ref", "lib")  # the checker: MIGraphX's CPU ref target
        cmd = ["g++", check_src, "-o", CHECK_BIN] + flags + [
            f"-L{LIB}", f"-L{mgx_lib}", f"-L{ref_lib}", "-Wl,--no-as-needed", "-lmigraphx_cuda", "-lmigraphx_ref",
            "-lmigraphx", "-lmgx_cuda_kernels", f"-L{cuda_lib}", "-lcudart",
            "-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath,$ORIGIN/../../baseline/_ref/lib",
            "-Wl,-rpath,$ORIGIN/../../oracle/_ref/lib", f"-Wl,-rpath,{cuda_lib}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed for {check_src}:\n{r.stderr[-6000:]}")
    # an application that links libmigraphx.so only: both targets arrive through dlopen
    dl_src = os.path.join(SRC, "dlopen_main.cpp")
    if os.path.exists(dl_src) and (force or _newer(DLOPEN_BIN, [dl_src] + headers)):
        cmd = ["g++", dl_src, "-o", DLOPEN_BIN] + flags + [
            f"-L{mgx_lib}", "-lmigraphx", "-ldl", "-Wl,-rpath,$ORIGIN/../../baseline/_ref/lib"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed for {dl_src}:\n{r.stderr[-6000:]}")
    return TARGET_LIB


if __name__ == "__main__":
    print(build_target(verbose=True))
