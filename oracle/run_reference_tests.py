#!/usr/bin/env python3
"""Compile the reference's OWN golden tests for the quantized path, where they lie, against
the oracle build (oracle/_ref/lib) and run them.  This checks that the locally built
MIGraphX `ref` target - the thing the numpy restatement is pinned to - reproduces every
known-answer vector the reference ships for this path:

  test/ref/quantizelinear.cpp, dequantizelinear.cpp, unpack_int4.cpp, pack_int4.cpp,
  pack_unpack_int4.cpp, dot_op.cpp (dot and quant_dot cases)

With --passes it also compiles and runs the reference's tests of the target-independent pieces the
`cuda` plug-in compiles programs with - the same host library the plug-in links: simplify_qdq,
the quantize_* passes, fuse_pointwise, memory_coloring, schedule, replace_allocate,
eliminate_allocation, dead_code_elimination, the interpreter loop (eval_test), the operators' shape
rules (op_shape_test) and the half / fp8e4m3fn types.

Nothing is copied; the executable goes to oracle/_ref/bin/.  The pass/fail summary is
printed; tests/test_reference_golden_tests.py runs this where the reference sources exist.

Usage: python oracle/run_reference_tests.py [--ref <MIGraphX source tree>]
"""
import argparse
import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import build_ref  # noqa: E402

FILES = ["quantizelinear.cpp", "dequantizelinear.cpp", "unpack_int4.cpp", "pack_int4.cpp",
         "pack_unpack_int4.cpp", "dot_op.cpp", "main.cpp"]
# stand-alone test programs of test/ (each has its own main)
PASS_TESTS = ["simplify_qdq_test", "quantization", "fuse_pointwise", "memory_coloring_test", "schedule_test",
              "replace_allocate", "eliminate_allocation_test", "dead_code_elimination_test", "eval_test",
              "op_shape_test", "half", "fp8e4m3fn"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=build_ref.reference_dir())
    ap.add_argument("--passes", action="store_true", help="the tests of the passes and types on the path instead")
    a = ap.parse_args()
    out = os.path.join(HERE, "_ref")
    lib, obj = (os.path.join(out, d) for d in ("lib", "obj"))
    gen = os.path.join(build_ref.HOST, "gen")
    hostlib = os.path.join(build_ref.HOST, "lib")
    bindir = os.path.join(out, "bin")
    os.makedirs(bindir, exist_ok=True)
    tdir = os.path.join(a.ref, "test", "ref")
    flags = ["-std=c++17", "-O1", "-w", "-pthread", "-DMIGRAPHX_USE_EIGEN=0",
             f"-I{gen}/include", f"-I{a.ref}/src/include", f"-I{a.ref}/test/include",
             f"-I{a.ref}/src/targets/ref/include"]

    link = [f"-L{lib}", f"-L{hostlib}", "-Wl,--no-as-needed", "-lmigraphx_ref", "-lmigraphx",
            f"-Wl,-rpath,{lib}", f"-Wl,-rpath,{hostlib}", "-lpthread"]
    if a.passes:
        def build_and_run(name):
            src = os.path.join(a.ref, "test", name + ".cpp")
            exe = os.path.join(bindir, "reftest_" + name)
            if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
                subprocess.check_call(["g++", src, "-o", exe] + flags + link)
            r = subprocess.run([exe], capture_output=True, text=True)
            text = r.stdout + r.stderr
            return name, r.returncode, text.count("[   RUN    ]") or text.count("RUN"), text.count("FAILED")

        with cf.ThreadPoolExecutor(4) as ex:
            results = list(ex.map(build_and_run, PASS_TESTS))
        print("Reference tests of the passes and types on the path (test/<name>.cpp), run against the")
        print("MIGraphX host library + ref target built by oracle/build_ref.py")
        print("command: python oracle/run_reference_tests.py --passes")
        for name, rc, ran, failed in results:
            print(f"{name}: exit code {rc}, cases run {ran}, FAILED {failed}")
        print(f"test cases run: {sum(r[2] for r in results)}")
        print(f"lines containing FAILED: {sum(r[3] for r in results)}")
        return max(abs(r[1]) for r in results)

    def cc(f):
        o = os.path.join(obj, "reftest_" + f[:-4] + ".o")
        src = os.path.join(tdir, f)
        if not os.path.exists(o) or os.path.getmtime(o) < os.path.getmtime(src):
            subprocess.check_call(["g++", "-c", src, "-o", o] + flags)
        return o

    with cf.ThreadPoolExecutor(4) as ex:
        objs = list(ex.map(cc, FILES))
    exe = os.path.join(bindir, "ref_tests")
    subprocess.check_call(["g++", "-o", exe] + objs + link)
    r = subprocess.run([exe], capture_output=True, text=True)
    text = r.stdout + r.stderr
    lines = text.strip().splitlines()
    ran = [l for l in lines if "[   RUN    ]" in l or "RUN" in l]
    failed = [l for l in lines if "FAILED" in l]
    summary = [
        "Reference golden tests (test/ref: " + ", ".join(FILES[:-1]) + ")",
        "run against the MIGraphX core + ref target built by oracle/build_ref.py",
        "command: python oracle/run_reference_tests.py",
        f"exit code: {r.returncode}",
        f"test cases run: {len(ran)}",
        f"lines containing FAILED: {len(failed)}",
    ] + failed[:50] + ["", "tail of output:"] + lines[-8:]
    print("\n".join(summary))
    return r.returncode


if __name__ == "__main__":
    sys.exit(main())
