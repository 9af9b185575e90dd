#!/usr/bin/env python3
"""Build the UNMODIFIED MIGraphX core library and its CPU `ref` target from the
reference sources where they lie (both destinations are git-ignored):

  baseline/_ref/lib/libmigraphx.so   the host library (IR, passes, program::compile / eval)
                                     the `cuda` target plug-in plugs into, and
  baseline/_ref/gen/include          the few headers the reference's cmake would generate;
  oracle/_ref/lib/libmigraphx_ref.so MIGraphX's own CPU interpreter target (src/targets/ref):
                                     the parity oracle and the timed CPU baseline, with
  oracle/_ref/lib/libmgx_ref_oracle.so  this repository's C-ABI window onto it.

Only what is under oracle/_ref is test infrastructure; nothing the product links or loads
lives there.

No reference source is copied.  The reference's own build system (cmake +
ROCmCMakeBuildTools) is not run; the few files it would generate are produced
here with the same trivial content:
  * migraphx/export.h, migraphx/ref/export.h  (visibility macros, cmake/ExportHeader)
  * migraphx/version.h                        (src/version.h.in, version from CMakeLists.txt)
  * one translation unit per group of builtin operators holding
    MIGRAPHX_REGISTER_OP(op::<name>) (cmake/RegisterOp.cmake:24-62 over the
    operator list at src/CMakeLists.txt:177-328; the list is parsed from that
    file at build time)
  * stand-ins for msgpack / sqlite (third-party libraries absent here): sqlite throws, the
    msgpack entry points carry JSON text (save / load still round-trip).

Usage: python oracle/build_ref.py [--ref <MIGraphX source tree>] [--jobs 8]
"""
import argparse
import concurrent.futures as cf
import hashlib
import os
import re
import subprocess
import sys
import sysconfig
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")            # ref target, oracle window, object cache
HOST = os.path.join(ROOT, "baseline", "_ref")  # host library + generated headers


def reference_dir():
    """The MIGraphX source tree: $MIGRAPHX_SOURCE_DIR, else a directory named `reference` next
    to this repository."""
    return os.environ.get("MIGRAPHX_SOURCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")


def nlohmann_include():
    cands = [
        os.path.join(sysconfig.get_paths()["purelib"], "include", "cudnn_frontend", "thirdparty"),
        "/usr/include",
    ]
    for c in cands:
        if os.path.exists(os.path.join(c, "nlohmann", "json.hpp")):
            return c
    raise SystemExit("nlohmann/json.hpp not found")


def write_if_changed(path, text):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    if os.path.exists(path) and open(path).read() == text:
        return
    with open(path, "w") as f:
        f.write(text)


def parse_version(ref):
    txt = open(os.path.join(ref, "CMakeLists.txt")).read()
    m = re.search(r"rocm_setup_version\(VERSION\s+(\d+)\.(\d+)\.(\d+)", txt)
    if not m:
        raise SystemExit("cannot find version in reference CMakeLists.txt")
    return tuple(int(x) for x in m.groups())


def parse_ops(ref):
    txt = open(os.path.join(ref, "src", "CMakeLists.txt")).read()
    m = re.search(r"register_migraphx_ops\(\s*\n(.*?)\n\)", txt, re.S)
    ops = m.group(1).split()
    extra = []
    for mm in re.finditer(r"^register_op\(migraphx HEADER (\S+) OPERATORS ([^)]*)\)", txt, re.M):
        extra.append((mm.group(1), mm.group(2).split()))
    return ops, extra


def gen_files(ref, gen):
    major, minor, patch = parse_version(ref)
    inc = os.path.join(gen, "include", "migraphx")
    for name, macro in (("export.h", "MIGRAPHX"), ("ref/export.h", "MIGRAPHX_REF"),
                        ("cuda/export.h", "MIGRAPHX_CUDA")):
        write_if_changed(os.path.join(inc, name), f"""#pragma once
#define {macro}_EXPORT __attribute__((visibility("default")))
#define {macro}_NO_EXPORT __attribute__((visibility("hidden")))
""")
    write_if_changed(os.path.join(inc, "version.h"), f"""#pragma once
#define MIGRAPHX_VERSION_MAJOR {major}
#define MIGRAPHX_VERSION_MINOR {minor}
#define MIGRAPHX_VERSION_PATCH {patch}
#define MIGRAPHX_VERSION_TWEAK ""
#define MIGRAPHX_SO_MAJOR_VERSION ({major} * 1000 * 1000 + {minor} * 1000 + {patch})
""")
    ops, extra = parse_ops(ref)
    units = []
    group = 8
    entries = [(f"migraphx/op/{o}.hpp", [f"op::{o}"]) for o in ops] + extra
    for gi in range(0, len(entries), group):
        body = ["#include <migraphx/register_op.hpp>"]
        for hdr, _ in entries[gi:gi + group]:
            body.append(f"#include <{hdr}>")
        body.append("namespace migraphx {\ninline namespace MIGRAPHX_INLINE_NS {")
        for _, names in entries[gi:gi + group]:
            for n in names:
                body.append(f"MIGRAPHX_REGISTER_OP({n})")
        body.append("} // namespace MIGRAPHX_INLINE_NS\n} // namespace migraphx\n")
        p = os.path.join(gen, "ops", f"register_ops_{gi // group:02d}.cpp")
        write_if_changed(p, "\n".join(body))
        units.append(p)
    stub = os.path.join(gen, "stubs.cpp")
    write_if_changed(stub, """// msgpack-c and sqlite3 are not available in this environment.  sqlite: the entry points exist
// so that the library links, and throw when used.  msgpack: the four entry points carry the
// value's JSON text as their byte stream instead of msgpack (binary blobs included, as json.cpp
// writes them), so that migraphx::save / load round-trip a program in their default format; the
// files are not interchangeable with .mxr files written by a build that has msgpack-c.
#include <migraphx/msgpack.hpp>
#include <migraphx/sqlite.hpp>
#include <migraphx/json.hpp>
#include <migraphx/errors.hpp>
namespace migraphx {
inline namespace MIGRAPHX_INLINE_NS {
std::vector<char> to_msgpack(const value& v)
{
    const auto s = to_json_string(v);
    return {s.begin(), s.end()};
}
void to_msgpack(const value& v, std::function<void(const char*, std::size_t)> writer)
{
    const auto s = to_json_string(v);
    writer(s.data(), s.size());
}
value from_msgpack(const char* buffer, std::size_t size) { return from_json_string(std::string(buffer, size)); }
value from_msgpack(const std::vector<char>& buffer) { return from_msgpack(buffer.data(), buffer.size()); }
sqlite sqlite::read(const fs::path&) { MIGRAPHX_THROW("sqlite unavailable in this build"); }
sqlite sqlite::write(const fs::path&) { MIGRAPHX_THROW("sqlite unavailable in this build"); }
std::vector<std::unordered_map<std::string, std::string>> sqlite::execute(const std::string&) { MIGRAPHX_THROW("sqlite unavailable in this build"); }
} // namespace MIGRAPHX_INLINE_NS
} // namespace migraphx
""")
    units.append(stub)
    return units


def compile_one(args):
    src, obj, flags = args
    if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
        return src, 0, "", 0.0
    os.makedirs(os.path.dirname(obj), exist_ok=True)
    t = time.time()
    r = subprocess.run(["g++", "-c", src, "-o", obj] + flags, capture_output=True, text=True)
    return src, r.returncode, r.stderr[-4000:], time.time() - t


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=reference_dir())
    ap.add_argument("--jobs", type=int, default=max(1, min(8, os.cpu_count() or 1)))
    a = ap.parse_args()
    ref = a.ref
    if not os.path.isdir(os.path.join(ref, "src")):
        print(f"[build_ref] reference sources not found at {ref}; keeping prebuilt files")
        return 0
    gen = os.path.join(HOST, "gen")
    obj = os.path.join(OUT, "obj")
    lib = os.path.join(OUT, "lib")
    hostlib = os.path.join(HOST, "lib")
    os.makedirs(lib, exist_ok=True)
    os.makedirs(hostlib, exist_ok=True)
    gen_units = gen_files(ref, gen)

    src = os.path.join(ref, "src")
    # msgpack.cpp / sqlite.cpp need third-party libraries that are absent (stubs above).
    # fuse_attention.cpp / rewrite_gelu.cpp need tens of GB of compiler memory under
    # g++ 13; only the HIP GPU target's pass list uses them (src/targets/gpu/target.cpp),
    # nothing in the core library or the ref target references their symbols.
    skip = {"msgpack.cpp", "sqlite.cpp", "fuse_attention.cpp", "rewrite_gelu.cpp"}
    core = [os.path.join(src, f) for f in sorted(os.listdir(src))
            if f.endswith(".cpp") and f not in skip]
    bdir = os.path.join(src, "op", "builder")
    core += [os.path.join(bdir, f) for f in sorted(os.listdir(bdir)) if f.endswith(".cpp")]
    core += gen_units
    refdir = os.path.join(src, "targets", "ref")
    reft = [os.path.join(refdir, f) for f in ("target.cpp", "lowering.cpp")]

    base = ["-std=c++17", "-fPIC", "-w", "-pthread", "-DNDEBUG",
            "-DMIGRAPHX_USE_EIGEN=0", "-DMIGRAPHX_HAS_EXECUTORS=0",
            '-DMIGRAPHX_CXX_COMPILER="g++"',
            f"-I{gen}/include", f"-I{src}/include", f"-I{bdir}/include",
            f"-I{refdir}/include", f"-I{nlohmann_include()}"]

    def objname(s):
        h = hashlib.sha1(s.encode()).hexdigest()[:8]
        return os.path.join(obj, os.path.basename(s)[:-4] + "_" + h + ".o")

    jobs = []
    for s in core + reft:
        jobs.append((s, objname(s), base + ["-O2"]))
    t0 = time.time()
    failed = []
    with cf.ThreadPoolExecutor(a.jobs) as ex:
        for i, (s, rc, err, dt) in enumerate(ex.map(compile_one, jobs)):
            if rc != 0:
                failed.append(s)
                print(f"[build_ref] FAILED {s}\n{err}", flush=True)
            elif dt > 0:
                print(f"[build_ref] {i + 1}/{len(jobs)} {os.path.basename(s)} {dt:.0f}s", flush=True)
    if failed:
        print(f"[build_ref] {len(failed)} translation units failed")
        return 1
    core_objs = [objname(s) for s in core]
    ref_objs = [objname(s) for s in reft]
    libmgx = os.path.join(hostlib, "libmigraphx.so")
    libref = os.path.join(lib, "libmigraphx_ref.so")
    newest = max(os.path.getmtime(o) for o in core_objs)
    if not os.path.exists(libmgx) or os.path.getmtime(libmgx) < newest:
        subprocess.check_call(["g++", "-shared", "-o", libmgx] + core_objs + ["-ldl", "-lpthread"])
    if not os.path.exists(libref) or os.path.getmtime(libref) < max(os.path.getmtime(o) for o in ref_objs + [libmgx]):
        subprocess.check_call(["g++", "-shared", "-o", libref] + ref_objs +
                              [f"-L{hostlib}", "-lmigraphx", "-Wl,-rpath,$ORIGIN/../../../baseline/_ref/lib",
                               "-lpthread"])
    # our own C-ABI window onto the ref target (oracle/ref_oracle.cpp)
    tool_src = os.path.join(HERE, "ref_oracle.cpp")
    tool = os.path.join(lib, "libmgx_ref_oracle.so")
    builders = os.path.join(ROOT, "amdmigraphx_b200", "csrc", "target", "programs.hpp")
    if not os.path.exists(tool) or os.path.getmtime(tool) < max(os.path.getmtime(tool_src), os.path.getmtime(libref),
                                                                os.path.getmtime(builders)):
        subprocess.check_call(["g++", "-shared", "-O2", "-o", tool, tool_src] + base +
                              [f"-L{lib}", f"-L{hostlib}", "-Wl,--no-as-needed", "-lmigraphx_ref", "-lmigraphx",
                               "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../../baseline/_ref/lib"])
    # symbol tables of the template-heavy library are ~350 MB; the dynamic symbols stay
    subprocess.call(["strip", "--strip-unneeded", libmgx, libref])
    print(f"[build_ref] done in {time.time() - t0:.0f}s -> {hostlib}, {lib}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
