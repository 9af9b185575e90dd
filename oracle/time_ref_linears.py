"""Times MIGraphX's own `ref` target (the build under oracle/_ref) on single linears of the
benchmark configurations: the CPU baseline of the quantized path, one operator at a time.

Test infrastructure, like everything under oracle/: nothing of the product imports it.

  fp8 sweep      quant_dot e4m3fn [M,4096] x [4096,4096] -> float, M = 1, 16, 128, in full
                 (src/targets/ref/lowering.cpp:205-249 -> gemm_naive, src/gemm.cpp:43-63)
  int4 decoders  every linear shape of Llama-2-7B and Llama-2-70B at one token:
                 unpack_int4 -> dequantizelinear (fp16, groups of 128) -> dot, the operators the
                 MatMulNBits parser emits (src/onnx/parse_matmulnbits.cpp:85-158); `ref` dequantises
                 the whole [N,K] weight on every evaluation, so that is part of its time

Usage: python oracle/time_ref_linears.py [--quick]     (prints one JSON object per line)
"""
import argparse
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import ref_target as R  # noqa: E402


def time_fp8(m, n, k, rng):
    a = rng.integers(0, 0x78, size=(m, k), dtype=np.uint8)  # finite e4m3fn codes
    b = rng.integers(0, 0x78, size=(k, n), dtype=np.uint8)
    _, secs = R.quant_dot(a, b, fp8=True, want_seconds=True)
    return {"config": "fp8 sweep", "op": "quant_dot fp8e4m3fn", "M": m, "N": n, "K": k, "seconds": secs,
            "gops": 2.0 * m * n * k / secs / 1e9}


def time_int4(name, m, n, k, rng, group=128):
    bp = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = rng.uniform(0.005, 0.02, size=(n, k // group)).astype(np.float16)
    a = rng.normal(0, 1, size=(m, k)).astype(np.float16)
    t0 = time.perf_counter()
    q = R.unpack_int4(bp)
    t1 = time.perf_counter()
    s = np.repeat(scales, group, axis=1)
    z = np.full(q.shape, 8, dtype=np.uint8)
    t2 = time.perf_counter()
    w = R.dequantizelinear(q, s, z)
    t3 = time.perf_counter()
    wt = np.ascontiguousarray(w.T)
    t4 = time.perf_counter()
    R.dot(a, wt)
    t5 = time.perf_counter()
    ref_seconds = (t1 - t0) + (t3 - t2) + (t5 - t4)  # the three ref operators; numpy staging left out
    return {"config": name, "op": "unpack_int4 + dequantizelinear + dot (fp16)", "M": m, "N": n, "K": k,
            "seconds": ref_seconds, "unpack_s": t1 - t0, "dequantize_s": t3 - t2, "dot_s": t5 - t4,
            "weight_bytes": n * k // 2 + 2 * n * k // group}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="the smallest shape of each kind only")
    a = ap.parse_args()
    if not R.available():
        print(json.dumps({"unavailable": "oracle/_ref is not built (oracle/build_ref.py)"}))
        return 1
    rng = np.random.default_rng(0)
    print(json.dumps({"threads": R.hardware_threads()}), flush=True)
    for m in ((1,) if a.quick else (1, 16, 128)):
        print(json.dumps(time_fp8(m, 4096, 4096, rng)), flush=True)
    llama7b = [("Llama-2-7B q/k/v/o", 4096, 4096), ("Llama-2-7B gate/up", 11008, 4096),
               ("Llama-2-7B down", 4096, 11008)]
    llama70b = [("Llama-2-70B q/o", 8192, 8192), ("Llama-2-70B k/v", 1024, 8192),
                ("Llama-2-70B gate/up", 28672, 8192), ("Llama-2-70B down", 8192, 28672)]
    for name, n, k in (llama7b[:1] if a.quick else llama7b + llama70b):
        print(json.dumps(time_int4(name, 1, n, k, rng)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
