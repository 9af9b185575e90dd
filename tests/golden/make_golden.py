#!/usr/bin/env python3
"""Generate tests/golden/ref_fixtures.npz: seeded inputs and the outputs MIGraphX's own
`ref` target (built from the reference sources by oracle/build_ref.py) produces for them.

The fixtures travel with the repository, so the CPU tests can pin the numpy restatement
and the GPU tests can check the CUDA kernels against the real reference on machines where
the reference sources and its build are absent.

Usage: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import ref_target as R  # noqa: E402
from oracle import mgx_oracle as O  # noqa: E402  (only for fp8 encoding of inputs)


def main():
    rng = np.random.default_rng(20240607)
    fx = {}

    # ---- quantizelinear: per-tensor, per-channel, zero points, ties, saturation -------
    for tag, dt in (("f32", np.float32), ("f16", np.float16)):
        x = (rng.normal(0, 1, size=(24, 64)) * 3).astype(dt)
        x.flat[:8] = np.array([0.01, 0.03, -0.01, -0.03, 1000, -1000, 0.05, -0.05], dtype=dt)
        s = np.array([0.02], dtype=dt)
        fx[f"q_{tag}_x"] = x
        fx[f"q_{tag}_scale"] = s
        fx[f"q_{tag}_i8"] = R.quantizelinear(x, s, None, "int8")
        fx[f"q_{tag}_u8_zp128"] = R.quantizelinear(x, s, np.array([128], dtype=np.uint8), "uint8")
        fx[f"q_{tag}_fp8"] = R.quantizelinear(x, s, None, "fp8e4m3fn")
    x = rng.normal(0, 2, size=(24, 64)).astype(np.float32)
    s_col = rng.uniform(0.01, 0.05, size=(1, 64)).astype(np.float32)
    z_col = rng.integers(-20, 20, size=(1, 64)).astype(np.int8)
    fx["qc_x"], fx["qc_scale"], fx["qc_zp"] = x, s_col, z_col
    fx["qc_i8"] = R.quantizelinear(x, s_col, z_col, "int8")

    # ---- dequantizelinear ---------------------------------------------------------------
    xi = rng.integers(-2 ** 26, 2 ** 26, size=(16, 48)).astype(np.int32)
    sc = rng.uniform(1e-5, 1e-3, size=(1, 48)).astype(np.float32)
    fx["dq_i32_x"], fx["dq_i32_scale"] = xi, sc
    fx["dq_i32_y"] = R.dequantizelinear(xi, sc)
    x8 = rng.integers(0, 256, size=(16, 48)).astype(np.uint8)
    z8 = rng.integers(0, 16, size=(1, 48)).astype(np.uint8)
    sh = rng.uniform(0.005, 0.02, size=(1, 48)).astype(np.float16)
    fx["dq_u8_x"], fx["dq_u8_zp"], fx["dq_u8_scale"] = x8, z8, sh
    fx["dq_u8_y"] = R.dequantizelinear(x8, sh, z8)
    codes = rng.integers(0, 0x7F, size=(16, 48)).astype(np.uint8)
    codes |= rng.integers(0, 2, size=codes.shape).astype(np.uint8) << 7
    fx["dq_fp8_x"] = codes
    fx["dq_fp8_y"] = R.dequantizelinear(codes, sc, None, True)

    # ---- int4 pack / unpack -------------------------------------------------------------
    p = rng.integers(0, 256, size=(6, 32)).astype(np.uint8)
    fx["u4_packed"] = p
    fx["u4_unpacked_u8"] = R.unpack_int4(p)
    fx["u4_unpacked_i8"] = R.unpack_int4(p.view(np.int8))
    v = rng.integers(-20, 30, size=(6, 64)).astype(np.int8)
    fx["p4_values_i8"] = v
    fx["p4_packed_i8"] = R.pack_int4(v)
    fx["p4_packed_u8"] = R.pack_int4(v.astype(np.uint8))

    # ---- quant_dot ----------------------------------------------------------------------
    a = rng.integers(-128, 128, size=(2, 72, 160)).astype(np.int8)
    b = rng.integers(-128, 128, size=(2, 160, 48)).astype(np.int8)
    fx["qd_i8_a"], fx["qd_i8_b"] = a, b
    fx["qd_i8_c"] = R.quant_dot(a, b)
    af = O.fp8e4m3fn_encode(rng.normal(0, 60, size=(40, 128)).clip(-448, 448))
    bf = O.fp8e4m3fn_encode(rng.normal(0, 60, size=(128, 56)).clip(-448, 448))
    fx["qd_fp8_a"], fx["qd_fp8_b"] = af, bf
    fx["qd_fp8_c"] = R.quant_dot(af, bf, fp8=True)

    # ---- config-1 shaped block at reduced size: Q -> quant_dot -> DQ -> add -> relu/gelu --
    M, K, N = 64, 256, 96
    x = rng.normal(0, 1, size=(M, K)).astype(np.float32)
    w = rng.integers(-127, 128, size=(K, N)).astype(np.int8)
    xs = np.array([0.02], dtype=np.float32)
    ws = rng.uniform(0.001, 0.01, size=N).astype(np.float32)
    bias = rng.normal(0, 0.1, size=N).astype(np.float32)
    xq = R.quantizelinear(x, xs, None, "int8")
    acc = R.quant_dot(xq, w)
    scale = R.binary("mul", np.broadcast_to(xs, (M, N)).copy(), np.broadcast_to(ws, (M, N)).copy())
    fx["blk_x"], fx["blk_w"], fx["blk_xscale"], fx["blk_wscale"], fx["blk_bias"] = x, w, xs, ws, bias
    fx["blk_xq"], fx["blk_acc"], fx["blk_scale"] = xq, acc, scale[0].copy()
    fx["blk_relu"] = R.qlinear_epilogue(acc, scale, bias, "relu")
    fx["blk_gelu"] = R.qlinear_epilogue(acc, scale, bias, "gelu_erf")
    fx["blk_none"] = R.qlinear_epilogue(acc, scale, bias, None)

    # ---- weight-only int4 linear (MatMulNBits IR) -----------------------------------------
    for tag, (M, N, K, g) in {"a": (3, 40, 256, 128), "b": (16, 64, 512, 32)}.items():
        a16 = rng.normal(0, 1, size=(M, K)).astype(np.float16)
        bp = rng.integers(0, 256, size=(N, K // 2)).astype(np.uint8)
        s16 = rng.uniform(0.005, 0.02, size=(N, K // g)).astype(np.float16)
        zp = rng.integers(0, 16, size=(N, K // g)).astype(np.uint8)
        fx[f"w4{tag}_a"], fx[f"w4{tag}_bp"], fx[f"w4{tag}_scales"], fx[f"w4{tag}_zp"] = a16, bp, s16, zp
        fx[f"w4{tag}_group"] = np.array([g])
        fx[f"w4{tag}_y_zp8"] = R.w4a16_linear(a16, bp, s16, None, 8, g)
        fx[f"w4{tag}_y_zp"] = R.w4a16_linear(a16, bp, s16, zp, 8, g)

    out = os.path.join(HERE, "ref_fixtures.npz")
    np.savez_compressed(out, **fx)
    print(f"wrote {out}: {len(fx)} arrays, {os.path.getsize(out) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
