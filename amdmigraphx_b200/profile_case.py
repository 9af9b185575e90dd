"""Small single-kernel cases for profiler captures and timing.

    python -m amdmigraphx_b200.profile_case qgemm_i8 --m 8192 --n 8192 --k 8192 --iters 3
    python -m amdmigraphx_b200.profile_case qgemm_fp8 | quantize | w4a16

Each case launches one kernel `--iters` times on inputs larger than the L2 cache and prints
the CUDA-event time per launch with the algorithmic work rate.
"""
import argparse
import json

from . import capi


def main():
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["qgemm_i8", "qgemm_fp8", "quantize", "w4a16"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--act", default="gelu_erf")
    ap.add_argument("--out", default="f16", choices=["f16", "f32", "raw"])
    ap.add_argument("--residual", action="store_true", help="add a residual of the output type")
    ap.add_argument("--qout", action="store_true", help="also write the int8 quantizelinear of the output")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    M, N, K = a.m, a.n, a.k
    act = None if a.act == "none" else a.act
    if a.case in ("qgemm_i8", "qgemm_fp8"):
        A = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        B = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        if a.case == "qgemm_fp8":
            A = (A.float() / 64).to(torch.float8_e4m3fn)
            B = (B.float() / 64).to(torch.float8_e4m3fn)
        scale = torch.rand(N, device=dev) * 1e-4
        bias = torch.randn(N, device=dev)
        if a.out == "raw":
            odt = torch.int32 if a.case == "qgemm_i8" else torch.float32
            out = torch.empty((1, M, N), dtype=odt, device=dev)
            fn = lambda: capi.qgemm(A, B, b_layout=capi.B_NK, out=out)  # noqa: E731
        else:
            out = torch.empty((1, M, N), dtype=torch.float16 if a.out == "f16" else torch.float32, device=dev)
            res = torch.randn((1, M, N), device=dev).to(out.dtype) if a.residual else None
            qo = torch.empty((1, M, N), dtype=torch.int8, device=dev) if a.qout else None
            fn = lambda: capi.qgemm(A, B, b_layout=capi.B_NK, scale=scale, bias=bias, act=act, out=out,  # noqa: E731
                                    residual=res, q_out=qo, q_scale=0.02 if a.qout else None)
        work, unit = 2.0 * M * N * K, "TOPS"
    elif a.case == "quantize":
        x = torch.randn((M, N), device=dev)
        s = torch.tensor([0.02], device=dev)
        fn = lambda: capi.quantizelinear(x, s, out_dtype=torch.int8)  # noqa: E731
        work, unit = 5.0 * M * N, "GB/s"
    else:
        x = torch.randn((M, K), device=dev, dtype=torch.float16)
        bp = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev)
        sc = (torch.rand(N, K // 128, device=dev) * 0.015 + 0.005).half()
        fn = lambda: capi.w4a16(x, bp, sc)  # noqa: E731
        work, unit = N * K / 2 + N * K / 128 * 2 + 2 * M * K + 2 * M * N, "GB/s"
    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / a.iters
    rate = work / (ms * 1e-3) / (1e12 if unit == "TOPS" else 1e9)
    print(json.dumps({"case": a.case, "m": M, "n": N, "k": K, "us_per_launch": ms * 1e3,
                      "rate": rate, "unit": unit, "device_status": capi.device_status()}))


if __name__ == "__main__":
    main()
