#!/usr/bin/env python3
"""Benchmark of the quantized-GEMM hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference --gpus N --steps K --warmup W
    python bench.py --case qgemm_i8 --m 3072 --n 3072 --k 768 ...   (one kernel, for profilers)

Workload (own arm): BASELINE config 2 as a MIGraphX program - a BERT-base-shaped int8 encoder
stack in fp16 (token + position embedding, 12 layers of QDQ int8 linears with per-tensor
activation scales from a calibration run and per-channel weight scales, fp16 attention /
softmax / GELU / LayerNorm), batch 8 x 384 tokens - compiled with make_target("cuda") ->
program::compile and run with program::eval through the plug-in (libmigraphx_cuda.so, driven
from here through lib/libmgx_cuda_runner.so).  With N GPUs the batch of 8 sequences is split
into 8/N per GPU (one process and one compiled program per GPU, no data-path collective):
strong scaling.
Metric: int8 QDQ GEMM throughput in TOPS = 2*M*N*K of the program's quant_dots / step time
(the attention, LayerNorm and embedding work of the step is inside the time, not the count).

Reference arm: the same program (one layer, a bounded number of tokens) on MIGraphX's own CPU
`ref` target (oracle/_ref, built from the reference sources) on the host cores.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "int8_qdq_gemm_tops"
UNIT = "TOPS"
BERT = dict(seq=384, layers=12, hidden=768, heads=12, ffn=3072, vocab=30522)
GLOBAL_BATCH = 8
WORKLOAD = ("BERT-base-shaped int8 encoder stack as one MIGraphX program on the cuda target: embedding + "
            "12 layers x [QKV / O / FFN1+GELU / FFN2 QDQ int8 linears, fp16 attention with softmax, "
            "two fp16 LayerNorms], batch 8 x seq 384")


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler(object):
    """nvidia-smi samples of SM clock and throttle reasons while the benchmark runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = []
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) >= 9:
                    rows.append(f)
            os.unlink(self.path)
        except OSError:
            pass
        if not rows:
            return out
        clocks = sorted(float(r[1]) for r in rows if r[1].replace(".", "").isdigit())
        power = [float(r[3]) for r in rows if r[3].replace(".", "").isdigit()]
        # "under load": samples in the upper half of the power range
        if power:
            thr = (max(power) + min(power)) / 2
            loaded = sorted(float(r[1]) for r in rows
                            if r[3].replace(".", "").isdigit() and float(r[3]) >= thr)
            clocks = loaded or clocks
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        out.update(sm_mhz=clocks[len(clocks) // 2] if clocks else None,
                   sm_max_mhz=float(rows[0][2]) if rows[0][2].replace(".", "").isdigit() else None,
                   reasons=sorted(reasons), samples=len(rows),
                   power_w_max=max(power) if power else None)
        return out


# ------------------------------------------------------------------ the plug-in, through the runner
class BertDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("batch", "seq", "layers", "hidden", "heads", "ffn", "vocab")] + \
               [("seed", ctypes.c_uint32), ("offload_copy", ctypes.c_int32), ("fixed_scales", ctypes.c_int32),
                ("reserved", ctypes.c_int32)]


class Runner(object):
    """libmgx_cuda_runner.so: make_target("cuda") -> program::compile -> program::eval."""
    _lib = None

    @classmethod
    def lib(cls):
        if cls._lib is None:
            path = os.path.join(ROOT, "amdmigraphx_b200", "lib", "libmgx_cuda_runner.so")
            if not os.path.exists(path):
                raise SystemExit(f"{path} is missing: build it with `python -m amdmigraphx_b200.build` "
                                 "(the benchmark has no other path to the cuda target)")
            lib = ctypes.CDLL(path)
            vp = ctypes.c_void_p
            lib.mgx_runner_last_error.restype = ctypes.c_char_p
            lib.mgx_runner_create_bert.argtypes = [ctypes.POINTER(BertDesc), ctypes.POINTER(vp)]
            lib.mgx_runner_destroy.argtypes = [vp]
            lib.mgx_runner_set_ids.argtypes = [vp, ctypes.POINTER(ctypes.c_int32), ctypes.c_size_t]
            lib.mgx_runner_eval.argtypes = [ctypes.POINTER(vp), ctypes.c_int, ctypes.c_int,
                                            ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double)]
            lib.mgx_runner_read_output.argtypes = [vp, vp, ctypes.c_size_t]
            lib.mgx_runner_quant_ops.argtypes = [vp]
            lib.mgx_runner_quant_ops.restype = ctypes.c_double
            lib.mgx_runner_tokens.argtypes = [vp]
            lib.mgx_runner_tokens.restype = ctypes.c_int64
            lib.mgx_runner_launches.argtypes = [vp]
            lib.mgx_runner_output_bytes.argtypes = [vp]
            lib.mgx_runner_output_bytes.restype = ctypes.c_size_t
            lib.mgx_runner_op_counts.argtypes = [vp, ctypes.c_char_p, ctypes.c_size_t]
            cls._lib = lib
        return cls._lib

    @classmethod
    def check(cls, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: {cls.lib().mgx_runner_last_error().decode()}")

    def __init__(self, batch, offload, seed=0, fixed_scales=False, **dims):
        d = dict(BERT)
        d.update(dims)
        desc = BertDesc(batch=batch, seed=seed, offload_copy=1 if offload else 0,
                        fixed_scales=1 if fixed_scales else 0, reserved=0, **d)
        self.h = ctypes.c_void_p()
        self.check(self.lib().mgx_runner_create_bert(ctypes.byref(desc), ctypes.byref(self.h)),
                   "mgx_runner_create_bert")
        self.batch, self.seq, self.hidden, self.offload = batch, d["seq"], d["hidden"], offload
        self.quant_ops = self.lib().mgx_runner_quant_ops(self.h)
        self.launches = self.lib().mgx_runner_launches(self.h)
        self.out_bytes = self.lib().mgx_runner_output_bytes(self.h)

    def set_ids(self, ids):
        import numpy as np
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        self.check(self.lib().mgx_runner_set_ids(self.h, ids.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                                                 ids.size), "mgx_runner_set_ids")

    def output(self):
        import numpy as np
        out = np.empty((self.batch * self.seq, self.hidden), dtype=np.float16)
        self.check(self.lib().mgx_runner_read_output(self.h, out.ctypes.data, out.nbytes), "mgx_runner_read_output")
        return out

    def op_counts(self):
        buf = ctypes.create_string_buffer(8192)
        self.lib().mgx_runner_op_counts(self.h, buf, len(buf))
        return json.loads(buf.value.decode())

    @classmethod
    def eval_many(cls, runners, steps):
        """steps x program::eval, rotating over the runners; (device ms, host ms) of the whole run."""
        arr = (ctypes.c_void_p * len(runners))(*[r.h for r in runners])
        dms, wms = ctypes.c_float(0), ctypes.c_double(0)
        cls.check(cls.lib().mgx_runner_eval(arr, len(runners), steps, ctypes.byref(dms), ctypes.byref(wms)),
                  "mgx_runner_eval")
        return float(dms.value), float(wms.value)

    def close(self):
        if self.h:
            self.lib().mgx_runner_destroy(self.h)
            self.h = None


class LlamaDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("batch", "hidden", "heads", "kv_heads", "head", "ffn", "cache", "group")] + \
               [("seed", ctypes.c_uint32), ("reserved", ctypes.c_int32)]


class LlamaLayerRunner(Runner):
    """One Llama-shaped decoder layer at a decode step as a compiled cuda program (device-resident)."""

    def __init__(self, batch, hidden, heads, kv_heads, head, ffn, cache, group=128, seed=1):
        lib = self.lib()
        lib.mgx_runner_create_llama_layer.argtypes = [ctypes.POINTER(LlamaDesc), ctypes.POINTER(ctypes.c_void_p)]
        desc = LlamaDesc(batch=batch, hidden=hidden, heads=heads, kv_heads=kv_heads, head=head, ffn=ffn, cache=cache,
                         group=group, seed=seed, reserved=0)
        self.h = ctypes.c_void_p()
        self.check(lib.mgx_runner_create_llama_layer(ctypes.byref(desc), ctypes.byref(self.h)),
                   "mgx_runner_create_llama_layer")
        self.launches = lib.mgx_runner_launches(self.h)


# ------------------------------------------------------------------ CPU reference legs
def _ref_sample_tokens(budget_s):
    """Tokens of one encoder layer the ref target gets through in about budget_s seconds."""
    from oracle import ref_target as R
    secs, _ = R.time_bert_encoder(1, 16, 1, **{k: BERT[k] for k in ("hidden", "heads", "ffn", "vocab")})
    t = int(16 * budget_s / max(secs, 1e-3))
    return max(16, min(BERT["seq"], t // 16 * 16))


def cpu_reference(steps, warmup, total_budget_s):
    """The benchmark's program (one layer, one sequence of T tokens, T sized to the time budget) on
    MIGraphX's CPU ref target: TOPS over its quant_dots, like the own arm's value."""
    from oracle import ref_target as R
    if not R.available():
        raise SystemExit("oracle/_ref is not built: run `python oracle/build_ref.py` where the MIGraphX "
                         "sources are available")
    tokens = _ref_sample_tokens(total_budget_s / max(1, steps + warmup))
    dims = {k: BERT[k] for k in ("hidden", "heads", "ffn", "vocab")}
    secs, ops = R.time_bert_encoder(1, tokens, 1, warmup=warmup, repeat=steps, **dims)
    return {"value": ops * steps / secs / 1e12, "unit": UNIT, "cores": R.hardware_threads(), "kind": "reference",
            "ms_per_step": secs / steps * 1e3, "tokens": tokens,
            "sample": f"the benchmark's encoder program cut to 1 layer x 1 sequence of {tokens} tokens "
                      f"({ops / 1e9:.2f} GOP of quant_dot per step, {steps} steps in {secs:.1f} s) on MIGraphX's "
                      "CPU ref target"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    r = cpu_reference(args.steps, args.warmup, 150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": r["sample"]},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------ checks of the timed shapes
def _sample_rows(m, n, seed):
    import numpy as np
    if n >= m:
        return np.arange(m)
    rng = np.random.default_rng(seed)
    return np.sort(np.concatenate(([0, m - 1], rng.choice(np.arange(1, m - 1), size=n - 2, replace=False))))


def check_qgemm(dev, m, n, k, kind, out, act, rows=64, seed=0, half_math=False):
    """One launch of the shape against the CPU oracle on a seeded sample of rows (all columns).
    kind: "i8" | "fp8"; out: "f32" | "f16"; half_math: the fp16 model's epilogue (every operator
    rounded to half).  Returns None when it agrees, else a description."""
    import numpy as np
    import torch
    from amdmigraphx_b200 import capi
    from oracle import mgx_oracle as O
    rng = np.random.default_rng(seed)
    a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    b = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    scale = rng.uniform(1e-5, 1e-4, size=n).astype(np.float32)
    bias = rng.normal(0, 0.5, size=n).astype(np.float32)
    ta, tb = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
    odt = torch.float16 if out == "f16" else torch.float32
    if kind == "fp8":
        ta = (ta.float() / 64).to(torch.float8_e4m3fn)
        tb = (tb.float() / 64).to(torch.float8_e4m3fn)
        scale = np.full(1, 3e-2, dtype=np.float32)
    d = capi.qgemm(ta, tb, b_layout=capi.B_NK, scale=torch.from_numpy(scale).to(dev),
                   scale_mode=capi.SCALE_PER_TENSOR if kind == "fp8" else capi.SCALE_PER_COL,
                   bias=torch.from_numpy(bias).to(dev), act=act, out_dtype=odt, half_math=half_math)
    torch.cuda.synchronize()
    pick = _sample_rows(m, rows, seed + 1)
    got = d[torch.from_numpy(pick).to(dev)].float().cpu().numpy()
    if kind == "i8":
        acc = O.quant_dot_int8(a[pick], b.T)
        if half_math:
            ref = O.qlinear_epilogue_half_chain(acc, scale[None, :], bias.astype(np.float16), act)
        else:
            ref = O.qlinear_epilogue(acc, scale[None, :], bias, act, None, np.float16 if out == "f16" else np.float32)
        rtol, atol = (2e-2, 1e-2) if out == "f16" else (1e-5, 1e-5)
    else:
        acc = O.quant_dot_fp8(ta[torch.from_numpy(pick).to(dev)].view(torch.uint8).cpu().numpy(),
                              tb.view(torch.uint8).cpu().numpy().T)
        ref = O.qlinear_epilogue(acc, scale.reshape(1, 1), bias, act, None, np.float32)
        rtol, atol = 2e-2, 1e-2
    ref = ref.astype(np.float32)
    bad = ~(np.abs(got - ref) <= atol + rtol * np.abs(ref))
    if bad.any():
        return f"{kind} {m}x{n}x{k}: {int(bad.sum())} of {bad.size} sampled elements differ from the oracle"
    return None


# ------------------------------------------------------------------ secondary measurements
def _graph_time_us(fn, launches, stream, min_ms=0.0):
    """Average device time of one call of fn, measured over replays of a CUDA graph of `launches`
    calls (at least two replays, and as many as it takes to fill min_ms)."""
    import torch
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(launches):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 2
        while True:
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if ms >= min_ms or reps >= 1 << 16:
                break
            reps = max(reps * 2, int(reps * min_ms / max(ms, 1e-3) * 1.1))
    return ms / (reps * launches) * 1e3


def secondary_measurements(dev, peaks, failures):
    """The other halves of the headline metric, on one GPU: large int8 / fp8 QDQ GEMMs (config 3),
    quantizelinear, and the int4 weight-only linears of Llama-2-7B / 70B-shaped layers (configs 4, 5;
    linears only).  Every timed GEMM shape is first checked against the CPU oracle on sampled rows;
    a shape that fails gets no number."""
    import torch
    from amdmigraphx_b200 import capi
    out = {}
    stream = torch.cuda.Stream()
    peak8 = 2.0 * float(peaks["bf16_tflops"])
    peak8s = 2.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    M = N = K = 8192
    for name, fp8 in (("int8_qdq_gemm_8192", False), ("fp8_qdq_gemm_8192", True)):
        bad = check_qgemm(dev, M, N, K, "fp8" if fp8 else "i8", "f32", "gelu_erf", rows=32)
        if bad:
            failures.append(bad)
            out[name] = {"failed_check": bad}
            continue
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        if fp8:
            a = (a.float() / 64).to(torch.float8_e4m3fn)
            b = (b.float() / 64).to(torch.float8_e4m3fn)
        scale = torch.rand(N, device=dev) * 1e-4
        bias = torch.randn(N, device=dev)
        d = torch.empty((1, M, N), dtype=torch.float32, device=dev)
        fn = lambda: capi.qgemm(a, b, b_layout=capi.B_NK, scale=scale, bias=bias, act="gelu_erf", out=d)  # noqa: E731
        us = _graph_time_us(fn, 4, stream)
        us_long = _graph_time_us(fn, 4, stream, min_ms=1500.0)
        tops, tops_long = 2.0 * M * N * K / us / 1e6, 2.0 * M * N * K / us_long / 1e6
        out[name] = {"us": us, "tops": tops, "frac_of_2x_bf16_burst": tops / peak8,
                     "frac_of_4500_datasheet": tops / 4500.0,
                     "sustained_1p5s": {"us": us_long, "tops": tops_long, "frac_of_2x_bf16_sustained": tops_long / peak8s},
                     "checked": "32 sampled rows x all columns against the CPU oracle",
                     "what": "M=N=K=8192, dequantizelinear + bias + GELU fused, fp32 out"}
        del a, b, d
    # dot on fp16 operands (attention, un-quantised linears), the same kernel with kind::f16 MMAs
    a = torch.randn((M, K), device=dev).half()
    b = torch.randn((N, K), device=dev).half()
    d = torch.empty((1, M, N), dtype=torch.float16, device=dev)
    us = _graph_time_us(lambda: capi.qgemm(a, b, b_layout=capi.B_NK, out=d), 4, stream)
    tf = 2.0 * M * N * K / us / 1e6
    out["fp16_dot_8192"] = {"us": us, "tflops": tf, "frac_of_bf16_burst": tf / float(peaks["bf16_tflops"]),
                            "what": "M=N=K=8192 fp16 x fp16 -> fp32 accumulate -> fp16 out"}
    del a, b, d
    # quantizelinear: fp32 / fp16 -> int8, per-tensor scale; HBM bound (bytes in + out)
    for name, dt, bpe in (("quantizelinear_f32_i8", torch.float32, 5), ("quantizelinear_f16_i8", torch.float16, 3)):
        xs = [torch.randn((8192, 8192), device=dev, dtype=dt) for _ in range(2)]  # 2 x >= 128 MB: larger than L2
        s = torch.tensor([0.02], device=dev, dtype=dt)
        q = torch.empty((8192, 8192), dtype=torch.int8, device=dev)
        import ctypes as C
        lib = capi.load()
        st = (C.c_int64 * 2)(0, 0)
        code = capi.F32 if dt == torch.float32 else capi.F16

        def qfn():
            for x in xs:
                capi.check(lib.mgx_cuda_quantizelinear(C.c_void_p(x.data_ptr()), code, x.stride(0),
                                                       C.c_void_p(s.data_ptr()), st, None, None,
                                                       C.c_void_p(q.data_ptr()), capi.I8, q.stride(0), 8192, 8192,
                                                       capi._stream()), "mgx_cuda_quantizelinear")
        us = _graph_time_us(qfn, 2, stream) / len(xs)
        gbs = 8192 * 8192 * bpe / us / 1e3
        out[name] = {"us": us, "gbs": gbs, "frac_of_measured_hbm": gbs / float(peaks["hbm_gbs"]),
                     "what": f"[8192, 8192] {str(dt).split('.')[-1]} -> int8, per-tensor scale, bytes in + out / time"}
        del xs, q
    # config 3: the fp8 e4m3fn QDQ GEMM sweep (per-tensor scale, bias + GELU fused, fp32 out)
    sweep = {}
    for (n, k) in ((4096, 4096), (8192, 8192), (14336, 4096)):
        b = (torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev).float() / 64).to(torch.float8_e4m3fn)
        scale = torch.full((1,), 3e-4, device=dev)
        bias = torch.randn(n, device=dev)
        for m in (1, 16, 128, 1024, 4096, 8192):
            key = f"M{m}_N{n}_K{k}"
            bad = check_qgemm(dev, m, n, k, "fp8", "f32", "gelu_erf", rows=16, seed=m + n)
            if bad:
                failures.append(bad)
                sweep[key] = {"failed_check": bad}
                continue
            a = (torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev).float() / 64).to(torch.float8_e4m3fn)
            d = torch.empty((1, m, n), dtype=torch.float32, device=dev)
            us = _graph_time_us(lambda: capi.qgemm(a, b, b_layout=capi.B_NK, scale=scale,
                                                   scale_mode=capi.SCALE_PER_TENSOR, bias=bias,
                                                   act="gelu_erf", out=d), 4, stream)
            sweep[key] = {"us": round(us, 2), "tops": round(2.0 * m * n * k / us / 1e6, 1)}
            del a, d
        del b
    out["fp8_qdq_gemm_sweep"] = {"points": sweep, "what": "e4m3fn x e4m3fn -> fp32, per-tensor scale, bias + "
                                 "erf-GELU fused; 4 launches per CUDA graph, operands L2-resident for the small "
                                 "points; every point checked on 16 sampled rows against the CPU oracle first"}
    hid, ffn, group = 4096, 11008, 128
    shapes = [(hid, hid)] * 4 + [(ffn, hid), (ffn, hid), (hid, ffn)]  # q k v o gate up down: (N, K)
    layers = 3  # 3 x 101 MB of packed weights: larger than L2
    weights = []
    for _ in range(layers):
        weights.append([(torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev),
                         (torch.rand(n, k // group, device=dev) * 0.015 + 0.005).half()) for (n, k) in shapes])
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    wbytes = sum(n * k // 2 + n * (k // group) * 2 for (n, k) in shapes)
    for batch in (1, 16):
        xs = {k: torch.randn(batch, k, device=dev, dtype=torch.float16) for k in (hid, ffn)}

        def layer_pass():
            for lw in weights:
                for (bp, sc) in lw:
                    capi.w4a16(xs[bp.shape[1] * 2], bp, sc, group=group, workspace=ws)
        us = _graph_time_us(layer_pass, 2, stream) / layers
        gbs = wbytes / us / 1e3
        out[f"int4_decode_batch{batch}"] = {
            "us_per_layer_linears": us, "tokens_per_s_linears_only_32_layers": batch / (32 * us * 1e-6),
            "weight_gbs": gbs, "frac_of_measured_hbm": gbs / float(peaks["hbm_gbs"]),
            "what": "7 int4 weight-only linears of a Llama-2-7B-shaped layer (group 128, fp16 scales), "
                    "packed weights + scales bytes / time"}
    # prefill: the same seven linears at 512 tokens
    xs = {k: torch.randn(512, k, device=dev, dtype=torch.float16) for k in (hid, ffn)}

    def prefill_pass():
        for (bp, sc) in weights[0]:
            capi.w4a16(xs[bp.shape[1] * 2], bp, sc, group=group, workspace=ws)
    us = _graph_time_us(prefill_pass, 1, stream)
    flops = sum(2.0 * 512 * n * k for (n, k) in shapes)
    out["int4_prefill_512"] = {"us_per_layer_linears": us, "tflops": flops / us / 1e6,
                               "what": "7 int4 weight-only linears of a Llama-2-7B-shaped layer at 512 tokens "
                                       "(tcgen05 fp16 GEMM, weights dequantised in flight into tensor memory)"}
    del weights
    # one large weight matrix (the gate/up projection of a Llama-2-70B-shaped layer)
    n, k = 28672, 8192
    big = [(torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev),
            (torch.rand(n, k // group, device=dev) * 0.015 + 0.005).half()) for _ in range(3)]
    bbytes = n * k // 2 + n * (k // group) * 2
    for batch in (1, 16):
        x = torch.randn(batch, k, device=dev, dtype=torch.float16)

        def big_pass():
            for (bp, sc) in big:
                capi.w4a16(x, bp, sc, group=group, workspace=ws)
        us = _graph_time_us(big_pass, 2, stream) / len(big)
        gbs = bbytes / us / 1e3
        out[f"int4_decode_28672x8192_batch{batch}"] = {
            "us": us, "weight_gbs": gbs, "frac_of_measured_hbm": gbs / float(peaks["hbm_gbs"]),
            "what": "one int4 weight-only linear N=28672 K=8192 (group 128), 3 rotating weight "
                    "copies of 117 MB"}
    del big
    torch.cuda.empty_cache()
    # configs 4 and 5 as programs: one decoder layer at a decode step through the plug-in (RMSNorm,
    # packed-QKV / O / gate / up / down int4 linears, rotary embedding, KV-cache append, decode attention,
    # SwiGLU, residual adds), two compiled instances with their own weights (2 x 101 MB for config 4: more
    # than the L2) and caches taking turns
    for name, dims, layers in (("c4_llama7b_layer_decode_batch1",
                                dict(batch=1, hidden=4096, heads=32, kv_heads=32, head=128, ffn=11008, cache=2048), 32),
                               ("c4_llama7b_layer_decode_batch16",
                                dict(batch=16, hidden=4096, heads=32, kv_heads=32, head=128, ffn=11008, cache=2048), 32),
                               ("c5_llama70b_tp8_shard_layer_decode_batch16",
                                dict(batch=16, hidden=8192, heads=8, kv_heads=1, head=128, ffn=3584, cache=4096), 80)):
        try:
            layers_r = [LlamaLayerRunner(seed=81 + i, **dims) for i in range(2)]
            for _ in range(4):
                Runner.eval_many(layers_r, 2)
            dms, _ = Runner.eval_many(layers_r, 30)
            us = dms / 30 * 1e3
            d = dims
            wbytes = sum(n * k // 2 + n * (k // 128) * 2 for (n, k) in (
                ((d["heads"] + 2 * d["kv_heads"]) * d["head"], d["hidden"]), (d["hidden"], d["heads"] * d["head"]),
                (d["ffn"], d["hidden"]), (d["ffn"], d["hidden"]), (d["hidden"], d["ffn"])))
            # the caches are ~3/4 full in the seeded case (past lengths uniform in [cache / 2, cache))
            kvbytes = 2 * d["batch"] * d["kv_heads"] * int(0.75 * d["cache"]) * d["head"] * 2
            out[name] = {"us_per_layer": us, "launches_per_layer": layers_r[0].launches,
                         "tokens_per_s_at_this_depth": d["batch"] / (layers * us * 1e-6), "layers": layers,
                         "weight_and_cache_gbs": (wbytes + kvbytes) / us / 1e3,
                         "frac_of_measured_hbm": (wbytes + kvbytes) / us / 1e3 / float(peaks["hbm_gbs"]),
                         "what": "one decoder layer per eval() through make_target(\"cuda\") -> compile -> eval, "
                                 "weights + the read part of the KV caches / time"}
            for r in layers_r:
                r.close()
        except RuntimeError as e:
            out[name] = {"error": str(e)[:300]}
    return out


# ------------------------------------------------------------------ own arm
def tp_decode_secondary(dev, world, rank, batch=16, reps=20, nlayers=3):
    """Config 5's tensor parallelism on the ranks of this run: the int4 weight-only linears of a
    Llama-2-70B-shaped decoder layer (hidden 8192, 64 query / 8 KV heads of 128, FFN 28672, group 128)
    at batch 16, QKV and gate/up split by output columns, o_proj and down_proj by input rows with one
    mgx_cuda_all_reduce (NCCL, in place, on the compute stream) after each.  Every rank calls this;
    returns time per layer (max over ranks) and the packed-weight bytes all ranks stream per second."""
    import torch
    import torch.distributed as dist
    from amdmigraphx_b200 import capi
    ids = [capi.Communicator.make_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0, device=dev)
    comm = capi.Communicator(ids[0], world, rank)
    hid, kv, ffn, group = 8192, 2048, 28672, 128
    shapes = [((hid + kv) // world, hid, False), (hid, hid // world, True),
              (2 * ffn // world, hid, False), (hid, ffn // world, True)]
    gen = torch.Generator(device=dev)
    gen.manual_seed(1 + rank)
    layers = [[(torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=gen),
                (torch.rand(n, k // group, device=dev, generator=gen) * 0.015 + 0.005).half(), red)
               for (n, k, red) in shapes] for _ in range(nlayers)]
    xs = {k: torch.randn(batch, k, device=dev, dtype=torch.float16) for (_, k, _) in shapes}
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    wbytes = sum(n * k // 2 + n * (k // group) * 2 for (n, k, _) in shapes)

    def one_layer(lw):
        for (bp, sc, red) in lw:
            y = capi.w4a16(xs[bp.shape[1] * 2], bp, sc, group=group, workspace=ws)
            if red:
                comm.all_reduce_(y)

    for i in range(3):
        one_layer(layers[i % nlayers])
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        one_layer(layers[i % nlayers])
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps * 1e3], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t.item())
    comm.destroy()
    return {"workload": "llama-2-70b-shaped int4 decode linears of one layer, tensor parallel over the run's GPUs "
                        "(column / row split, two all-reduces per layer)",
            "batch": batch, "us_per_layer": us, "weight_gbs_all_ranks": world * wbytes / us / 1e3,
            "all_reduce_bytes": batch * hid * 2, "launches_per_layer": "4 linears (3 kernels each) + 2 all-reduces"}


def read_traffic():
    """DRAM bytes per launch of the dominant kernel from the machine-readable record written next
    to its ncu summary (profiles/qgemm_traffic.json); None when there is no record."""
    p = os.path.join(ROOT, "profiles", "qgemm_traffic.json")
    if not os.path.exists(p):
        return None, None
    d = json.load(open(p))
    return d.get("dram_bytes_per_launch"), d.get("note")


def run_own_arm(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from amdmigraphx_b200 import capi
    from amdmigraphx_b200.workloads import EncoderGemms

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    if GLOBAL_BATCH % world != 0:
        raise SystemExit(f"--gpus must divide the batch of {GLOBAL_BATCH} sequences")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    capi.load()
    batch = GLOBAL_BATCH // world  # this rank's sequences

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        tv = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
        return float(tv.item())

    failures = []
    warm = max(4, args.warmup)  # the target records its CUDA graph on the third eval()
    # ---- the compiled programs.  Three device-resident instances (weights, tables and arena of
    # ~200 MB each) take turns, so that no step finds its weights in the 126 MB L2.
    nsets = 3
    rng = np.random.default_rng(1234 + rank)
    progs = [Runner(batch, offload=False) for _ in range(nsets)]
    for p in progs:
        p.set_ids(rng.integers(0, BERT["vocab"], size=(batch, BERT["seq"])))
    ops_step = progs[0].quant_ops
    launches_step = progs[0].launches
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(warm):
        Runner.eval_many(progs, nsets)
    y0 = progs[0].output().astype(np.float32)
    if not np.isfinite(y0).all() or abs(float(y0.std()) - 1.0) > 0.5:
        failures.append("the encoder program's output is not a LayerNorm-ed tensor (non-finite or wrong spread)")
    barrier()
    dev_ms, wall_ms = Runner.eval_many(progs, args.steps)
    barrier()
    ms_step = max_over_ranks(dev_ms / args.steps)
    wall_step = max_over_ranks(wall_ms / args.steps)

    # ---- end to end: the same program compiled with offload_copy - eval() takes the token ids
    # from (page-locked) host memory and returns the result in host memory; both copies are
    # inside eval() and inside the timed region.
    e2e_progs = [Runner(batch, offload=True) for _ in range(nsets)]
    for p in e2e_progs:
        p.set_ids(rng.integers(0, BERT["vocab"], size=(batch, BERT["seq"])))
    for _ in range(warm):
        Runner.eval_many(e2e_progs, nsets)
    barrier()
    esteps = args.steps
    e_dev_ms, e_wall_ms = Runner.eval_many(e2e_progs, esteps)
    barrier()
    e2e_ms = max_over_ranks(max(e_dev_ms, e_wall_ms) / esteps)
    h2d = batch * BERT["seq"] * 4
    d2h = e2e_progs[0].out_bytes
    op_counts = progs[0].op_counts()
    for p in e2e_progs:
        p.close()

    # ---- roofline leg: the quant_dot launches of a step by themselves, issued through the C ABI
    # exactly as the compiled program issues them (same shapes, epilogues and output types), as one
    # CUDA graph per weight set, replayed for at least a second between CUDA events on the
    # launching stream.
    stream = torch.cuda.Stream()
    chains = [EncoderGemms(dev, tokens=batch * BERT["seq"], seed=s) for s in range(nsets)]
    for (m, n, k, out, act) in chains[0].distinct_shapes():
        bad = check_qgemm(dev, m, n, k, "i8", out, act, rows=48, seed=n + k, half_math=out == "f16")
        if bad:
            failures.append(bad)
    with torch.cuda.stream(stream):
        for c in chains:
            c.step()
        torch.cuda.synchronize()
        graphs = []
        for c in chains:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                c.step()
            graphs.append(g)
        for g in graphs:
            g.replay()
        torch.cuda.synchronize()

        def timed(reps):
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record()
            for i in range(reps):
                graphs[i % nsets].replay()
            r1.record()
            torch.cuda.synchronize()
            return r0.elapsed_time(r1)
        burst_reps = max(3, min(args.steps, 30))
        g_ms = timed(burst_reps)
        long_reps = max(burst_reps, int(1100.0 / max(g_ms / burst_reps, 1e-3)))
        gl_ms = timed(long_reps)
    g_ops = chains[0].ops_per_step()
    g_n = chains[0].gemms_per_step()
    status = capi.device_status()
    clocks = sampler.stop() if sampler is not None else None
    tp = None
    if world > 1 and not args.no_secondary:
        # after the timed regions and the clock samples of the headline
        try:
            tp = tp_decode_secondary(dev, world, rank)
        except Exception as e:  # the secondary figure must not take the headline down with it
            tp = {"error": f"{type(e).__name__}: {e}"}

    if rank == 0:
        peaks, basis = measured_peaks()
        peak8 = 2.0 * float(peaks["bf16_tflops"])
        peak8s = 2.0 * float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
        achieved = g_ops * burst_reps / (g_ms * 1e-3) / 1e12
        achieved_long = g_ops * long_reps / (gl_ms * 1e-3) / 1e12
        traffic, traffic_note = read_traffic()
        line = {
            "metric": METRIC, "value": world * ops_step / (ms_step * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "seq_len": BERT["seq"],
                       "sequences_per_gpu": batch, "tokens_per_gpu": batch * BERT["seq"],
                       "quant_dot_ops_per_step_per_gpu": ops_step,
                       "api": "make_target(\"cuda\") -> program::compile -> program::eval (libmigraphx_cuda.so), one "
                              "eval() per step; host ms per step " + f"{wall_step:.3f}",
                       "launch": f"{launches_step} kernel-launching instructions per eval(), replayed by the target "
                                 "as one CUDA graph",
                       "program_ops": op_counts,
                       "l2": f"{nsets} compiled instances of the program (own weights, tables and arena) take turns: "
                             "consecutive steps share nothing in the 126 MB L2",
                       "parallelism": f"batch {GLOBAL_BATCH} split into {batch} sequence(s) per GPU over {world} "
                                      "GPU(s), no collective"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak8, "unit": "TFLOP/s",
                         "frac": achieved / peak8, "traffic": traffic, "traffic_note": traffic_note,
                         "kernel": "qgemm_kernel (tcgen05 kind::i8): the quant_dot launches of a step "
                                   f"({g_n}, M = {batch * BERT['seq']}) issued as the compiled program issues them and "
                                   "replayed as a CUDA graph of their own, fused epilogues included",
                         "launches_timed": g_n * burst_reps, "avg_launch_us": g_ms / (g_n * burst_reps) * 1e3,
                         "sustained": {"achieved": achieved_long, "seconds": gl_ms * 1e-3,
                                       "frac_of_2x_bf16_sustained": achieved_long / peak8s,
                                       "frac_of_2x_bf16_burst": achieved_long / peak8},
                         "frac_of_4500_datasheet": achieved / 4500.0,
                         "peak_basis": f"2 x {basis} bf16 burst ({peaks['bf16_tflops']} TFLOP/s): "
                                       "8-bit operands issue at twice the bf16 rate"},
            "e2e": {"value": world * ops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "how": "program compiled with offload_copy: every eval() copies the token ids from page-locked "
                           "host memory to the device, runs the program and copies the fp16 result to page-locked "
                           "host memory; one eval() per step, nothing overlaps between steps"},
            "gpu_launches": args.steps * launches_step,
            "clocks": clocks, "device_status": status,
        }
        if world == 1 and not args.no_secondary:
            line["secondary"] = secondary_measurements(dev, peaks, failures)
        if tp is not None:
            line["secondary"] = {"tp_int4_decode_llama70b": tp}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = {k: v for k, v in cpu_reference(3, 1, 20.0).items()
                                    if k in ("value", "unit", "cores", "kind", "sample")}
        if failures or status != 0:
            # a number for work that came out wrong is worth nothing
            print(json.dumps({"error": "parity check failed", "failures": failures, "device_status": status}),
                  flush=True)
            if world > 1:
                dist.destroy_process_group()
            return 1
        print(json.dumps(line), flush=True)
    for p in progs:
        p.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------ single-kernel cases
def run_case(a):
    """One kernel launched --iters times on inputs larger than L2; prints the CUDA-event time per
    launch with the algorithmic work rate.  The commands of the ncu summaries under profiles/."""
    import torch
    from amdmigraphx_b200 import capi
    dev = torch.device("cuda:0")
    M, N, K = a.m, a.n, a.k
    act = None if a.act == "none" else a.act
    if a.case == "encoder":
        # the benchmark's program by itself: --m sequences, --n layers, fixed activation scales (no
        # calibration run, so that the launches of the process are those of eval() alone)
        import numpy as np
        r = Runner(a.m, offload=False, fixed_scales=True, layers=a.n)
        r.set_ids(np.random.default_rng(0).integers(0, BERT["vocab"], size=(a.m, BERT["seq"])))
        for _ in range(a.case_warmup):
            Runner.eval_many([r], 1)
        dms, wms = Runner.eval_many([r], a.iters)
        print(json.dumps({"case": a.case, "sequences": a.m, "layers": a.n, "launches_per_eval": r.launches,
                          "device_ms_per_eval": dms / a.iters, "host_ms_per_eval": wms / a.iters,
                          "tops": r.quant_ops / (dms / a.iters * 1e-3) / 1e12, "ops": r.op_counts(),
                          "device_status": capi.device_status()}))
        return 0
    if a.case == "llama_layer":
        # a decoder layer at a decode step through the plug-in, --m batch entries: config 4 (2048 cached
        # positions), or with --kv-heads 1 one tensor-parallel shard (of 8) of config 5 (4096 cached positions)
        if a.kv_heads == 1:
            r = LlamaLayerRunner(batch=a.m, hidden=8192, heads=8, kv_heads=1, head=128, ffn=3584, cache=4096)
        else:
            r = LlamaLayerRunner(batch=a.m, hidden=4096, heads=32, kv_heads=32, head=128, ffn=11008, cache=2048)
        for _ in range(a.case_warmup):
            Runner.eval_many([r], 1)
        dms, wms = Runner.eval_many([r], a.iters)
        print(json.dumps({"case": a.case, "batch": a.m, "launches_per_eval": r.launches,
                          "device_us_per_eval": dms / a.iters * 1e3, "host_us_per_eval": wms / a.iters * 1e3,
                          "ops": r.op_counts(), "device_status": capi.device_status()}))
        return 0
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
                                    residual=res, q_out=qo, q_scale=0.02 if a.qout else None,
                                    write_d=not a.qonly, half_math=a.half_math)
        work, unit = 2.0 * M * N * K, "TOPS"
    elif a.case == "quantize":
        x = torch.randn((M, N), device=dev, dtype=torch.float16 if a.out == "f16" else torch.float32)
        s = torch.tensor([0.02], device=dev, dtype=x.dtype)
        fn = lambda: capi.quantizelinear(x, s, out_dtype=torch.int8)  # noqa: E731
        work, unit = (x.element_size() + 1.0) * M * N, "GB/s"
    elif a.case == "attention":
        # --m sequences of --n tokens, --k heads of 64: the encoder's attention on a fused QKV buffer
        width = K * 64
        qkv = torch.randn((M * N, 3 * width), device=dev, dtype=torch.float16)
        q, k_, v = qkv[:, :width], qkv[:, width:2 * width], qkv[:, 2 * width:]
        fn = lambda: capi.attention(q, k_, v, M, N, K, 0.125, q_scale=0.006,  # noqa: E731
                                    fp32_softmax=a.act == "fp32")
        work, unit = 4.0 * M * K * N * N * 64, "TOPS"
    elif a.case == "gqa_decode":
        # --m batch entries, --n cache positions (all valid), --k query heads, --kv-heads KV heads of 128
        kc = torch.randn((M, a.kv_heads, N, 128), device=dev, dtype=torch.float16)
        vc = torch.randn((M, a.kv_heads, N, 128), device=dev, dtype=torch.float16)
        qd = torch.randn((M, K, 128), device=dev, dtype=torch.float16)
        lens = torch.full((M, 1), N - 1, dtype=torch.int32, device=dev)
        fn = lambda: capi.gqa_decode_attention(qd, kc, vc, lens, 0.08837890625)  # noqa: E731
        work, unit = 2.0 * kc.numel() * 2, "GB/s"
    elif a.case == "layernorm":
        x = torch.randn((M, N), device=dev, dtype=torch.float16)
        g = torch.randn(N, device=dev, dtype=torch.float16)
        b_ = torch.randn(N, device=dev, dtype=torch.float16)
        fn = lambda: capi.layernorm(x, g, b_, 1e-12, q_scale=0.04, dq_scale=0.04)  # noqa: E731
        work, unit = (2.0 + 2.0 + 1.0 + 2.0) * M * N, "GB/s"
    else:
        x = torch.randn((M, K), device=dev, dtype=torch.float16)
        bp = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev)
        sc = (torch.rand(N, K // 128, device=dev) * 0.015 + 0.005).half()
        fn = lambda: capi.w4a16(x, bp, sc)  # noqa: E731
        work, unit = N * K / 2 + N * K / 128 * 2 + 2 * M * K + 2 * M * N, "GB/s"
    for _ in range(a.case_warmup):
        fn()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(a.iters):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / a.iters
    rate = work / (ms * 1e-3) / (1e12 if unit == "TOPS" else 1e9)
    print(json.dumps({"case": a.case, "m": M, "n": N, "k": K, "us_per_launch": ms * 1e3,
                      "rate": rate, "unit": unit, "device_status": capi.device_status()}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--case", default=None, choices=["qgemm_i8", "qgemm_fp8", "quantize", "w4a16", "encoder", "attention", "layernorm",
                                                        "gqa_decode", "llama_layer"],
                    help="run one kernel by itself (for profiler captures) instead of the benchmark")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--kv-heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--case-warmup", type=int, default=1)
    ap.add_argument("--act", default="gelu_erf")
    ap.add_argument("--out", default="f16", choices=["f16", "f32", "raw"])
    ap.add_argument("--residual", action="store_true", help="--case: add a residual of the output type")
    ap.add_argument("--qout", action="store_true", help="--case: also write the int8 quantizelinear of the output")
    ap.add_argument("--half-math", action="store_true",
                    help="--case: fp16 output whose epilogue operators round to half one by one (fp16 models)")
    ap.add_argument("--qonly", action="store_true", help="--case: with --qout, write only the quantised output")
    args = ap.parse_args()
    if args.case is not None:
        return run_case(args)
    # One JSON line on stdout, whatever libraries print (NCCL announces its version there): during
    # the run file descriptor 1 points at stderr, and print() goes to the real stdout.
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = real_stdout
    try:
        if args.impl == "reference":
            return run_reference_arm(args)
        return run_own_arm(args)
    finally:
        real_stdout.flush()


if __name__ == "__main__":
    sys.exit(main())
