"""Synthetic workloads of the quantized-GEMM path, assembled from C-ABI calls.

BertInt8LinearStack is the QDQ-linear part of a BERT-base-shaped int8 encoder stack
(12 layers, hidden 768, FFN 3072, tokens = batch x 384): per layer four quantizelinear
launches and four quant_dot launches whose epilogues carry dequantizelinear (per-tensor
activation scale x per-channel weight scale), bias, erf-GELU (FFN1) or the residual add
(O-proj, FFN2).  The Q/K/V projections share their input and are issued as one quant_dot
with the three weight matrices concatenated along N, the horizontal fusion MIGraphX
applies to dots with a common input.  Attention scores/softmax and LayerNorm are not part
of this stack: the chain stays data dependent by feeding the Q slice of the QKV output
forward.

Weights are random int8 with per-output-channel scales, stored [N, K] (K contiguous), the
layout the `cuda` target gives constant weights at finalize time.
"""
import numpy as np

from . import capi


class QLinear(object):
    """One QDQ linear: y = act(dequant(quant_dot(quantizelinear(x), W)) + bias) (+ residual)."""

    def __init__(self, rng, k, n, device, act_scale=0.02, act=None):
        import torch
        self.k, self.n, self.act = k, n, act
        w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        w_scale = rng.uniform(0.001, 0.01, size=n).astype(np.float32)
        x_scale = np.array([act_scale], dtype=np.float32)
        self.w_nk_host = w
        self.w = torch.from_numpy(w).to(device)                      # [N, K]
        self.x_scale = torch.from_numpy(x_scale).to(device)
        # the scale literal simplify_qdq leaves: mul(bcast(x_scale), bcast(w_scale)) in fp32
        self.scale_host = (x_scale * w_scale).astype(np.float32)
        self.scale = torch.from_numpy(self.scale_host).to(device)
        self.bias_host = rng.normal(0, 0.1, size=n).astype(np.float32)
        self.bias = torch.from_numpy(self.bias_host).to(device)
        self.x_scale_host = x_scale

    def ops(self, m):
        return 2 * m * self.n * self.k


class BertInt8LinearStack(object):
    def __init__(self, device, layers=12, hidden=768, ffn=3072, tokens=3072, seed=0, fuse_quant=True):
        import torch
        self.fuse_quant = fuse_quant
        rng = np.random.default_rng(seed)
        self.device, self.tokens, self.hidden, self.ffn = device, tokens, hidden, ffn
        self.layers = []
        for _ in range(layers):
            self.layers.append({
                "qkv": QLinear(rng, hidden, 3 * hidden, device),
                "o": QLinear(rng, hidden, hidden, device),
                "ffn1": QLinear(rng, hidden, ffn, device, act="gelu_erf"),
                "ffn2": QLinear(rng, ffn, hidden, device, act_scale=0.01),
            })
        t = tokens
        f16 = dict(dtype=torch.float16, device=device)
        i8 = dict(dtype=torch.int8, device=device)
        self.x = torch.empty((t, hidden), **f16)
        self.xq = torch.empty((t, hidden), **i8)
        self.qkv = torch.empty((t, 3 * hidden), **f16)
        self.cq = torch.empty((t, hidden), **i8)
        self.o = torch.empty((t, hidden), **f16)
        self.oq = torch.empty((t, hidden), **i8)
        self.h = torch.empty((t, ffn), **f16)
        self.hq = torch.empty((t, ffn), **i8)
        self.y = torch.empty((t, hidden), **f16)

    # -- bookkeeping ---------------------------------------------------------------------
    def ops_per_step(self):
        return sum(l.ops(self.tokens) for layer in self.layers for l in layer.values())

    def launches_per_step(self):
        # fused: the quantizelinear feeding O-proj's successor, FFN2 and the next layer's QKV
        # runs inside the producing GEMM's epilogue; only the attention-context one stays
        if self.fuse_quant:
            return len(self.layers) * 5 + 1
        return len(self.layers) * 8

    def gemms_per_step(self):
        return len(self.layers) * 4

    def weight_bytes(self):
        return sum(l.w.numel() for layer in self.layers for l in layer.values())

    # -- one QDQ linear through the C ABI --------------------------------------------------
    def _quant(self, x, xq, lin):
        lib = capi.load()
        import ctypes
        rows, cols = x.shape
        st = (ctypes.c_int64 * 2)(0, 0)
        capi.check(lib.mgx_cuda_quantizelinear(
            ctypes.c_void_p(x.data_ptr()), capi.F16, x.stride(0), ctypes.c_void_p(lin.x_scale_f16.data_ptr()),
            st, None, None, ctypes.c_void_p(xq.data_ptr()), capi.I8, xq.stride(0), rows, cols,
            capi._stream()), "mgx_cuda_quantizelinear")

    def _gemm(self, xq, lin, out, residual=None, q_out=None, q_lin=None, write_d=True):
        capi.qgemm(xq, lin.w, b_layout=capi.B_NK, scale=lin.scale, scale_mode=capi.SCALE_PER_COL,
                   bias=lin.bias, act=lin.act, residual=residual, out=out, q_out=q_out,
                   q_scale=None if q_lin is None else q_lin.x_scale_f16_host, write_d=write_d)

    def prepare(self):
        """fp16 copies of the activation scales (quantizelinear takes its scale in x's type)."""
        import torch
        for layer in self.layers:
            for lin in layer.values():
                lin.x_scale_f16 = lin.x_scale.to(torch.float16)
                lin.x_scale_f16_host = float(np.float16(lin.x_scale_host[0]))

    def step(self, x_in=None, gemm_only=False):
        """One pass over the stack; returns the last layer's output [tokens, hidden] fp16.
        gemm_only leaves out the stand-alone quantizelinear launches (the quant_dot launches
        then read whatever an earlier full pass left in their int8 inputs): the same 48
        quant_dot launches by themselves, for timing the dominant kernel."""
        x = self.x if x_in is None else x_in
        quant = (lambda *a: None) if gemm_only else self._quant
        if not self.fuse_quant:
            for layer in self.layers:
                quant(x, self.xq, layer["qkv"])
                self._gemm(self.xq, layer["qkv"], self.qkv)
                ctx = self.qkv[:, : self.hidden]  # stand-in for the attention context (row stride 3*hidden)
                quant(ctx, self.cq, layer["o"])
                self._gemm(self.cq, layer["o"], self.o, residual=x if x.stride(0) == self.o.stride(0) else None)
                quant(self.o, self.oq, layer["ffn1"])
                self._gemm(self.oq, layer["ffn1"], self.h)
                quant(self.h, self.hq, layer["ffn2"])
                self._gemm(self.hq, layer["ffn2"], self.y, residual=self.o)
                x = self.y
            return self.y
        # fused form: every quantizelinear whose input is produced by a GEMM epilogue runs there
        # (dequantizelinear -> add -> [gelu] -> [add] -> quantizelinear is one pointwise module)
        quant(x, self.xq, self.layers[0]["qkv"])
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1]["qkv"] if i + 1 < len(self.layers) else None
            self._gemm(self.xq, layer["qkv"], self.qkv)
            ctx = self.qkv[:, : self.hidden]
            quant(ctx, self.cq, layer["o"])
            self._gemm(self.cq, layer["o"], self.o, residual=x if x.stride(0) == self.o.stride(0) else None,
                       q_out=self.oq, q_lin=layer["ffn1"])
            # FFN1's fp16 output has no other consumer: only its quantised form is written
            self._gemm(self.oq, layer["ffn1"], self.h, q_out=self.hq, q_lin=layer["ffn2"], write_d=False)
            self._gemm(self.hq, layer["ffn2"], self.y, residual=self.o,
                       q_out=self.xq if nxt is not None else None, q_lin=nxt)
            x = self.y
        return self.y


class EncoderGemms(object):
    """The quant_dot launches of one step of the BERT-shaped int8 encoder program, issued through
    the C ABI with the shapes, epilogues and output types the `cuda` target's lowering gives them
    (csrc/target/lowering.cpp): per layer the Q/K/V projections (one launch of N = 3 x hidden when
    the lowering fuses them, else three), the attention output projection (+ residual), FFN1
    (+ erf-GELU, only its int8 quantizelinear written) and FFN2 (+ residual); fp16 results.
    The int8 inputs hold random data: this chain exists to time the dominant kernel by itself."""

    def __init__(self, device, tokens, layers=12, hidden=768, ffn=3072, seed=0, qkv_fused=True):
        import torch
        rng = np.random.default_rng(seed)
        self.tokens, self.hidden, self.ffn, self.qkv_fused = tokens, hidden, ffn, qkv_fused
        self.layers = []
        for _ in range(layers):
            layer = {}
            if qkv_fused:
                layer["qkv"] = QLinear(rng, hidden, 3 * hidden, device)
            else:
                for name in ("q", "k", "v"):
                    layer[name] = QLinear(rng, hidden, hidden, device)
            layer["o"] = QLinear(rng, hidden, hidden, device)
            layer["ffn1"] = QLinear(rng, hidden, ffn, device, act="gelu_erf")
            layer["ffn2"] = QLinear(rng, ffn, hidden, device, act_scale=0.01)
            self.layers.append(layer)
        t = tokens
        f16 = dict(dtype=torch.float16, device=device)
        self.xq = torch.randint(-127, 128, (t, hidden), dtype=torch.int8, device=device)
        self.cq = torch.randint(-127, 128, (t, hidden), dtype=torch.int8, device=device)
        self.hq = torch.empty((t, ffn), dtype=torch.int8, device=device)
        self.qkv = torch.empty((t, 3 * hidden), **f16)
        self.h = torch.empty((t, ffn), **f16)  # FFN1's un-quantised result: described, never written
        self.res = torch.randn((t, hidden), **f16)
        self.o = torch.empty((t, hidden), **f16)
        self.y = torch.empty((t, hidden), **f16)

    def ops_per_step(self):
        return sum(l.ops(self.tokens) for layer in self.layers for l in layer.values())

    def gemms_per_step(self):
        return sum(len(layer) for layer in self.layers)

    def distinct_shapes(self):
        t, h, f = self.tokens, self.hidden, self.ffn
        return [(t, 3 * h if self.qkv_fused else h, h, "f16", None), (t, f, h, "f16", "gelu_erf"),
                (t, h, f, "f16", None)]

    def _gemm(self, xq, lin, out, residual=None, q_out=None, q_scale=None, write_d=True):
        # half_math: the program is an fp16 model (the convert to half follows dequantizelinear
        # directly), so the lowering asks for every epilogue operator's half rounding
        capi.qgemm(xq, lin.w, b_layout=capi.B_NK, scale=lin.scale, scale_mode=capi.SCALE_PER_COL,
                   bias=lin.bias, act=lin.act, residual=residual, out=out, q_out=q_out,
                   q_scale=q_scale, write_d=write_d, half_math=True)

    def step(self):
        h = self.hidden
        for layer in self.layers:
            if self.qkv_fused:
                self._gemm(self.xq, layer["qkv"], self.qkv)
            else:
                for i, name in enumerate(("q", "k", "v")):
                    self._gemm(self.xq, layer[name], self.qkv[:, i * h:(i + 1) * h])
            self._gemm(self.cq, layer["o"], self.o, residual=self.res)
            self._gemm(self.xq, layer["ffn1"], self.h, q_out=self.hq, q_scale=0.03, write_d=False)
            self._gemm(self.hq, layer["ffn2"], self.y, residual=self.res)
        return self.y
