"""GPU tests of the fused LayerNorm and attention kernels through the C ABI against the CPU
restatement of the instruction chains they stand in for (oracle/mgx_oracle.py: layernorm_chain,
attention_chain - every operator of the chain rounding to the tensor type like MIGraphX's ref
target).  fp32 LayerNorm: rtol 1e-5 (fp32 tree sums against double); fp16: the fp16 tolerance of
this repository's tests, rtol 2e-2 / atol 1e-2, and far tighter in practice."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,dtype", [(384, 768, np.float16), (100, 768, np.float32), (33, 1024, np.float16),
                                             (7, 8, np.float16), (64, 3072, np.float16), (5, 2048, np.float32),
                                             (3072, 768, np.float16)])
def test_layernorm_matches_chain(cuda_device, rows, cols, dtype):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(rows + cols)
    x = (rng.normal(0.3, 1.5, size=(rows, cols))).astype(dtype)
    g = rng.uniform(0.5, 1.5, size=cols).astype(dtype)
    b = rng.normal(0, 0.2, size=cols).astype(dtype)
    eps = float(np.float32(O.half_trunc(np.float64(1e-5)))) if dtype == np.float16 else 1e-5
    t = lambda a: torch.from_numpy(a).to(cuda_device)  # noqa: E731
    y, q = capi.layernorm(t(x), t(g), t(b), eps=eps, q_scale=float(np.float16(0.04)))
    torch.cuda.synchronize()
    ref = O.layernorm_chain(x, g, b, eps)
    got = y.cpu().numpy()
    if dtype == np.float32:
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=2e-5)
    else:
        np.testing.assert_allclose(got.astype(np.float32), ref.astype(np.float32), rtol=2e-2, atol=1e-2)
        # the sums' order is the only difference: almost every element is bit-identical
        assert np.mean(got.view(np.uint16) != ref.view(np.uint16)) < 0.02
    # the fused quantizelinear is the operator applied to the kernel's own y: bit-exact
    q_ref = O.quantizelinear(got, np.array([0.04], dtype=dtype).astype(np.float16).astype(dtype), None, "int8")
    np.testing.assert_array_equal(q.cpu().numpy(), q_ref)


def test_layernorm_only_quantised_output_and_no_affine(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(9)
    x = rng.normal(0, 1, size=(50, 768)).astype(np.float16)
    xd = torch.from_numpy(x).to(cuda_device)
    y, _ = capi.layernorm(xd, None, None, eps=1e-5)
    y2, q, dq = capi.layernorm(xd, None, None, eps=1e-5, q_scale=0.03125, q_zero_point=3.0, write_y=False,
                               dq_scale=0.03125)
    torch.cuda.synchronize()
    assert y2 is None
    np.testing.assert_allclose(y.cpu().numpy().astype(np.float32),
                               O.layernorm_chain(x, None, None, 1e-5).astype(np.float32), rtol=2e-2, atol=1e-2)
    q_ref = O.quantizelinear(y.cpu().numpy(), np.array([0.03125], dtype=np.float16),
                             np.array([3], dtype=np.int8), "int8")
    np.testing.assert_array_equal(q.cpu().numpy(), q_ref)
    # the third result is dequantizelinear of the quantised tensor, bit for bit
    dq_ref = O.dequantizelinear(q_ref, np.array([0.03125], dtype=np.float16), np.array([3], dtype=np.int8))
    np.testing.assert_array_equal(dq.cpu().numpy().view(np.uint16), np.asarray(dq_ref, dtype=np.float16).view(np.uint16))


@pytest.mark.parametrize("batch,seq,heads", [(1, 384, 12), (2, 200, 4), (3, 64, 2), (1, 77, 1), (8, 384, 12),
                                             (1, 1024, 2), (1, 1100, 2)])
def test_attention_matches_chain(cuda_device, batch, seq, heads):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(batch * 1000 + seq)
    width = heads * 64
    # Q, K and V as column slices of one [rows, 3 * width] matrix (a fused QKV projection's output)
    qkv = rng.normal(0, 1.0, size=(batch * seq, 3 * width)).astype(np.float16)
    dq = torch.from_numpy(qkv).to(cuda_device)
    q, k, v = dq[:, :width], dq[:, width:2 * width], dq[:, 2 * width:]
    scale = 0.125
    o, oq = capi.attention(q, k, v, batch, seq, heads, scale, q_scale=float(np.float16(0.006)))
    torch.cuda.synchronize()
    if seq in (200, 384) and batch <= 2:
        # the fp32-softmax kernel on the same problem: the fp16 tolerance, not the chain's bits
        o2, _ = capi.attention(q, k, v, batch, seq, heads, scale, fp32_softmax=True)
        torch.cuda.synchronize()
        d = (o2.float() - o.float()).abs()
        assert float(d.max()) <= 1e-2 and float((d ** 2).mean().sqrt()) <= 2e-3 * float((o.float() ** 2).mean().sqrt())
    if batch * seq * seq * heads > 3e7:
        # the large case: check a sample of sequences and heads
        sel_b, sel_h = [0, batch - 1], [0, heads // 2, heads - 1]
    else:
        sel_b, sel_h = list(range(batch)), list(range(heads))
    got = o.cpu().numpy().reshape(batch, seq, heads, 64)
    err2, ref2, differ, total = 0.0, 0.0, 0, 0
    for b in sel_b:
        rows = slice(b * seq, (b + 1) * seq)
        for h in sel_h:
            cols = slice(h * 64, (h + 1) * 64)
            ref = O.attention_chain(qkv[rows, :width][:, cols], qkv[rows, width:2 * width][:, cols],
                                    qkv[rows, 2 * width:][:, cols], 1, seq, 1, scale)
            np.testing.assert_allclose(got[b, :, h, :].astype(np.float32), ref.astype(np.float32),
                                       rtol=2e-2, atol=1e-2)
            err2 += float(((got[b, :, h, :].astype(np.float64) - ref.astype(np.float64)) ** 2).sum())
            ref2 += float((ref.astype(np.float64) ** 2).sum())
            differ += int((np.ascontiguousarray(got[b, :, h, :]).view(np.uint16) != ref.view(np.uint16)).sum())
            total += ref.size
    # the results are averages of the values (small numbers): beyond the element-wise tolerance, the
    # error must be small against their typical magnitude (the kernel keeps more precision than the
    # chain of half-rounding operators it stands in for)
    assert np.sqrt(err2) <= 2e-3 * np.sqrt(ref2), (np.sqrt(err2), np.sqrt(ref2))
    # the kernel makes the chain's own roundings: nearly every result is the reference's half bit
    # for bit (the rest: neighbouring halves, from the order of the fp32 sums and the last bit of exp)
    assert differ <= 0.03 * total, (differ, total)
    assert np.sqrt(err2) <= 2e-4 * np.sqrt(ref2), (np.sqrt(err2), np.sqrt(ref2))
    if seq <= 1024 and batch <= 2:
        # the three-pass form (what sequences beyond 1024 keys run) makes the same roundings
        o3, _ = capi.attention(q, k, v, batch, seq, heads, scale, three_pass=True)
        torch.cuda.synchronize()
        same = (o3.view(torch.int16) == o.view(torch.int16)).float().mean()
        assert float(same) >= 0.97
    q_ref = O.quantizelinear(o.cpu().numpy(), np.array([0.006], dtype=np.float16), None, "int8")
    np.testing.assert_array_equal(oq.cpu().numpy(), q_ref)
