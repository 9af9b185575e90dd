"""GPU test: every QDQ linear of the BERT-base-shaped int8 stack (real shapes, batch 1 x 384
tokens) against the CPU oracle, and the stack's launch bookkeeping."""
import numpy as np
import pytest

from oracle import mgx_oracle as O

pytestmark = pytest.mark.gpu


def _oracle_linear(x16, lin, residual=None):
    xq = O.quantizelinear(x16, lin.x_scale_host.astype(np.float16), None, "int8")
    acc = O.quant_dot_int8(xq, lin.w_nk_host.T)
    return O.qlinear_epilogue(acc, lin.scale_host[None, :], lin.bias_host, lin.act, residual,
                              np.float16)


@pytest.mark.parametrize("fused", [False, True])
def test_bert_layer_linears_match_oracle(cuda_device, fused):
    import torch
    from amdmigraphx_b200.workloads import BertInt8LinearStack
    stack = BertInt8LinearStack(cuda_device, layers=1, tokens=384, seed=3, fuse_quant=fused)
    stack.prepare()
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, size=(384, 768)).astype(np.float16)
    stack.x.copy_(torch.from_numpy(x))
    y = stack.step().cpu().numpy()
    layer = stack.layers[0]
    qkv = _oracle_linear(x, layer["qkv"])
    got_qkv = stack.qkv.cpu().numpy()
    np.testing.assert_array_equal(got_qkv, qkv)  # int8 path with fp16 out: identical bits
    o = _oracle_linear(np.ascontiguousarray(qkv[:, :768]), layer["o"], residual=x)
    np.testing.assert_array_equal(stack.o.cpu().numpy(), o)
    if fused:
        # O-proj's epilogue also wrote quantizelinear(o) for FFN1: identical to the operator
        oq = O.quantizelinear(o, layer["ffn1"].x_scale_host.astype(np.float16), None, "int8")
        np.testing.assert_array_equal(stack.oq.cpu().numpy(), oq)
    h = _oracle_linear(o, layer["ffn1"])
    if fused:
        # only the quantised GELU output exists; the fast erf may move a value across a
        # rounding boundary: at most one quantisation step, and rarely
        hq_ref = O.quantizelinear(h, layer["ffn2"].x_scale_host.astype(np.float16), None, "int8")
        got_hq = stack.hq.cpu().numpy()
        diff = np.abs(got_hq.astype(np.int32) - hq_ref.astype(np.int32))
        assert diff.max() <= 1 and np.mean(diff != 0) < 1e-3
        acc = O.quant_dot_int8(got_hq, layer["ffn2"].w_nk_host.T)
        y_ref = O.qlinear_epilogue(acc, layer["ffn2"].scale_host[None, :], layer["ffn2"].bias_host,
                                   None, o, np.float16)
        np.testing.assert_array_equal(y, y_ref)
        assert stack.launches_per_step() == 6
    else:
        got_h = stack.h.cpu().numpy()
        np.testing.assert_allclose(got_h.astype(np.float32), h.astype(np.float32), rtol=2e-2, atol=1e-2)
        # the GELU output feeds the next quantizelinear: compare the last linear on the GPU's own h
        y_ref = _oracle_linear(got_h, layer["ffn2"], residual=o)
        np.testing.assert_array_equal(y, y_ref)
        assert stack.launches_per_step() == 8
    assert stack.ops_per_step() == 2 * 384 * (768 * 2304 + 768 * 768 + 2 * 768 * 3072)
