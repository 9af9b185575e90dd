"""The decoder's cache / rotary / decode-attention kernels through the C ABI against numpy
restatements of the reference operators (oracle/mgx_oracle.py)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import mgx_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from amdmigraphx_b200 import capi
    capi.load()
    return torch.device("cuda:0")


@pytest.mark.parametrize("batch,kvh,seq,head,cache,dtype", [(2, 2, 1, 32, 48, np.float16), (3, 1, 1, 128, 333, np.float16),
                                                           (1, 4, 16, 64, 64, np.float16), (2, 3, 1, 20, 50, np.float32),
                                                           (2, 2, 5, 7, 31, np.int8)])
def test_concat_past_present(cuda_device, batch, kvh, seq, head, cache, dtype):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(batch * 100 + head)
    mk = (lambda shp: rng.integers(-100, 100, size=shp).astype(dtype)) if dtype == np.int8 else \
        (lambda shp: rng.normal(size=shp).astype(dtype))
    past = mk((batch, kvh, cache, head))
    # the new rows as a slice of a packed QKV tensor (strided along the heads)
    packed = mk((batch, kvh + 3, seq, head))
    present = packed[:, 2:2 + kvh]
    lens = rng.integers(0, cache - seq, size=(batch, 1)).astype(np.int32)
    dp = torch.from_numpy(packed).to(cuda_device)[:, 2:2 + kvh]
    dpast = torch.from_numpy(past).to(cuda_device)
    for lt in (np.int32, np.int64):
        got = capi.concat_past_present(dp, torch.from_numpy(lens.astype(lt)).to(cuda_device), dpast.clone())
        np.testing.assert_array_equal(got.cpu().numpy(), O.concat_past_present(present, lens, past))


@pytest.mark.parametrize("batch,heads,kvh,seq,head,interleaved", [(2, 4, 2, 1, 32, False), (1, 8, 1, 16, 128, False),
                                                                 (2, 2, 2, 1, 64, True), (1, 4, 4, 9, 64, True)])
def test_gqa_rotary_embedding(cuda_device, batch, heads, kvh, seq, head, interleaved):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(heads * 10 + seq)
    max_seq = 64
    qkv = rng.normal(size=(batch, heads + 2 * kvh, seq, head)).astype(np.float16)
    ang = np.arange(max_seq)[:, None] * (10000.0 ** (-2.0 * np.arange(head // 2) / head))[None, :]
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    lens = rng.integers(0, max_seq, size=(batch, 1)).astype(np.int32)
    got = capi.gqa_rotary_embedding(torch.from_numpy(qkv).to(cuda_device), torch.from_numpy(lens).to(cuda_device),
                                    torch.from_numpy(cos).to(cuda_device), torch.from_numpy(sin).to(cuda_device),
                                    heads, kvh, interleaved)
    ref = O.gqa_rotary_embedding(qkv, lens, cos, sin, heads, kvh, interleaved)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("batch,heads,kvh,head,cache", [(1, 32, 32, 128, 2048), (16, 8, 1, 128, 4096), (3, 8, 2, 64, 200),
                                                        (2, 4, 2, 128, 333), (2, 8, 1, 64, 1100), (5, 4, 4, 64, 65),
                                                        (300, 2, 1, 64, 130), (2, 8, 2, 128, 300), (1, 64, 8, 128, 515)])
def test_gqa_decode_attention_matches_chain(cuda_device, batch, heads, kvh, head, cache):
    import torch
    from amdmigraphx_b200 import capi
    assert capi.gqa_decode_supported(batch, heads, kvh, head, cache)
    rng = np.random.default_rng(batch * 7 + cache)
    # queries as a slice of the packed rotary output [batch, heads + 2 kv_heads, 1, head]
    packed = rng.normal(size=(batch, heads + 2 * kvh, head)).astype(np.float16)
    kc = rng.normal(size=(batch, kvh, cache, head)).astype(np.float16)
    vc = rng.normal(size=(batch, kvh, cache, head)).astype(np.float16)
    lens = rng.integers(0, cache, size=(batch, 1)).astype(np.int32)
    lens[0, 0] = cache - 1  # a full cache
    if batch > 1:
        lens[1, 0] = 0      # a single position
    scale = float(np.float16(1.0 / np.sqrt(head)))
    dq = torch.from_numpy(packed).to(cuda_device)[:, :heads]
    got = capi.gqa_decode_attention(dq, torch.from_numpy(kc).to(cuda_device), torch.from_numpy(vc).to(cuda_device),
                                    torch.from_numpy(lens).to(cuda_device), scale)
    torch.cuda.synchronize()
    sel = list(range(batch)) if batch <= 16 else [0, 1, batch // 2, batch - 1]
    ref = O.gqa_decode_chain(packed[sel][:, :heads], kc[sel], vc[sel], lens[sel], scale)
    g = got.cpu().numpy()[sel]
    # the north-star tolerance of fp16 results ...
    np.testing.assert_allclose(g.astype(np.float32), ref.astype(np.float32), rtol=2e-2, atol=1e-2)
    # ... and nearly every half the reference's bit for bit (the rest: neighbouring halves, from the
    # order of the fp32 sums and the last bit of exp)
    differ = int((g.view(np.uint16) != ref.view(np.uint16)).sum())
    assert differ <= 0.03 * ref.size, (differ, ref.size)
    err = np.sqrt(((g.astype(np.float64) - ref.astype(np.float64)) ** 2).sum())
    assert err <= 3e-4 * np.sqrt((ref.astype(np.float64) ** 2).sum())


def test_gqa_decode_attention_rejects_what_it_has_no_kernel_for(cuda_device):
    import torch
    from amdmigraphx_b200 import capi
    assert not capi.gqa_decode_supported(1, 32, 32, 96, 2048)     # head size
    assert not capi.gqa_decode_supported(1, 48, 16, 128, 2048)    # 3 query heads per KV head
    assert not capi.gqa_decode_supported(1, 8, 1, 128, 1 << 20)   # a CTA's share beyond shared memory
    q = torch.zeros((1, 32, 96), dtype=torch.float16, device=cuda_device)
    kc = torch.zeros((1, 32, 64, 96), dtype=torch.float16, device=cuda_device)
    lens = torch.zeros((1, 1), dtype=torch.int32, device=cuda_device)
    with pytest.raises(RuntimeError):
        capi.gqa_decode_attention(q, kc, kc, lens, 0.1)


@pytest.mark.parametrize("batch,heads,seq,head", [(2, 6, 1, 64), (1, 40, 1, 128), (1, 3, 9, 32), (16, 9, 1, 128)])
def test_rotary_embedding_builder_form(cuda_device, batch, heads, seq, head):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(heads * 3 + seq)
    max_pos = 96
    # x as a slice of a transposed packed QKV tensor: strided along batch / head / row
    packed = rng.normal(size=(batch, seq, heads + 2, head)).astype(np.float16)
    x = packed.transpose(0, 2, 1, 3)[:, :heads]
    ang = np.arange(max_pos)[:, None] * (10000.0 ** (-2.0 * np.arange(head // 2) / head))[None, :]
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    pos = rng.integers(0, max_pos, size=(batch, seq)).astype(np.int32)
    dx = torch.from_numpy(packed).to(cuda_device).permute(0, 2, 1, 3)[:, :heads]
    for pt in (np.int32, np.int64):
        got = capi.rotary_embedding(dx, torch.from_numpy(pos.astype(pt)).to(cuda_device),
                                    torch.from_numpy(cos).to(cuda_device), torch.from_numpy(sin).to(cuda_device))
        ref = O.rotary_builder_chain(x, pos, cos, sin)
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("rows,cols", [(1, 4096), (16, 4096), (5, 256), (33, 1000)])
def test_rmsnorm_matches_parser_chain(cuda_device, rows, cols):
    import torch
    from amdmigraphx_b200 import capi
    rng = np.random.default_rng(rows + cols)
    x = (rng.normal(size=(rows, cols)) * rng.uniform(0.1, 4.0, size=(rows, 1))).astype(np.float16)
    g = rng.uniform(0.5, 1.5, size=cols).astype(np.float16)
    y, _ = capi.layernorm(torch.from_numpy(x).to(cuda_device), torch.from_numpy(g).to(cuda_device), None, eps=1e-5,
                          rms=True)
    ref = O.rmsnorm_chain(x, g, 1e-5)
    got = y.cpu().numpy()
    # the mean of squares is a tree of fp32 partial sums here and a double sum in the reference: where
    # they land in different halves a whole row moves by one half step
    np.testing.assert_allclose(got.astype(np.float32), ref.astype(np.float32), rtol=2e-3, atol=1e-6)
    same_rows = (got.view(np.uint16) == ref.view(np.uint16)).all(axis=1).mean()
    assert same_rows >= 0.8
