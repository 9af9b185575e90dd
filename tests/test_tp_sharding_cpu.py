"""CPU test (gloo, world size 2) of the tensor-parallel sharding used for the int4 decoder:
column-split gate/up, row-split down with a sum all-reduce of the partial results must
reproduce the unsharded linear (the oracle) within the fp16 tolerance."""
import os

import numpy as np
import pytest


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    from amdmigraphx_b200 import tp
    from oracle import mgx_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)  # same data on every rank
        M, H, F, g = 4, 256, 512, 128
        x = rng.normal(0, 1, size=(M, H)).astype(np.float16)
        up = (rng.integers(0, 256, size=(F, H // 2), dtype=np.uint8),
              rng.uniform(0.005, 0.02, size=(F, H // g)).astype(np.float16))
        down = (rng.integers(0, 256, size=(H, F // 2), dtype=np.uint8),
                rng.uniform(0.005, 0.02, size=(H, F // g)).astype(np.float16))
        # unsharded reference
        h_full = O.w4a16_linear(x, up[0], up[1], None, 8, g)
        y_full = O.w4a16_linear(h_full, down[0], down[1], None, 8, g).astype(np.float32)
        # this rank's shards
        ubp, usc, _ = tp.shard_columns(up[0], up[1], None, rank, world)
        h_local = O.w4a16_linear(x, ubp, usc, None, 8, g)           # [M, F/world]
        np.testing.assert_array_equal(h_local, tp.shard_activation(h_full, rank, world))
        dbp, dsc, _ = tp.shard_rows(down[0], down[1], None, rank, world, g)
        part = O.w4a16_linear(h_local, dbp, dsc, None, 8, g).astype(np.float32)
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        np.testing.assert_allclose(t.numpy(), y_full, rtol=2e-2, atol=1e-2)
        with pytest.raises(ValueError):
            tp.shard_rows(down[0], down[1], None, rank, 3, g)
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_column_then_row_split_matches_unsharded():
    import torch.multiprocessing as mp
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))
