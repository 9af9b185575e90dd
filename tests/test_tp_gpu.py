"""GPU test on 2 GPUs (skipped with fewer): tensor-parallel int4 MLP - column-split up
projection, row-split down projection, mgx_cuda_all_reduce over NCCL on the compute stream -
against the unsharded linear on the CPU oracle."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from amdmigraphx_b200 import capi, tp
    from oracle import mgx_oracle as O
    try:
        ids = [capi.Communicator.make_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = capi.Communicator(ids[0], world, rank)
        rng = np.random.default_rng(11)
        M, H, F, g = 16, 1024, 2048, 128
        x = rng.normal(0, 1, size=(M, H)).astype(np.float16)
        up = (rng.integers(0, 256, size=(F, H // 2), dtype=np.uint8),
              rng.uniform(0.005, 0.02, size=(F, H // g)).astype(np.float16))
        down = (rng.integers(0, 256, size=(H, F // 2), dtype=np.uint8),
                rng.uniform(0.005, 0.02, size=(H, F // g)).astype(np.float16))
        ubp, usc, _ = tp.shard_columns(up[0], up[1], None, rank, world)
        dbp, dsc, _ = tp.shard_rows(down[0], down[1], None, rank, world, g)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
        h = capi.w4a16(t(x), t(ubp), t(usc), group=g)
        y = capi.w4a16(h, t(dbp), t(dsc), group=g)
        comm.all_reduce_(y)
        torch.cuda.synchronize()
        assert capi.device_status() == 0
        # each linear against the unsharded oracle at the single-operator tolerance: the up
        # projection's shard against its columns, the down projection on the hidden tensor the
        # GPUs actually produced (gathered over the ranks)
        h_full = O.w4a16_linear(x, up[0], up[1], None, 8, g)
        cols = F // world
        np.testing.assert_allclose(h.cpu().numpy().astype(np.float32),
                                   h_full[:, rank * cols:(rank + 1) * cols].astype(np.float32), rtol=2e-2, atol=1e-2)
        parts = [None] * world
        dist.all_gather_object(parts, h.cpu().numpy())
        h_gpu = np.concatenate(parts, axis=1)
        y_full = O.w4a16_linear(h_gpu, down[0], down[1], None, 8, g).astype(np.float32)
        np.testing.assert_allclose(y.cpu().numpy().astype(np.float32), y_full, rtol=2e-2, atol=1e-2)
        comm.destroy()
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_int4_mlp(cuda_device):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    port = 29700 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def test_all_reduce_inside_a_compiled_program(cuda_device, tmp_path):
    """One process per GPU, each compiling ITS shard of a tensor-parallel int4 MLP - column-split up
    projection, row-split down projection, cuda::all_reduce as the last instruction - through
    make_target("cuda") -> program::compile -> program::eval; every rank's result against the
    unsharded MLP on MIGraphX's ref target (cuda_target_check run tp_int4_mlp)."""
    import json
    import subprocess
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "amdmigraphx_b200", "bin", "cuda_target_check")
    world = 2
    idfile = str(tmp_path / "nccl_id")
    procs = []
    for rank in range(world):
        env = dict(os.environ, MGX_TP_RANK=str(rank), MGX_TP_WORLD=str(world), MGX_TP_ID_FILE=idfile,
                   MIGRAPHX_CUDA_DEVICE=str(rank), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([exe, "run", "tp_int4_mlp"], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        try:
            out, err = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append((p.returncode, out, err))
    for rc, out, err in outs:
        lines = [l for l in out.splitlines() if l.startswith("{")]
        assert lines, out + err[-2000:]
        res = json.loads(lines[-1])
        assert res.get("pass"), res
