"""Tensor-parallel decode of the int4 weight-only linears of a Llama-2-70B-shaped layer
(hidden 8192, 64 query / 8 KV heads of 128, FFN 28672, group 128), one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29555 -m amdmigraphx_b200.tp_decode_bench --batch 16

QKV and gate/up are split by output columns, o_proj and down_proj by input rows with one
mgx_cuda_all_reduce (NCCL) after each; attention itself and the norms are not part of this
path.  Prints one JSON line: time per layer (max over ranks, CUDA events on the compute stream)
and the packed-weight bytes all ranks stream per second.
"""
import argparse
import json
import os


def main():
    import torch
    import torch.distributed as dist
    from amdmigraphx_b200 import capi

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--layers", type=int, default=3, help="distinct layers of weights cycled through")
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        ids = [capi.Communicator.make_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = capi.Communicator(ids[0], world, rank)
    hid, kv, ffn, group = 8192, 2048, 28672, 128
    # per-rank shapes (N, K): column split divides N, row split divides K
    shapes = [((hid + kv) // world, hid, False), (hid, hid // world, True),
              (2 * ffn // world, hid, False), (hid, ffn // world, True)]
    gen = torch.Generator(device=dev)
    gen.manual_seed(1 + rank)
    layers = []
    for _ in range(a.layers):
        layers.append([(torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=gen),
                        (torch.rand(n, k // group, device=dev, generator=gen) * 0.015 + 0.005).half(),
                        reduce) for (n, k, reduce) in shapes])
    xs = {k: torch.randn(a.batch, k, device=dev, dtype=torch.float16) for (_, k, _) in shapes}
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    wbytes = sum(n * k // 2 + n * (k // group) * 2 for (n, k, _) in shapes)

    def one_layer(lw):
        for (bp, sc, reduce) in lw:
            y = capi.w4a16(xs[bp.shape[1] * 2], bp, sc, group=group, workspace=ws)
            if reduce and comm is not None:
                comm.all_reduce_(y)

    for i in range(3):
        one_layer(layers[i % a.layers])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.reps):
        one_layer(layers[i % a.layers])
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / a.reps * 1e3
    status = capi.device_status()
    if world > 1:
        t = torch.tensor([us], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item())
    if rank == 0:
        print(json.dumps({"workload": "llama-2-70b-shaped int4 decode linears, tensor parallel",
                          "n_gpus": world, "batch": a.batch, "us_per_layer": us,
                          "weight_gbs_all_ranks": world * wbytes / us / 1e3,
                          "tokens_per_s_linears_only_80_layers": a.batch / (80 * us * 1e-6),
                          "device_status": status}), flush=True)
    if comm is not None:
        comm.destroy()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
