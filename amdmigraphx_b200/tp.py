"""Tensor-parallel sharding of the int4 weight-only linears (config 5: Llama-2-70B-shaped
decoder, 2/4/8 ranks).  Megatron layout: q/k/v/gate/up are split by output columns (each rank
keeps N/world rows of the packed [N, K/2] weight), o/down by input rows (each rank keeps
K/world of every weight row, i.e. a column slice of the packed matrix and of the scales) and
their partial results are summed with one all-reduce.  Pure index arithmetic on numpy arrays
or torch tensors; the exchange itself is mgx_cuda_all_reduce (capi.Communicator).
"""


def shard_columns(bp, scales, zp, rank, world):
    """Output-column split: rows [rank*N/world, (rank+1)*N/world) of the packed weight."""
    n = bp.shape[0]
    if n % world != 0:
        raise ValueError("N must be divisible by the number of ranks")
    lo, hi = rank * n // world, (rank + 1) * n // world
    return bp[lo:hi], scales[lo:hi], None if zp is None else zp[lo:hi]


def shard_rows(bp, scales, zp, rank, world, group):
    """Input-row (K) split: k in [rank*K/world, (rank+1)*K/world) of every weight row.  The
    slice must cover whole quantisation groups so that scales split the same way."""
    k = bp.shape[1] * 2
    if k % world != 0 or (k // world) % group != 0:
        raise ValueError("K / world must be a multiple of the group size")
    klo, khi = rank * k // world, (rank + 1) * k // world
    glo, ghi = klo // group, khi // group
    return (bp[:, klo // 2:khi // 2], scales[:, glo:ghi], None if zp is None else zp[:, glo:ghi])


def shard_activation(x, rank, world):
    """The slice of the activation a row-split linear consumes on this rank."""
    k = x.shape[-1]
    return x[..., rank * k // world:(rank + 1) * k // world]
