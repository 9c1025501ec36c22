"""One call of the operator spread over the GPUs of a node, one process per GPU.

Each rank takes a slice of the call along a natural axis (whole requests, or a query-token
range), runs the single-GPU operator on it, and writes into its slice of `attention_out`.
Nothing is exchanged on the data path. Only if the caller wants the whole output on every
rank is there one collective afterwards (`torch.distributed.all_gather`, NCCL on GPUs).

A rank whose slice fails does not leave the others waiting: every rank contributes a failure
flag to one small all-reduce before the optional gather, and all ranks raise together.
"""

from __future__ import annotations

from .diagnostics import require
from .sharding import partition, shard_by_request, shard_by_token_range


def shard_for_rank(tensors, rank, world, ratio, mode="auto", weights=None):
    """This rank's slice of a call and the token range `(t0, t1)` it covers."""
    batches = int(tensors["ori_block_table"].shape[0])
    tokens = int(tensors["q"].shape[0])
    if mode == "auto":
        mode = "request" if batches >= world else "tokens"
    require(mode in ("request", "tokens"), "shard mode must be 'request', 'tokens' or 'auto'")
    if mode == "request":
        return shard_by_request(tensors, rank, world, ratio)
    if weights is not None:
        from .sharding import balanced_token_partition

        t0, t1 = balanced_token_partition(weights, world)[rank]
    else:
        t0, t1 = partition(tokens, world)[rank]
    return shard_by_token_range(tensors, t0, t1, ratio)


def run_sharded(tensors, ratio=2, *, mode="auto", gather=False, compute=None, group=None, weights=None,
                flag_device=None):
    """Run this rank's slice; optionally replicate the full output on every rank.

    `tensors` maps the thirteen operator names to tensors holding the WHOLE call on every rank
    (read-only inputs may be replicated or be views of a larger buffer; `attention_out` is
    written only in this rank's token range unless `gather` is set). `compute(shard)` defaults to
    the CUDA operator. `flag_device` is where the one-word failure flag lives (default: the output's
    device; "cpu" for a host-side process group). Returns the token range this rank computed.
    """
    import torch
    import torch.distributed as dist

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    shard, (t0, t1) = shard_for_rank(tensors, rank, world, ratio, mode, weights)
    if compute is None:
        from .ops import sparse_mla

        def compute(call):
            sparse_mla(*(call[name] for name in (
                "q", "ori_kv", "cmp_kv", "cmp_sparse_indices", "ori_block_table", "cmp_block_table",
                "cu_seqlens_q", "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv",
                "ori_topk_length", "sinks", "attention_out")))

    failure = None
    try:
        if t1 > t0:
            compute(shard)
    except Exception as error:  # reported on every rank below
        failure = error
    out = tensors["attention_out"]
    flag = torch.tensor([0 if failure is None else 1], dtype=torch.int32,
                        device=out.device if flag_device is None else flag_device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    if int(flag.item()):
        raise RuntimeError(
            f"sparse_mla shard failed on {'this' if failure is not None else 'another'} rank "
            f"(rank {rank}); output gather skipped; device retries are disabled") from failure
    if gather:
        ranges = [shard_for_rank(tensors, r, world, ratio, mode, weights)[1] for r in range(world)]
        longest = max(b - a for a, b in ranges)
        mine = out.new_zeros((longest,) + tuple(out.shape[1:]))
        mine[: t1 - t0] = out[t0:t1]
        pieces = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(pieces, mine, group=group)
        for (a, b), piece in zip(ranges, pieces):
            out[a:b] = piece[: b - a]
    return t0, t1
