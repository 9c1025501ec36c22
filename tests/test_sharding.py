"""Splitting a call across GPUs: slices are legal calls with unchanged causal edges.

The device kernel cannot run here, so the oracle stands in for it inside each slice; what is
tested is the host logic: partitions, re-based lengths, the two-process driver over `gloo`,
the optional output gather and the all-ranks failure report.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ascendflow_b200 import sharding as S
from oracle import sparse_mla_oracle as O


def small_problem(b=3, t=9, context=16, seed=11, ratio=2):
    policy = O.make_policy(b, t, h=2, d=4, page=4, ratio=ratio, max_seq=16, window=3, topk=4, blocks=4 * b)
    arrays, rows, _ = O.performance_inputs(policy, context, seed)
    return dict(arrays, **O.materialize_caches(policy, rows)), policy


def test_partition_covers_everything_once():
    for total in (0, 1, 7, 8, 384):
        for parts in (1, 2, 3, 8):
            ranges = S.partition(total, parts)
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1


def test_balanced_partition_follows_the_weights():
    weights = list(range(1, 65))  # triangular work, as in a full causal prefill
    ranges = S.balanced_token_partition(weights, 4)
    assert ranges[0][0] == 0 and ranges[-1][1] == 64
    loads = [sum(weights[a:b]) for a, b in ranges]
    assert max(loads) / (sum(weights) / 4) < 1.2
    assert ranges[0][1] - ranges[0][0] > ranges[-1][1] - ranges[-1][0]


@pytest.mark.parametrize("ratio", [1, 2])
@pytest.mark.parametrize("world", [2, 3])
def test_request_shards_keep_every_token_edge(world, ratio):
    data, policy = small_problem(ratio=ratio)
    whole = O.resolve_rows(data, policy)
    pieces = []
    for rank in range(world):
        shard, (t0, t1) = S.shard_by_request(data, rank, world, ratio)
        local = dict(policy, B=len(shard["seqused_ori_kv"]), T=t1 - t0)
        assert int(shard["cu_seqlens_q"][0]) == 0 and int(shard["cu_seqlens_q"][-1]) == t1 - t0
        pieces.append(O.resolve_rows(shard, local))
    assert np.array_equal(np.concatenate(pieces), whole)


@pytest.mark.parametrize("ratio", [1, 2])
def test_token_range_shards_keep_every_token_edge(ratio):
    data, policy = small_problem(b=2, t=10, context=15, ratio=ratio)
    whole = O.resolve_rows(data, policy)
    reference = O.oracle(data, policy)
    for t0, t1 in [(0, 3), (3, 5), (5, 10), (2, 9), (4, 4), (0, 10)]:
        shard, _ = S.shard_by_token_range(data, t0, t1, ratio)
        local = dict(policy, B=len(shard["seqused_ori_kv"]), T=t1 - t0)
        assert np.array_equal(O.resolve_rows(shard, local), whole[t0:t1]), (t0, t1)
        if t1 > t0:
            assert np.array_equal(O.oracle(shard, local), reference[t0:t1])


def test_more_ranks_than_requests_is_refused_for_request_mode():
    data, _ = small_problem(b=2, t=4)
    with pytest.raises(ValueError, match="more ranks than requests"):
        S.shard_by_request(data, 0, 3, 2)


# ---- two processes over gloo -------------------------------------------------------------------

def _free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _worker(rank, world, port, mode, fail_rank, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ascendflow_b200.multi_gpu import run_sharded

        data, policy = small_problem(b=4, t=12, context=16, seed=5)
        tensors = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in data.items()}
        tensors["attention_out"] = torch.full_like(tensors["q"], float("nan"))

        def compute(shard):
            if rank == fail_rank:
                raise ValueError("injected shard failure")
            local = dict(policy, B=int(shard["ori_block_table"].shape[0]), T=int(shard["q"].shape[0]))
            as_numpy = {k: v.numpy() for k, v in shard.items() if k != "attention_out"}
            shard["attention_out"].copy_(torch.from_numpy(O.oracle(as_numpy, local)))

        try:
            t0, t1 = run_sharded(tensors, 2, mode=mode, gather=True, compute=compute)
            expected = O.oracle(data, policy)
            results[rank] = ("ok", bool(np.array_equal(tensors["attention_out"].numpy(), expected)), (t0, t1))
        except RuntimeError as error:
            results[rank] = ("error", str(error), None)
    finally:
        dist.destroy_process_group()


def _launch(mode, fail_rank=-1, world=2):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), mode, fail_rank, results), nprocs=world, join=True)
    return dict(results)


@pytest.mark.parametrize("mode", ["request", "tokens"])
def test_two_ranks_compute_disjoint_slices_and_gather_the_whole_output(mode):
    results = _launch(mode)
    assert all(results[r][0] == "ok" and results[r][1] for r in range(2)), results
    assert results[0][2][1] == results[1][2][0] and results[0][2][0] == 0 and results[1][2][1] == 12


def test_a_failing_rank_makes_every_rank_raise_and_skips_the_gather():
    results = _launch("request", fail_rank=1)
    assert results[0][0] == "error" and "another rank" in results[0][1]
    assert results[1][0] == "error" and "this rank" in results[1][1]
    assert all("gather skipped" in results[r][1] for r in range(2))
