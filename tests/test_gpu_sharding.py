"""Slices of a call on a real GPU: the pieces reproduce the whole call bit for bit.

The CPU suite proves the slicing arithmetic against the oracle with a stand-in compute step;
here the CUDA operator runs the slices: two token ranges of a prefill call, the requests of a
decode call, and `run_sharded` itself in a single-rank process group.
"""

import os
import socket

import pytest

pytestmark = pytest.mark.gpu

ORDER = ("q", "ori_kv", "cmp_kv", "cmp_sparse_indices", "ori_block_table", "cmp_block_table", "cu_seqlens_q",
         "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length", "sinks", "attention_out")


def whole_and_reference(config, seed):
    import torch

    from ascendflow_b200 import ops, workloads as W

    tensors, meta, work = W.device_case(**config, seed=seed)
    ops.sparse_mla(*(tensors[name] for name in ORDER))
    torch.cuda.synchronize()
    expected = tensors["attention_out"].clone()
    tensors["attention_out"].fill_(float("nan"))
    return tensors, expected


def run_slice(shard):
    from ascendflow_b200 import ops

    ops.sparse_mla(*(shard[name] for name in ORDER))


@pytest.mark.parametrize("cut", [1, 777, 2048])
def test_two_token_ranges_of_a_prefill_call(cut):
    import torch

    from ascendflow_b200 import sharding

    config = dict(batches=1, queries=2048 + 64, context=8192, max_seq=8192)
    tensors, expected = whole_and_reference(config, seed=5)
    total = config["queries"]
    for t0, t1 in ((0, cut), (cut, total)):
        shard, _ = sharding.shard_by_token_range(tensors, t0, t1, 2)
        run_slice(shard)
    torch.cuda.synchronize()
    assert torch.equal(tensors["attention_out"].view(torch.int16), expected.view(torch.int16))


def test_request_shards_of_a_decode_call():
    import torch

    from ascendflow_b200 import multi_gpu

    config = dict(batches=12, queries=6, context=16384, max_seq=16384)
    tensors, expected = whole_and_reference(config, seed=6)
    for rank in range(5):  # uneven: 12 requests over 5 ranks
        shard, (t0, t1) = multi_gpu.shard_for_rank(tensors, rank, 5, 2, mode="request")
        assert t1 > t0
        run_slice(shard)
    torch.cuda.synchronize()
    assert torch.equal(tensors["attention_out"].view(torch.int16), expected.view(torch.int16))


def test_balanced_ranges_of_a_full_causal_prefill():
    """Early tokens of a full-causal call attend to fewer rows: ranges of equal work, not equal length."""
    import numpy as np
    import torch

    from ascendflow_b200 import multi_gpu

    config = dict(batches=1, queries=1536, context=1536, max_seq=2048)
    tensors, expected = whole_and_reference(config, seed=7)
    right = np.arange(1536) + 1
    weights = (np.minimum(128, right) + np.minimum(512, right // 2)).tolist()
    covered = 0
    for rank in range(4):
        shard, (t0, t1) = multi_gpu.shard_for_rank(tensors, rank, 4, 2, mode="tokens", weights=weights)
        assert t0 == covered
        covered = t1
        run_slice(shard)
    assert covered == 1536
    torch.cuda.synchronize()
    assert torch.equal(tensors["attention_out"].view(torch.int16), expected.view(torch.int16))


def test_run_sharded_in_a_single_rank_group():
    import torch
    import torch.distributed as dist

    from ascendflow_b200 import multi_gpu

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        config = dict(batches=3, queries=40, context=4096, max_seq=4096)
        tensors, expected = whole_and_reference(config, seed=8)
        # gloo reduces the failure flag on the host; the operator runs on the GPU
        group = dist.group.WORLD
        flag_device = tensors["attention_out"].device
        assert flag_device.type == "cuda"
        t0, t1 = multi_gpu.run_sharded(tensors, 2, mode="request", gather=False, group=group, flag_device="cpu")
        torch.cuda.synchronize()
        assert (t0, t1) == (0, 120)
        assert torch.equal(tensors["attention_out"].view(torch.int16), expected.view(torch.int16))
    finally:
        dist.destroy_process_group()
