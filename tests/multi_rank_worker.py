"""One rank of the two-GPU sharding test (started by tests/test_gpu_multi_rank.py under torchrun).

Every rank builds the same seeded call, computes the whole call alone (the single-GPU answer),
then runs `run_sharded` with the output all-gather over NCCL and compares bit for bit. One rank
raises on purpose in a third round, on the host and before anything is enqueued: all ranks must
raise together, before the gather.
"""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist

from ascendflow_b200 import multi_gpu, ops, workloads as W

ORDER = ("q", "ori_kv", "cmp_kv", "cmp_sparse_indices", "ori_block_table", "cmp_block_table", "cu_seqlens_q",
         "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length", "sinks", "attention_out")


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    for mode, config in (("request", dict(batches=6, queries=6, context=8192, max_seq=8192)),
                         ("tokens", dict(batches=1, queries=700, context=4096, max_seq=4096))):
        tensors, _, _ = W.device_case(**config, seed=31, device=device)
        ops.sparse_mla(*(tensors[name] for name in ORDER))
        torch.cuda.synchronize()
        expected = tensors["attention_out"].clone()
        tensors["attention_out"].zero_()
        t0, t1 = multi_gpu.run_sharded(tensors, 2, mode=mode, gather=True)
        torch.cuda.synchronize()
        assert t1 > t0
        assert torch.equal(tensors["attention_out"].view(torch.int16), expected.view(torch.int16)), (mode, rank)

    def failing(shard):
        if rank == 1:
            raise ValueError("rank 1 refuses")
        ops.sparse_mla(*(shard[name] for name in ORDER))

    try:
        multi_gpu.run_sharded(tensors, 2, mode="tokens", gather=True, compute=failing)
    except RuntimeError as error:
        assert "shard failed" in str(error), error
    else:
        raise AssertionError("a failing rank went unnoticed")
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("multi-rank sharding ok")


if __name__ == "__main__":
    main()
