"""The steps next to the operator: top-k index selection and cache append.

CPU: the oracle's definitions on hand-sized cases, and that what the selection produces is what
the operator's row selection accepts in full. GPU: the CUDA kernels against the oracle, bit for
bit (int32 indices, cache bytes), through the C ABI.
"""

import numpy as np
import pytest

from oracle import sparse_mla_oracle as O


def small(b=2, t=6, lengths=(40, 9), ratio=2):
    policy = O.make_policy(b, t, h=2, d=8, page=8, ratio=ratio, max_seq=64, window=4, topk=4, blocks=16)
    counts = O.query_counts(policy)
    lengths = np.asarray(lengths, dtype=np.int32)
    data = {
        "cu_seqlens_q": np.concatenate([[0], np.cumsum(counts)]).astype(np.int32),
        "seqused_ori_kv": lengths,
        "seqused_cmp_kv": (lengths // ratio).astype(np.int32),
        "cmp_residual_kv": (lengths % ratio).astype(np.int32),
    }
    return policy, data


def test_selection_takes_the_highest_scores_lowest_index_first_on_ties():
    policy, data = small()
    scores = np.zeros((6, 32), dtype=np.float32)
    scores[0, [3, 7, 11, 15, 16]] = [5, 4, 4, 4, 4]     # four of five: the tie at 4 is cut by index
    picked = O.select_topk_indices(scores, data, policy)
    geometry = O.token_geometry(dict(data, ori_topk_length=np.zeros((6, 1), np.int32)), policy)
    assert picked[0, 0].tolist() == [3, 7, 11, 15]
    # request 1 holds 9 rows and 3 queries: token 3 sees (9 - 3 + 0 + 1) // 2 = 3 compressed rows
    assert geometry["cutoff"][3] == 3 and picked[3, 0].tolist() == [0, 1, 2, -1]
    # all scores equal: the first TOPK visible rows
    assert picked[1, 0].tolist() == [0, 1, 2, 3]


def test_selection_is_accepted_in_full_by_the_operators_row_selection():
    rng = np.random.default_rng(5)
    policy = O.make_policy(3, 30, max_seq=4096, blocks=96)
    data = O.validation_inputs(policy, "mixed")
    scores = rng.normal(size=(30, 2048)).astype(np.float32)
    data["cmp_sparse_indices"] = O.select_topk_indices(scores, data, policy)
    resolved = O.resolve_rows(data, policy)
    geometry = O.token_geometry(data, policy)
    for token in range(30):
        listed = data["cmp_sparse_indices"][token, 0]
        live = listed[listed >= 0]
        assert len(live) == min(512, geometry["available"][token], geometry["cutoff"][token])
        assert (np.diff(live) > 0).all()
        assert (resolved[token, 128:128 + len(live)] >= 0).all() and (resolved[token, 128 + len(live):] < 0).all()


def test_append_puts_rows_where_the_window_looks_for_them():
    policy, data = small()
    rng = np.random.default_rng(2)
    cache = rng.normal(size=(16, 8, 1, 8)).astype(np.float32)
    table = np.stack([rng.permutation(8), rng.permutation(8) + 8]).astype(np.int32)
    new = rng.normal(size=(6, 8)).astype(np.float32)
    after = O.append_rows(cache, new, table, data["cu_seqlens_q"], data["seqused_ori_kv"])
    # token 5 is the last of request 1 (length 9): position 8 = page table[1][1], row 0
    assert np.array_equal(after[table[1, 1], 0, 0], new[5])
    assert np.array_equal(after[table[0, 4], 7, 0], new[2])          # request 0: positions 37, 38, 39
    changed = (after != cache).any(axis=(2, 3)).sum()
    assert changed == 6


@pytest.mark.gpu
@pytest.mark.parametrize("ratio,seed", [(2, 0), (2, 1), (1, 2)])
def test_gpu_selection_matches_the_oracle_bit_for_bit(ratio, seed):
    import torch

    from ascendflow_b200 import neighbours

    rng = np.random.default_rng(40 + seed)
    lens = [int(v) for v in rng.integers(0, 40, 5)]
    lens[0] = max(lens[0], 3)
    policy = O.make_policy(len(lens), sum(lens), ratio=ratio, max_seq=8192, blocks=8)
    lengths = np.array([int(rng.integers(max(n, 1), 8193)) for n in lens], dtype=np.int32)
    lengths[1] = max(lens[1], 1)                      # a cache that holds only its queries
    data = {
        "cu_seqlens_q": np.concatenate([[0], np.cumsum(lens)]).astype(np.int32),
        "seqused_ori_kv": lengths,
        "seqused_cmp_kv": (lengths // ratio).astype(np.int32),
        "cmp_residual_kv": (lengths % ratio).astype(np.int32),
    }
    span = 8192 // ratio
    scores = rng.normal(size=(sum(lens), span)).astype(np.float32)
    scores[::3] = np.round(scores[::3] * 2) / 2       # plenty of exact ties
    scores[5] = 1.25                                  # one token with nothing but ties
    expected = O.select_topk_indices(scores, data, policy)
    device = {k: torch.from_numpy(v).cuda() for k, v in data.items()}
    actual = neighbours.topk_indices(torch.from_numpy(scores).cuda(), device["cu_seqlens_q"], device["seqused_cmp_kv"],
                                     device["cmp_residual_kv"], ratio=ratio)
    assert np.array_equal(actual.cpu().numpy(), expected)


@pytest.mark.gpu
@pytest.mark.parametrize("max_seq,ratio", [(131072, 2), (32768, 2), (131072, 1), (262144, 2)])
def test_gpu_selection_over_long_rows(max_seq, ratio):
    """Decode-sized rows: up to 65536 scores are selected from one read (upper key halves kept in
    shared memory), longer rows by the streaming kernel. Continuous scores, heavy ties, one row of
    nothing but ties (more of them than the kernel's tie list holds), one of negative values."""
    import torch

    from ascendflow_b200 import neighbours

    rng = np.random.default_rng(max_seq // 1024 + ratio)
    lens = [2, 1, 3, 2]
    span = max_seq // ratio
    policy = O.make_policy(len(lens), sum(lens), ratio=ratio, max_seq=max_seq, blocks=8)
    lengths = np.array([max_seq, max_seq - 5, 4100, 700], dtype=np.int32)   # long, long, short, under TopK
    data = {
        "cu_seqlens_q": np.concatenate([[0], np.cumsum(lens)]).astype(np.int32),
        "seqused_ori_kv": lengths,
        "seqused_cmp_kv": (lengths // ratio).astype(np.int32),
        "cmp_residual_kv": (lengths % ratio).astype(np.int32),
    }
    scores = rng.normal(size=(sum(lens), span)).astype(np.float32)
    scores[1] = np.round(scores[1] * 4) / 4           # a few dozen distinct values: long runs of ties
    scores[2] = -3.5                                  # nothing but ties
    scores[3] = -np.abs(scores[3])                    # negative keys only
    scores[4, ::7] = np.float32(2.0)                  # a plateau that the threshold falls into
    expected = O.select_topk_indices(scores, data, policy)
    device = {k: torch.from_numpy(v).cuda() for k, v in data.items()}
    actual = neighbours.topk_indices(torch.from_numpy(scores).cuda(), device["cu_seqlens_q"], device["seqused_cmp_kv"],
                                     device["cmp_residual_kv"], ratio=ratio)
    assert np.array_equal(actual.cpu().numpy(), expected)


@pytest.mark.gpu
def test_gpu_selection_feeds_the_attention_call():
    """Scores -> indices on the device -> attention, against the oracle fed with the oracle's selection."""
    import torch

    from ascendflow_b200 import neighbours, ops
    from tests import support as S

    policy = O.make_policy(4, 16, max_seq=4096, blocks=128)
    data = O.validation_inputs(policy, "mixed")
    rng = np.random.default_rng(9)
    scores = rng.normal(size=(16, 2048)).astype(np.float32)
    data["cmp_sparse_indices"] = O.select_topk_indices(scores, data, policy)
    tensors, _ = S.to_device(data, policy)
    tensors["cmp_sparse_indices"] = neighbours.topk_indices(
        torch.from_numpy(scores).cuda(), tensors["cu_seqlens_q"], tensors["seqused_cmp_kv"], tensors["cmp_residual_kv"])
    assert np.array_equal(tensors["cmp_sparse_indices"].cpu().numpy(), data["cmp_sparse_indices"])
    ops.sparse_mla(*(tensors[name] for name in S.TENSOR_ORDER))
    S.assert_close(S.output_to_numpy(tensors["attention_out"], "bf16"), O.reference_fp32_from_data(data, policy), "selected on the device")


@pytest.mark.gpu
def test_gpu_append_matches_the_oracle_byte_for_byte():
    import torch

    from ascendflow_b200 import neighbours

    rng = np.random.default_rng(77)
    lens = [6, 0, 130, 1]
    lengths = np.array([700, 5, 130, 4096], dtype=np.int32)
    pages, blocks = 32, 4 * 32
    table = np.stack([rng.permutation(pages) + b * pages for b in range(4)]).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cache = rng.integers(0, 1 << 16, size=(blocks, 128, 1, 512), dtype=np.uint16)
    new = rng.integers(0, 1 << 16, size=(sum(lens), 512), dtype=np.uint16)
    expected = O.append_rows(cache, new, table, cu, lengths)
    as_bf16 = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    device_cache = as_bf16(cache)
    status = neighbours.cache_append(as_bf16(new), device_cache, torch.from_numpy(table).cuda(),
                                     torch.from_numpy(cu).cuda(), torch.from_numpy(lengths).cuda())
    assert status[0] == 0
    assert np.array_equal(device_cache.view(torch.int16).cpu().numpy().view(np.uint16), expected)
    # a length beyond the table: reported, nothing written there, the context stays usable
    bad = lengths.copy()
    bad[3] = pages * 128 + 1
    status = neighbours.cache_append(as_bf16(new), device_cache, torch.from_numpy(table).cuda(),
                                     torch.from_numpy(cu).cuda(), torch.from_numpy(bad).cuda())
    assert status[0] == 1 and status[1] == sum(lens) - 1
