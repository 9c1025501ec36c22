"""Hand-sized known-answer cases for the oracle.

These restate the scenarios the reference pins in
`tests/operators/test_sparse_attention.py:14-129`: a one-token problem with
PAGE 4, RATIO 2, WINDOW 3, TOPK 4 whose caches hold small exact values, so the
expected rows and outputs can be written down by hand.
"""

import numpy as np
import pytest

from oracle import sparse_mla_oracle as O


@pytest.fixture
def tiny():
    policy = {
        "B": 1, "T": 1, "H": 2, "D": 4, "PAGE": 4, "RATIO": 2, "WINDOW": 3, "TOPK": 4, "S": 8,
        "DTYPE": "bf16", "SCALE": 0.5,
    }
    data = {
        "q": np.zeros((1, 2, 4), dtype=np.float32),
        "ori_kv": np.arange(32, dtype=np.float32).reshape(2, 4, 1, 4) / 16,
        "cmp_kv": np.arange(16, dtype=np.float32).reshape(2, 2, 1, 4) / 4,
        "ori_block_table": np.array([[1, 0]], dtype=np.int32),
        "cmp_block_table": np.array([[1, 0]], dtype=np.int32),
        "seqused_ori_kv": np.array([5], dtype=np.int32),
        "ori_topk_length": np.array([[2]], dtype=np.int32),
        "cu_seqlens_q": np.array([0, 1], dtype=np.int32),
        "seqused_cmp_kv": np.array([2], dtype=np.int32),
        "cmp_residual_kv": np.array([1], dtype=np.int32),
        "cmp_sparse_indices": np.array([[[1, 1, 2, -1]]], dtype=np.int32),
        "sinks": np.zeros(2, dtype=np.float32),
    }
    return data, policy


def test_page_crossing_duplicates_and_compression_causality(tiny):
    data, policy = tiny
    rows, slots = O.selected_rows(data, policy, 0)
    # Raw positions 3 and 4 straddle a page; index 1 is listed twice and kept twice;
    # index 2 is incomplete at raw length 5 with ratio 2.
    assert slots == [0, 1, 3, 4]
    expected = np.stack([
        data["ori_kv"][1, 3, 0], data["ori_kv"][0, 0, 0], data["cmp_kv"][1, 1, 0], data["cmp_kv"][1, 1, 0],
    ])
    assert np.array_equal(rows, expected)
    # Physical ids: raw page 1 row 3 -> 7, raw page 0 row 0 -> 0, compressed page 1 row 1 -> 3.
    assert O.resolve_rows(data, policy)[0].tolist() == [7, 0, -1, 3, 3, -1, -1, -1]
    kv, bias = O.gather_oracle(data, policy)
    assert np.array_equal(kv[0, slots], rows)
    assert np.all(kv[0, [2, 5, 6, 7]] == 0)
    assert np.isfinite(bias[0]).tolist() == [True, True, False, True, True, False, False, False]


def test_one_sink_in_one_shared_denominator(tiny):
    data, policy = tiny
    rows, _ = O.selected_rows(data, policy, 0)
    actual = O.oracle(data, policy)
    # q = 0 and sink = 0: four rows of weight one plus exactly one sink of weight one.
    expected = O.round_b16(np.broadcast_to(rows.sum(axis=0) / 5, (1, 2, 4)).copy(), "bf16")
    assert np.array_equal(actual, expected)
    data["cmp_sparse_indices"][0, 0, :2] = [0, 1]
    assert not np.array_equal(O.oracle(data, policy), actual)


def test_empty_selection_is_zero_whatever_the_sink(tiny):
    data, policy = tiny
    for name in ("seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv"):
        data[name][:] = 0
    data["cmp_sparse_indices"][:] = -1
    data["sinks"][:] = [-80, 80]
    assert np.array_equal(O.oracle(data, policy), np.zeros_like(data["q"]))


def test_padding_is_skipped_and_window_narrowing_is_honoured(tiny):
    data, policy = tiny
    data["ori_topk_length"][:] = 1
    data["cmp_sparse_indices"][0, 0] = [0, -1, -1, -1]
    rows, slots = O.selected_rows(data, policy, 0)
    assert slots == [0, 3]
    assert np.array_equal(rows[0], data["ori_kv"][0, 0, 0])


def test_indices_after_the_first_negative_are_ignored(tiny):
    data, policy = tiny
    data["cmp_sparse_indices"][0, 0] = [0, -1, 1, 0]
    assert O.selected_rows(data, policy, 0)[1] == [0, 1, 3]


def test_four_verification_tokens_have_their_own_edges(tiny):
    data, policy = tiny
    policy["T"] = 4
    data["q"] = np.zeros((4, 2, 4), dtype=np.float32)
    data["cu_seqlens_q"] = np.array([0, 4], dtype=np.int32)
    data["seqused_ori_kv"][:] = 6
    data["seqused_cmp_kv"][:] = 3
    data["cmp_residual_kv"][:] = 0
    data["ori_topk_length"] = np.zeros((4, 1), dtype=np.int32)
    data["cmp_sparse_indices"] = np.array(
        [[[2, 0, 1, -1]], [[0, 2, 1, -1]], [[1, 0, 2, -1]], [[2, 0, 1, -1]]], dtype=np.int32
    )
    for token, compressed in enumerate(([], [0], [1, 0], [2, 0, 1])):
        expected = [data["ori_kv"][data["ori_block_table"][0, p // 4], p % 4, 0] for p in range(token, token + 3)]
        expected += [data["cmp_kv"][data["cmp_block_table"][0, p // 2], p % 2, 0] for p in compressed]
        rows, _ = O.selected_rows(data, policy, token)
        assert np.array_equal(rows, np.asarray(expected, dtype=np.float32))
    before = O.oracle(data, policy)
    data["ori_kv"][0, 1, 0] += 10  # raw position 5: visible to the last token only
    data["cmp_kv"][0, 0, 0] += 10  # compressed index 2: complete for the last token only
    after = O.oracle(data, policy)
    assert np.array_equal(before[:3], after[:3])
    assert not np.array_equal(before[3], after[3])


def test_validation_cases_attend_to_real_rows():
    policy = O.make_policy(1, 1, h=32, d=128, max_seq=4096, blocks=32)
    for case in ("window", "mixed", "padding", "duplicates", "replay", "sink"):
        rows, _ = O.selected_rows(O.validation_inputs(policy, case), policy, 0)
        assert len(rows) > 0 and np.any(rows != 0)


def test_flop_convention_reproduces_published_row_counts():
    # README.md:33-38 of the reference: TFLOPS = 4*H*D*sum(valid rows) / time.
    def rows(b, n, ctx):
        total = 0
        for j in range(n):
            right = ctx - n + j + 1
            total += min(128, right) + min(512, right // 2)
        return b * total

    policy = O.make_policy(1, 1)
    assert rows(1, 8192, 32768) == 5_242_880
    assert rows(1, 32768, 32768) == 20_701_248
    assert rows(64, 6, 131072) == 245_760
    assert rows(128, 6, 131072) == 491_520
    assert abs(O.valid_row_flops(5_242_880, policy) / 6.847e-3 / 1e12 - 100.4) < 0.1
    assert abs(O.valid_row_flops(491_520, policy) / 0.810e-3 / 1e12 - 79.5) < 0.1
