"""CUDA path against the CPU oracle, through the C ABI, on a B200.

Mirrors the reference's device validation (`benchmarks/attention/run_sparse.py:171-338`):
the eight named cases at the default policy (B4 / T16 / H64 / D512), ragged explicit query
lengths, guard bytes behind every buffer, inputs unchanged, the gathered index set compared
bit for bit, the output compared with the independent FP32 formula.
"""

import numpy as np
import pytest

from oracle import sparse_mla_oracle as O
from tests import support as S

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from ascendflow_b200 import ops as module

    return module


def default_policy(ratio=2, dtype="bf16", b=4, t=16, max_seq=4096):
    return O.make_policy(b, t, ratio=ratio, max_seq=max_seq, dtype=dtype, blocks=128)


def run_case(ops, data, policy, guard=True):
    import torch

    tensors, buffers = S.to_device(data, policy, guard=guard)
    before = {name: raw.clone() for name, raw in buffers.items() if name != "attention_out"}
    ops.sparse_mla(*(tensors[name] for name in S.TENSOR_ORDER))
    torch.cuda.synchronize()
    for name, raw in buffers.items():
        assert bool((raw[-S.GUARD:] == S.GUARD_BYTE).all()), f"{name}: guard bytes changed"
        if name != "attention_out":
            assert torch.equal(raw, before[name]), f"{name}: input changed"
    return tensors, S.output_to_numpy(tensors["attention_out"], policy["DTYPE"])


def resolved_on_device(ops, tensors, policy):
    names = ("cmp_sparse_indices", "ori_block_table", "cmp_block_table", "cu_seqlens_q",
             "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length")
    out = ops.resolve_rows(*(tensors[n] for n in names), ori_blocks=policy["ORI_BLOCKS"],
                           cmp_blocks=policy["CMP_BLOCKS"], cmp_page=policy["PAGE"] // policy["RATIO"])
    return out.cpu().numpy().astype(np.int64)


@pytest.mark.parametrize("case", O.CASES)
@pytest.mark.parametrize("ratio", [2, 1])
def test_named_validation_cases(ops, case, ratio):
    policy = default_policy(ratio)
    data = O.validation_inputs(policy, case)
    tensors, actual = run_case(ops, data, policy)
    assert np.array_equal(resolved_on_device(ops, tensors, policy), O.resolve_rows(data, policy))
    expected = O.reference_fp32_from_data(data, policy)
    S.assert_close(actual, expected, f"{case}/C{ratio}")
    if case == "empty":
        assert not actual.any()


@pytest.mark.parametrize("lens", [[0, 2, 0, 14], [16, 0, 0, 0], [1, 1, 1, 13], [5, 5, 5, 1]])
def test_explicit_query_lengths(ops, lens):
    policy = default_policy()
    data = O.validation_inputs(policy, "mixed", lens)
    tensors, actual = run_case(ops, data, policy)
    assert np.array_equal(resolved_on_device(ops, tensors, policy), O.resolve_rows(data, policy))
    S.assert_close(actual, O.reference_fp32_from_data(data, policy), str(lens))


def test_fp16_specialisation(ops):
    policy = default_policy(dtype="f16")
    for case in ("mixed", "sink", "replay"):
        data = O.validation_inputs(policy, case)
        _, actual = run_case(ops, data, policy)
        S.assert_close(actual, O.reference_fp32_from_data(data, policy), f"f16/{case}")


def test_single_token_and_odd_token_counts(ops):
    for b, t in ((1, 1), (1, 3), (2, 5), (7, 7)):
        policy = default_policy(b=b, t=t)
        policy["ORI_BLOCKS"] = policy["CMP_BLOCKS"] = 64
        data = O.validation_inputs(policy, "mixed")
        _, actual = run_case(ops, data, policy)
        S.assert_close(actual, O.reference_fp32_from_data(data, policy), f"B{b}T{t}")


def test_unsorted_indices_and_entries_after_padding(ops):
    policy = default_policy()
    data = O.validation_inputs(policy, "mixed")
    rng = np.random.default_rng(3)
    for token in range(policy["T"]):
        row = data["cmp_sparse_indices"][token, 0]
        live = int((row >= 0).sum())
        row[:live] = rng.permutation(row[:live])
        if live + 2 < len(row):
            row[live + 1] = 0  # after the first -1: must be ignored
    tensors, actual = run_case(ops, data, policy)
    assert np.array_equal(resolved_on_device(ops, tensors, policy), O.resolve_rows(data, policy))
    S.assert_close(actual, O.reference_fp32_from_data(data, policy), "unsorted")


def test_future_rows_do_not_leak(ops):
    """Changing cache rows only a later token may see leaves earlier tokens bit-identical."""
    import torch

    policy = default_policy(b=1, t=6, max_seq=1024)
    policy["ORI_BLOCKS"] = policy["CMP_BLOCKS"] = 8
    arrays, rows, _ = O.performance_inputs(policy, 700, 5)
    data = dict(arrays, **O.materialize_caches(policy, rows))
    tensors, first = run_case(ops, data, policy, guard=False)
    resolved = O.resolve_rows(data, policy)
    last_only_raw = set(resolved[5, :128].tolist()) - set(resolved[:5, :128].reshape(-1).tolist()) - {-1}
    assert last_only_raw
    flat = tensors["ori_kv"].view(-1, 512)
    flat[torch.as_tensor(sorted(last_only_raw), device=flat.device)] += 4.0
    ops.sparse_mla(*(tensors[name] for name in S.TENSOR_ORDER))
    second = S.output_to_numpy(tensors["attention_out"], "bf16")
    assert np.array_equal(first[:5], second[:5])
    assert not np.array_equal(first[5], second[5])


def test_reference_cpu_configuration(ops):
    """B=1, 256 queries at the end of a 4096-token context: every token checked."""
    from ascendflow_b200 import workloads as W

    tensors, meta, work = W.device_case(**W.CONFIGS["cpu_reference_q256_ctx4k"], seed=11)
    policy = O.make_policy(1, 256, max_seq=4096)
    ops.sparse_mla(*tensors.values())
    actual = S.output_to_numpy(tensors["attention_out"], "bf16")
    tokens = list(range(256))
    expected = S.sampled_reference(tensors, meta, policy, tokens)
    S.assert_close(actual, expected, "config 1")
    assert work["live_rows"] == 163_840 and work["flops"] == 4 * 64 * 512 * 163_840


def test_status_block_reports_a_bad_page_without_faulting(ops):
    import torch

    policy = default_policy()
    data = O.validation_inputs(policy, "mixed")
    data["ori_block_table"][1, :] = policy["ORI_BLOCKS"] + 5  # outside the cache: slot masked
    tensors, _ = S.to_device(data, policy)
    binding = ops.kernel("sparse_mla")(*(tensors[name] for name in S.TENSOR_ORDER))
    status = binding.status()
    assert status[0] == 1
    actual = S.output_to_numpy(tensors["attention_out"], "bf16")
    assert np.isfinite(actual).all()
    torch.cuda.synchronize()


def test_upstream_shaped_entry(ops):
    import torch

    from ascendflow_b200.diagnostics import CompileError
    from ascendflow_b200.upstream import sparse_flash_mla

    policy = default_policy()
    data = O.validation_inputs(policy, "mixed")
    tensors, _ = S.to_device(data, policy)
    names = ("q", "ori_kv", "cmp_kv", "cmp_sparse_indices", "ori_block_table", "cmp_block_table",
             "cu_seqlens_q", "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length", "sinks")
    out = sparse_flash_mla(*(tensors[n] for n in names), softmax_scale=512 ** -0.5, cmp_ratio=2)
    S.assert_close(S.output_to_numpy(out, "bf16"), O.reference_fp32_from_data(data, policy), "upstream entry")
    # No sink given: the denominator is the plain softmax sum.
    free = sparse_flash_mla(*(tensors[n] for n in names[:10]))
    data["sinks"] = np.full(64, -1.0e30, dtype=np.float32)
    S.assert_close(S.output_to_numpy(free, "bf16"), O.reference_fp32_from_data(data, policy), "no sink")
    with pytest.raises(CompileError, match="LSE"):
        sparse_flash_mla(*(tensors[n] for n in names), return_softmax_lse=True)
    with pytest.raises(CompileError, match="TND"):
        sparse_flash_mla(*(tensors[n] for n in names), layout_q="BSND")


def test_bounded_wait_gives_up_and_reports_without_hanging(ops):
    """Failure detection without a fault: a wait nobody satisfies expires, the status block says so,
    and the same context keeps working."""
    import ctypes as ct
    import time

    import torch

    from ascendflow_b200.build import library_path
    from ascendflow_b200.runtime.torch import _library

    library = _library(library_path())
    selftest = library.launch_sparse_mla_wait_expiry_selftest
    selftest.argtypes, selftest.restype = [ct.c_void_p, ct.c_void_p, ct.c_int64], ct.c_int
    read = library.read_status_sparse_mla
    read.argtypes, read.restype = [ct.c_void_p, ct.c_void_p, ct.POINTER(ct.c_int32)], ct.c_int
    workspace = torch.empty(1024, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    started = time.perf_counter()
    assert selftest(stream, workspace.data_ptr(), 2_000_000) == 0   # about a millisecond of clocks
    words = (ct.c_int32 * 8)()
    assert read(stream, workspace.data_ptr(), words) == 0
    assert time.perf_counter() - started < 5.0
    assert words[0] == 2 and words[2] == 1
    assert selftest(stream, workspace.data_ptr(), 0) == -1
    # The context is intact: a normal call still runs and is correct.
    policy = default_policy()
    data = O.validation_inputs(policy, "mixed")
    _, actual = run_case(ops, data, policy)
    S.assert_close(actual, O.reference_fp32_from_data(data, policy), "after the expired wait")


@pytest.mark.parametrize("seed", range(8))
def test_randomised_requests(ops, seed):
    """Random request mixes: ragged and empty requests, short caches, narrowed windows, padded,
    duplicated, unsorted and causally incomplete indices, both compression ratios."""
    rng = np.random.default_rng(1000 + seed)
    ratio = int(rng.choice([1, 2]))
    b = int(rng.integers(1, 7))
    lens = [int(v) for v in rng.integers(0, 9, b)]
    if sum(lens) == 0:
        lens[0] = 3
    max_seq = int(rng.choice([512, 1024, 4096]))
    policy = O.make_policy(b, sum(lens), ratio=ratio, max_seq=max_seq, blocks=int(rng.integers(8, 48)))
    data = O.validation_inputs(policy, str(rng.choice(["mixed", "padding", "duplicates", "replay", "sink"])), lens)
    # Per-request cache lengths anywhere from "just the queries" to the table capacity.
    lengths = np.array([int(rng.integers(max(n, 0), max_seq + 1)) for n in lens], dtype=np.int32)
    if rng.random() < 0.3:
        lengths[int(rng.integers(0, b))] = lens[int(rng.integers(0, b))]  # a cache holding only its queries
    lengths = np.maximum(lengths, np.array(lens, dtype=np.int32))
    data["seqused_ori_kv"] = lengths
    data["seqused_cmp_kv"] = (lengths // ratio).astype(np.int32)
    data["cmp_residual_kv"] = (lengths % ratio).astype(np.int32)
    span = max(1, max_seq // ratio)
    for token in range(policy["T"]):
        count = int(rng.integers(0, 513))
        row = np.full(512, -1, dtype=np.int32)
        row[:count] = rng.integers(0, span, count)   # any order, duplicates, some beyond the cutoff
        data["cmp_sparse_indices"][token, 0] = row
        data["ori_topk_length"][token, 0] = int(rng.choice([0, 0, 1, 5, 64, 128]))
    tensors, actual = run_case(ops, data, policy)
    assert np.array_equal(resolved_on_device(ops, tensors, policy), O.resolve_rows(data, policy))
    S.assert_close(actual, O.reference_fp32_from_data(data, policy), f"seed {seed}")


def test_blocks_walk_through_empty_and_short_tokens(ops):
    """More tokens than blocks, so that one persistent block meets, in turn, a full token, a token
    with nothing visible, another full one and tokens of one or two chunks: the roles hand work
    across token boundaries and must neither stall (status word) nor mix tokens up."""
    sms = 148
    lens = [sms, 2 * sms, sms + 52]           # block b gets tokens b, b + 148, b + 296, b + 444, ...
    policy = O.make_policy(len(lens), sum(lens), ratio=2, max_seq=4096, blocks=128)
    data = O.validation_inputs(policy, "mixed", lens)
    # Request 1 holds half as many cached rows as it has queries: its first 148 tokens see nothing.
    # Request 2 holds exactly its queries: token j sees j + 1 window rows (one or two chunks) and
    # (j + 1) // 2 compressed rows.
    lengths = np.array([2048, sms, lens[2]], dtype=np.int32)
    data["seqused_ori_kv"] = lengths
    data["seqused_cmp_kv"] = (lengths // 2).astype(np.int32)
    data["cmp_residual_kv"] = (lengths % 2).astype(np.int32)
    rng = np.random.default_rng(77)
    for token in range(policy["T"]):
        count = int(rng.integers(0, 513))
        row = np.full(512, -1, dtype=np.int32)
        row[:count] = rng.integers(0, 1024, count)
        data["cmp_sparse_indices"][token, 0] = row
    tensors, buffers = S.to_device(data, policy)
    binding = ops.kernel("sparse_mla")(*(tensors[name] for name in S.TENSOR_ORDER))
    assert binding.status()[0] == 0
    rows = O.resolve_rows(data, policy)
    live = (rows >= 0).sum(axis=1)
    assert (live[sms:2 * sms] == 0).all() and (live[:sms] > 0).all() and (live[2 * sms:3 * sms] > 0).all()
    actual = S.output_to_numpy(tensors["attention_out"], "bf16")
    assert not actual[sms:2 * sms].any()
    S.assert_close(actual, O.reference_fp32_from_data(data, policy), "empty and short tokens")


@pytest.mark.parametrize("seed,dtype", [(0, "bf16"), (1, "bf16"), (2, "bf16"), (1, "f16")])
def test_randomised_long_walks(ops, seed, dtype):
    """Several hundred tokens, so that every persistent block works through a random sequence of
    long, short and empty tokens: requests of 40-300 queries whose caches hold anything from
    nothing beyond a few rows to thousands of rows, random index counts, narrowed windows."""
    rng = np.random.default_rng(5000 + seed)
    ratio = int(rng.choice([1, 2]))
    b = int(rng.integers(3, 8))
    lens = [int(v) for v in rng.integers(40, 301, b)]
    max_seq = 4096
    policy = O.make_policy(b, sum(lens), ratio=ratio, max_seq=max_seq, dtype=dtype, blocks=int(rng.integers(40, 128)))
    data = O.validation_inputs(policy, str(rng.choice(["mixed", "padding", "replay"])), lens)
    # Caches shorter than the query count leave the request's first tokens with nothing to see.
    lengths = np.array([int(rng.choice([rng.integers(1, n + 1), rng.integers(n, max_seq + 1)])) for n in lens], dtype=np.int32)
    data["seqused_ori_kv"] = lengths
    data["seqused_cmp_kv"] = (lengths // ratio).astype(np.int32)
    data["cmp_residual_kv"] = (lengths % ratio).astype(np.int32)
    span = max(1, max_seq // ratio)
    for token in range(policy["T"]):
        count = int(rng.choice([0, 1, 40, 64, 65, 200, 512]))
        row = np.full(512, -1, dtype=np.int32)
        row[:count] = np.sort(rng.integers(0, span, count))
        data["cmp_sparse_indices"][token, 0] = row
        data["ori_topk_length"][token, 0] = int(rng.choice([0, 0, 0, 1, 64, 100]))
    tensors, _ = S.to_device(data, policy)
    binding = ops.kernel("sparse_mla" if dtype == "bf16" else "sparse_mla_f16")(*(tensors[name] for name in S.TENSOR_ORDER))
    assert binding.status()[0] == 0
    assert np.array_equal(resolved_on_device(ops, tensors, policy), O.resolve_rows(data, policy))
    actual = S.output_to_numpy(tensors["attention_out"], dtype)
    S.assert_close(actual, O.reference_fp32_from_data(data, policy), f"long walk {seed} {dtype}")


def test_gather_experiment_rows_are_bit_exact():
    """The isolated gather experiment (counterpart of the reference's gather study) checks its rows."""
    from ascendflow_b200 import gather_bench

    records = gather_bench.run(requests=8, queries=4, threads=(256,), depths=(2,), repeats=2)
    assert len(records) == 2 and all(r["rows_exact"] for r in records)
    assert {r["address"] for r in records} == {"lookup", "physical"}


@pytest.mark.parametrize("kernel_name,dtype", [("sparse_mla", "bf16"), ("sparse_mla_f16", "f16")])
def test_maximum_that_grows_in_later_chunks(ops, kernel_name, dtype):
    """Rows planted late in a token's slot list score far above everything before them, twice:
    the running maximum of one head moves by much more than the lazy-rescale threshold while
    the accumulator already holds earlier chunks, so the accumulator rows (which other threads
    hold than those that know the factor) must be rescaled."""
    import torch

    from ascendflow_b200 import workloads as W

    storage = torch.bfloat16 if dtype == "bf16" else torch.float16
    tensors, meta, _ = W.device_case(**W.CONFIGS["cpu_reference_q256_ctx4k"], seed=23, dtype=storage, sigma=0.5)
    policy = O.make_policy(1, 256, max_seq=4096, dtype=dtype)
    tokens = [40, 97, 160, 255]
    resolved = O.resolve_rows(meta, policy, tokens)
    cmp = tensors["cmp_kv"].view(-1, 512)
    used = set()
    for local, token in enumerate(tokens):
        head = (7 * local + 3) % 64
        for slot, factor in ((128 + 64 * 2 + 5, 1.0), (128 + 64 * 5 + 40, 3.0), (128 + 64 * 7 + 63, 6.0)):
            row = int(resolved[local, slot])
            assert row >= 0 and row not in used
            used.add(row)
            cmp[row] = (tensors["q"][token, head].float() * factor).to(storage)
    binding = ops.kernel(kernel_name)(*tensors.values())
    assert binding.status()[0] == 0
    actual = S.output_to_numpy(tensors["attention_out"], dtype)
    everyone = list(range(256))  # the planted rows are visible to other tokens as well
    S.assert_close(actual, S.sampled_reference(tensors, meta, policy, everyone), f"late maximum {dtype}")


def test_every_block_starts_with_a_run_of_empty_tokens(ops):
    """A first request whose cache holds nothing (1200 queries, seqused_ori_kv = 0) in a call large
    enough for blocks to take eight consecutive tokens per round: every block's first tokens are
    empty, so the resolver and the softmax warps could race ahead of the roles that only learn a
    token's chunk count later. Status stays 0, the empty request's rows are zero, the rest matches."""
    lens = [1200, 4800]
    policy = O.make_policy(len(lens), sum(lens), ratio=2, max_seq=8192, blocks=160)
    data = O.validation_inputs(policy, "mixed", lens)
    lengths = np.array([0, 5000], dtype=np.int32)
    data["seqused_ori_kv"] = lengths
    data["seqused_cmp_kv"] = (lengths // 2).astype(np.int32)
    data["cmp_residual_kv"] = (lengths % 2).astype(np.int32)
    rng = np.random.default_rng(91)
    for token in range(policy["T"]):
        row = np.full(512, -1, dtype=np.int32)
        count = int(rng.choice([0, 30, 512]))
        row[:count] = np.sort(rng.integers(0, 2500, count))
        data["cmp_sparse_indices"][token, 0] = row
    tensors, _ = S.to_device(data, policy)
    binding = ops.kernel("sparse_mla")(*(tensors[name] for name in S.TENSOR_ORDER))
    assert binding.status()[0] == 0
    actual = S.output_to_numpy(tensors["attention_out"], "bf16")
    assert not actual[:lens[0]].any()
    sample = sorted(rng.choice(np.arange(lens[0], policy["T"]), 96, replace=False).tolist())
    assert np.array_equal(resolved_on_device(ops, tensors, policy)[sample], O.resolve_rows(data, policy, sample))
    S.assert_close(actual[sample], S.sampled_reference(tensors, data, policy, sample), "after the empty request")
