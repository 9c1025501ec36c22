"""The CPU oracle against vectors produced by the reference's own oracle module.

`tests/golden/make_golden.py` wrote the fixture by running the reference's
`benchmarks/attention/sparse_reference.py` unmodified. Integer and byte results
(inputs, gathered rows, live masks, cache patches, codec words) must match bit
for bit. FP32 attention outputs are compared as 16-bit storage words with at
most one unit in the last place of slack, because BLAS summation order differs
between host CPUs.
"""

import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
from make_golden import SMALL, SUBSAMPLE, policy_of  # noqa: E402

from oracle import sparse_mla_oracle as O  # noqa: E402


def digest(array):
    array = np.ascontiguousarray(array)
    return hashlib.sha256(str(array.dtype).encode() + str(array.shape).encode() + array.tobytes()).hexdigest()


def ulp_distance(a_bits, b_bits):
    """Distance in storage-word steps for same-sign finite values (sign-magnitude order)."""
    a = a_bits.astype(np.int32)
    b = b_bits.astype(np.int32)
    a = np.where(a & 0x8000, -(a & 0x7FFF), a)
    b = np.where(b & 0x8000, -(b & 0x7FFF), b)
    return np.abs(a - b)


@pytest.mark.parametrize("name", list(SMALL))
@pytest.mark.parametrize("case", O.CASES)
def test_validation_case_matches_reference(golden, name, case):
    policy = policy_of(*SMALL[name])
    data = O.validation_inputs(policy, case)
    key = f"validation/{name}/{case}"
    for field, value in data.items():
        assert digest(value) == str(golden[f"{key}/input_sha256/{field}"]), field
    kv, bias = O.gather_oracle(data, policy)
    assert digest(kv) == str(golden[f"{key}/gather_kv_sha256"])
    live = np.unpackbits(golden[f"{key}/gather_live"])[: bias.size].reshape(bias.shape).astype(bool)
    assert np.array_equal(np.isfinite(bias), live)
    assert np.array_equal(O.resolve_rows(data, policy) >= 0, live)
    bits = O.encode_b16(O.oracle(data, policy), policy["DTYPE"])
    if name == "kernel_geometry":
        expected = golden[f"{key}/output_bits_sample"]
        actual = bits.reshape(-1)[::SUBSAMPLE]
    else:
        expected = golden[f"{key}/output_bits"]
        actual = bits
    assert actual.shape == expected.shape
    assert int(ulp_distance(actual, expected).max(initial=0)) <= 1
    # The bulk must be identical, not merely close.
    assert np.mean(actual == expected) > 0.995


@pytest.mark.parametrize("name", [n for n in SMALL if n != "kernel_geometry"])
def test_explicit_query_lengths_with_empty_requests(golden, name):
    key = f"validation/{name}/mixed_query_lens"
    if f"{key}/query_lens" not in golden:
        pytest.skip("fixture has no explicit-length case for this policy")
    policy = policy_of(*SMALL[name])
    lens = golden[f"{key}/query_lens"].tolist()
    data = O.validation_inputs(policy, "mixed", lens)
    kv, bias = O.gather_oracle(data, policy)
    assert digest(kv) == str(golden[f"{key}/gather_kv_sha256"])
    live = np.unpackbits(golden[f"{key}/gather_live"])[: bias.size].reshape(bias.shape).astype(bool)
    assert np.array_equal(np.isfinite(bias), live)
    bits = O.encode_b16(O.oracle(data, policy), policy["DTYPE"])
    assert int(ulp_distance(bits, golden[f"{key}/output_bits"]).max(initial=0)) <= 1


@pytest.mark.parametrize("name", ["prefill_c2", "prefill_c1", "chunk_c2", "decode_c2"])
def test_performance_inputs_match_reference_generator(golden, name):
    key = f"performance/{name}"
    b, t, ratio, context, seed = (int(v) for v in golden[f"{key}/arguments"])
    policy = policy_of(b, t, 2, 4, 4, ratio, 16, 3, 4, "bf16", 4 * b)
    arrays, rows, valid = O.performance_inputs(policy, context, seed)
    for field, value in arrays.items():
        assert digest(value) == str(golden[f"{key}/array_sha256/{field}"]), field
    expected_valid = np.unpackbits(golden[f"{key}/valid"])[: valid.size].reshape(valid.shape).astype(bool)
    assert np.array_equal(valid, expected_valid)
    caches = O.materialize_caches(policy, rows)
    for cache in ("ori_kv", "cmp_kv"):
        bits = O.encode_b16(caches[cache], "bf16")
        assert np.array_equal(bits, golden[f"{key}/cache_bits/{cache}"]), cache
    # The generator's live mask is exactly the oracle's (reference:
    # tests/tooling/test_sparse_performance.py:14-46).
    data = dict(arrays, **caches)
    _, bias = O.gather_oracle(data, policy)
    assert np.array_equal(np.isfinite(bias), valid)
    if name.startswith("prefill"):
        assert np.count_nonzero(valid[0]) == 1 + (ratio == 1)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_b16_codec_words(golden, dtype):
    probe = golden["codec/probe"]
    with np.errstate(over="ignore"):
        words = O.encode_b16(probe, dtype)
    assert np.array_equal(words, golden[f"codec/{dtype}"])
    again = O.encode_b16(O.decode_b16(words, dtype), dtype)
    finite = np.isfinite(O.decode_b16(words, dtype))
    assert np.array_equal(again[finite], words[finite])


def test_fp32_torch_form_agrees_with_numpy_form():
    policy = policy_of(*SMALL["c2_bf16"])
    for case in ("mixed", "sink", "replay", "empty"):
        data = O.validation_inputs(policy, case)
        fp32 = O.reference_fp32_from_data(data, policy, chunk=5)
        rounded = O.oracle(data, policy)
        # The batched form divides 0/denominator for empty tokens: zeros as well.
        assert np.allclose(O.round_b16(fp32, "bf16"), rounded, rtol=2 ** -7, atol=1e-6)
