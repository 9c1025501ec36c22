"""Full-size parity on a B200: properties that do not need the CPU oracle on every token.

At the benchmark sizes the oracle can only afford a sample, so the tcgen05 kernel is compared
(a) on every token with the independent warp-MMA implementation of the same operator, called
through its own C-ABI entry, and (b) on sampled tokens, including both ends and tile borders,
with the FP32 reference. The gathered index set is compared bit for bit on all tokens.
"""

import ctypes as ct

import numpy as np
import pytest

from oracle import sparse_mla_oracle as O
from tests import support as S

pytestmark = pytest.mark.gpu


def cross_check_output(tensors, meta, config):
    """Run the warp-MMA kernel on the same inputs into a fresh output tensor."""
    import torch

    from ascendflow_b200.build import library_path
    from ascendflow_b200.runtime.torch import _library

    library = _library(library_path())
    launch = library.launch_sparse_mla_warp_mma
    launch.argtypes = [ct.c_void_p] * 15 + [ct.c_int64] * 6
    launch.restype = ct.c_int
    out = torch.full_like(tensors["attention_out"], float("nan"))
    workspace = torch.empty(1024, dtype=torch.uint8, device=out.device)
    names = [n for n in S.TENSOR_ORDER if n != "attention_out"]
    blocks = tensors["ori_kv"].shape[0]
    status = launch(torch.cuda.current_stream().cuda_stream, *(tensors[n].data_ptr() for n in names),
                    out.data_ptr(), workspace.data_ptr(), config["batches"],
                    config["batches"] * config["queries"], tensors["ori_block_table"].shape[1], blocks,
                    tensors["cmp_kv"].shape[0], tensors["cmp_kv"].shape[1])
    assert status == 0
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("name", ["prefill_q8k_ctx32k", "decode_b64_q6_ctx128k"])
def test_benchmark_configuration(name):
    import torch

    from ascendflow_b200 import ops, workloads as W

    config = W.CONFIGS[name]
    tensors, meta, work = W.device_case(**config, seed=7)
    policy = O.make_policy(config["batches"], work["tokens"], max_seq=config["max_seq"])
    ops.sparse_mla(*tensors.values())
    torch.cuda.synchronize()
    assert ops.kernel("sparse_mla").bind(*tensors.values())().status()[0] == 0

    # (a) two independent implementations agree on every token
    other = cross_check_output(tensors, meta, config)
    ours = tensors["attention_out"].float()
    difference = (ours - other.float()).abs()
    assert torch.isfinite(ours).all()
    assert float(difference.max()) <= 2e-2
    relative = float(difference.pow(2).sum().sqrt() / other.float().pow(2).sum().sqrt())
    assert relative <= 5e-3, relative

    # (b) sampled tokens against the FP32 reference
    tokens = work["tokens"]
    rng = np.random.default_rng(3)
    sample = sorted(set([0, 1, 63, 64, 147, 148, tokens - 1] + rng.choice(tokens, 24, replace=False).tolist()))
    sample = [t for t in sample if 0 <= t < tokens]
    expected = S.sampled_reference(tensors, meta, policy, sample)
    actual = S.output_to_numpy(tensors["attention_out"][torch.as_tensor(sample, device=ours.device)], "bf16")
    S.assert_close(actual, expected, name)

    # (c) gathered index set, all tokens, bit exact
    names = ("cmp_sparse_indices", "ori_block_table", "cmp_block_table", "cu_seqlens_q",
             "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length")
    resolved = ops.resolve_rows(*(tensors[n] for n in names), ori_blocks=policy["ORI_BLOCKS"],
                                cmp_blocks=policy["CMP_BLOCKS"], cmp_page=64).cpu().numpy()
    assert np.array_equal(resolved, O.resolve_rows(meta, policy))
    assert int((resolved >= 0).sum()) == work["live_rows"]


def test_full_causal_prefill_has_short_early_tokens():
    """B=1, queries = context: early tokens see fewer than 128 + 512 rows, the first sees one."""
    import torch

    from ascendflow_b200 import ops, workloads as W

    config = dict(batches=1, queries=2048, context=2048, max_seq=4096)
    tensors, meta, work = W.device_case(**config, seed=13)
    policy = O.make_policy(1, 2048, max_seq=4096)
    ops.sparse_mla(*tensors.values())
    sample = [0, 1, 2, 3, 63, 64, 127, 128, 129, 255, 256, 1023, 1024, 1100, 2047]
    expected = S.sampled_reference(tensors, meta, policy, sample)
    actual = S.output_to_numpy(tensors["attention_out"][torch.as_tensor(sample, device="cuda")], "bf16")
    S.assert_close(actual, expected, "full causal prefill")
    other = cross_check_output(tensors, meta, config)
    assert float((tensors["attention_out"].float() - other.float()).abs().max()) <= 2e-2
