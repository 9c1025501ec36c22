"""The operator behind the argument list of the upstream call it corresponds to.

The reference's operator is the C1/C2 compute subset of vllm-ascend's
`torch.ops._C_ascend.npu_sparse_flash_mla` (docs/operators/sparse-mla.md:10-14 of the
reference); the positional list of the vendor entry is visible where the reference drives it
for comparison (benchmarks/references/sparse_mla_aclnn.py:95-137): q, ori_kv, cmp_kv, <unused>,
cmp_sparse_indices, the two block tables, cu_seqlens_q, three unused slots, the three length
tensors, ori_topk_length, <unused>, sinks, metadata, scale, ratio, ori_mask_mode, cmp_mask_mode,
window left/right, the two layout strings, topk_value_mode, return-LSE flag, output, LSE.

`sparse_flash_mla` takes the used ones of those, checks that the fixed modes are the ones this
path implements (TND queries, PA_BBND caches, band mask 4 on the window with 127 rows to the
left, causal mask 3 on compressed rows, logical indices, no LSE), allocates the output and
calls the CUDA operator. The reference itself provides no such registration
(docs/operators/sparse-mla.md:74-76); this adapter is a convenience for callers written against
the upstream signature.
"""

from __future__ import annotations

import torch

from .diagnostics import ErrorKind, require
from .ops import sparse_mla

WINDOW, FEATURES = 128, 512


def sparse_flash_mla(q, ori_kv, cmp_kv, cmp_sparse_indices, ori_block_table, cmp_block_table,
                     cu_seqlens_q, seqused_ori_kv, seqused_cmp_kv, cmp_residual_kv,
                     ori_topk_length=None, sinks=None, *, softmax_scale=None, cmp_ratio=None,
                     ori_mask_mode=4, cmp_mask_mode=3, ori_win_left=WINDOW - 1, ori_win_right=0,
                     layout_q="TND", layout_kv="PA_BBND", topk_value_mode=1, return_softmax_lse=False,
                     attention_out=None):
    """Returns `attention_out` `[T, H, D]` (allocated when not given)."""
    unsupported = dict(kind=ErrorKind.UNSUPPORTED)
    require(layout_q == "TND" and layout_kv == "PA_BBND", "only TND queries and PA_BBND caches", **unsupported)
    require(ori_mask_mode == 4 and cmp_mask_mode == 3, "only band window mask 4 and causal compressed mask 3", **unsupported)
    require(ori_win_left == WINDOW - 1 and ori_win_right == 0, "window is 128 rows ending at the query", **unsupported)
    require(topk_value_mode == 1, "indices are logical compressed positions", **unsupported)
    require(not return_softmax_lse, "LSE output is not part of this path", **unsupported)
    ratio = WINDOW // int(cmp_kv.shape[1])
    require(cmp_ratio is None or int(cmp_ratio) == ratio, "cmp_ratio differs from the compressed page size")
    require(softmax_scale is None or abs(float(softmax_scale) - FEATURES ** -0.5) < 1e-7,
            "softmax scale is fixed at 512^-0.5", **unsupported)
    tokens = q.shape[0]
    if ori_topk_length is None:  # upstream: no narrowing
        ori_topk_length = torch.zeros((tokens, 1), dtype=torch.int32, device=q.device)
    if sinks is None:
        # No sink: a logit so low that its weight underflows to zero in FP32.
        sinks = torch.full((q.shape[1],), -1.0e30, dtype=torch.float32, device=q.device)
    if attention_out is None:
        attention_out = torch.empty_like(q)
    return sparse_mla(q, ori_kv, cmp_kv, cmp_sparse_indices, ori_block_table, cmp_block_table,
                      cu_seqlens_q, seqused_ori_kv, seqused_cmp_kv, cmp_residual_kv, ori_topk_length,
                      sinks, attention_out)
