"""Seeded synthetic workloads with the reference's measurement shapes.

The reference measures on seeded synthetic tensors, not on a dataset
(`benchmarks/attention/sparse_performance.py:27-82`): full-length requests, one
random page permutation per request, and for token j of n a sorted draw without
replacement of `min(TOPK, right // RATIO)` compressed indices from
`[0, right // RATIO)` with `right = context - n + j + 1`. This module builds the
same structure with every tensor resident on a CUDA device. Differences, on
purpose: values are N(0, sigma) with sigma = 1 by default, and the caches are
filled completely on the device instead of zero-filled and patched from the host.
"""

from __future__ import annotations

import numpy as np
import torch

HEADS, FEATURES, WINDOW, TOPK, PAGE = 64, 512, 128, 512, 128

# The five named configurations: requests, query tokens per request, context, MAX_SEQ.
CONFIGS = {
    "cpu_reference_q256_ctx4k": dict(batches=1, queries=256, context=4096, max_seq=4096),
    "prefill_q8k_ctx32k": dict(batches=1, queries=8192, context=32768, max_seq=131072),
    "prefill_q32k_ctx32k": dict(batches=1, queries=32768, context=32768, max_seq=131072),
    "decode_b64_q6_ctx128k": dict(batches=64, queries=6, context=131072, max_seq=131072),
    "decode_b128_q6_ctx128k": dict(batches=128, queries=6, context=131072, max_seq=131072),
    # A smaller decode case (3.2 GB of caches) sized for multi-pass profiler captures.
    "decode_b16_q6_ctx128k": dict(batches=16, queries=6, context=131072, max_seq=131072),
}


def host_metadata(batches, queries, context, max_seq, ratio=2, seed=4102026):
    """Every int32 tensor of a call, as NumPy arrays, plus the live-row count."""
    rng = np.random.default_rng(seed)
    pages = max_seq // PAGE
    tables = np.stack([rng.permutation(pages) + r * pages for r in range(batches)]).astype(np.int32)
    tokens = batches * queries
    indices = np.full((tokens, 1, TOPK), -1, dtype=np.int32)
    live = 0
    for request in range(batches):
        for offset in range(queries):
            right = context - queries + offset + 1
            take = min(TOPK, right // ratio)
            if take:
                indices[request * queries + offset, 0, :take] = np.sort(
                    rng.choice(right // ratio, take, replace=False))
            live += min(WINDOW, right) + take
    return {
        "cmp_sparse_indices": indices,
        "ori_block_table": tables,
        "cmp_block_table": tables.copy(),
        "cu_seqlens_q": (np.arange(batches + 1) * queries).astype(np.int32),
        "seqused_ori_kv": np.full(batches, context, dtype=np.int32),
        "seqused_cmp_kv": np.full(batches, context // ratio, dtype=np.int32),
        "cmp_residual_kv": np.full(batches, context % ratio, dtype=np.int32),
        "ori_topk_length": np.zeros((tokens, 1), dtype=np.int32),
    }, live


def device_case(batches, queries, context, max_seq, *, ratio=2, seed=4102026, sigma=1.0,
                dtype=torch.bfloat16, device="cuda"):
    """All thirteen tensors on `device`, the host metadata and work counters."""
    meta, live = host_metadata(batches, queries, context, max_seq, ratio, seed)
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    tokens, blocks = batches * queries, batches * (max_seq // PAGE)

    def normal(shape):
        out = torch.empty(shape, dtype=dtype, device=device)
        flat = out.view(-1)
        step = 1 << 28  # draw in FP32 pieces, round to the storage type
        for first in range(0, flat.numel(), step):
            piece = flat[first : first + step]
            piece.copy_(torch.randn(piece.numel(), generator=generator, device=device) * sigma)
        return out

    tensors = {
        "q": normal((tokens, HEADS, FEATURES)),
        "ori_kv": normal((blocks, PAGE, 1, FEATURES)),
        "cmp_kv": normal((blocks, PAGE // ratio, 1, FEATURES)),
    }
    for name, value in meta.items():
        tensors[name] = torch.from_numpy(value).to(device)
    tensors["sinks"] = torch.linspace(-2, 2, HEADS, dtype=torch.float32, device=device)
    tensors["attention_out"] = torch.empty_like(tensors["q"])
    ordered = {name: tensors[name] for name in (
        "q", "ori_kv", "cmp_kv", "cmp_sparse_indices", "ori_block_table", "cmp_block_table",
        "cu_seqlens_q", "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length",
        "sinks", "attention_out")}
    return ordered, meta, work_counters(meta, live, batches, queries, context, ratio)


def work_counters(meta, live_rows, batches, queries, context, ratio=2):
    """FLOPs (4*H*D per live row, FMA = 2) and compulsory / logical byte counts of a call."""
    tokens = batches * queries
    indices = meta["cmp_sparse_indices"].reshape(batches, queries * TOPK)
    distinct = sum(int(np.unique(row[row >= 0]).size) for row in indices)
    window_union = batches * max(0, min(context, queries - 1 + WINDOW) if queries else 0)
    row_bytes = FEATURES * 2
    q_and_out = 2 * tokens * HEADS * row_bytes
    small = tokens * TOPK * 4 + sum(int(v.nbytes) for k, v in meta.items() if k != "cmp_sparse_indices")
    return {
        "tokens": tokens,
        "live_rows": int(live_rows),
        "flops": 4 * HEADS * FEATURES * int(live_rows),
        "unique_bytes": (distinct + window_union) * row_bytes + q_and_out + small,
        "logical_bytes": int(live_rows) * row_bytes + q_and_out + small,
    }
