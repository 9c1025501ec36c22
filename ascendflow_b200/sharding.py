"""Split one sparse MLA call across GPUs along its natural axes, without any exchange.

The operator has no cross-token or cross-request dependency, so a call is cut
either by request (decode: each GPU gets whole requests) or by query-token range
(prefill of one long request). Every shard is itself a legal call of the same
kernel: shapes shrink, `cu_seqlens_q` is re-based to zero and the per-request
lengths are trimmed so that each token keeps exactly the causal edges it has in
the unsharded call. Caches and block tables are read-only and can be replicated
or restricted to the shard's pages by the caller.

Causal edges follow the reference's geometry
(`examples/sparse_attention/gather.py:9-35`, `examples/sparse_attention/attention.py:339-341`):
for token j of n in a request with raw length L and C completed compressed rows
plus residual r (ratio R),

    right  = max(0, L - n + j + 1)
    cutoff = max(0, C*R + r - n + j + 1) // R

A shard holding tokens [j0, j1) of that request therefore presents
L' = L - (n - j1) and C'*R + r' = C*R + r - (n - j1) with n' = j1 - j0.

Works on anything sliceable like a NumPy array or a torch tensor.
"""

from __future__ import annotations

from .diagnostics import require

PER_TOKEN = ("q", "cmp_sparse_indices", "ori_topk_length", "attention_out")
PER_REQUEST = ("ori_block_table", "cmp_block_table")


def partition(total, parts):
    """`parts` contiguous ranges covering [0, total), sizes differing by at most one."""
    require(parts > 0 and total >= 0, "partition needs a positive part count")
    base, extra = divmod(total, parts)
    edges = [0]
    for index in range(parts):
        edges.append(edges[-1] + base + (1 if index < extra else 0))
    return [(edges[i], edges[i + 1]) for i in range(parts)]


def balanced_token_partition(weights, parts):
    """Contiguous token ranges of near-equal total weight (rows attended per token)."""
    total = float(sum(weights))
    ranges, start, running, target = [], 0, 0.0, total / parts
    for index, weight in enumerate(weights):
        running += weight
        remaining_parts = parts - len(ranges) - 1
        remaining_tokens = len(weights) - index - 1
        if len(ranges) < parts - 1 and (running >= target * (len(ranges) + 1) or remaining_tokens == remaining_parts):
            ranges.append((start, index + 1))
            start = index + 1
    ranges.append((start, len(weights)))
    while len(ranges) < parts:
        ranges.append((len(weights), len(weights)))
    return ranges


def _lengths(arrays):
    return [int(v) for v in arrays["cu_seqlens_q"]]


def shard_by_request(arrays, rank, world, ratio):
    """Requests [b0, b1) of the call, as a self-contained call. Returns (shard, (t0, t1))."""
    cu = _lengths(arrays)
    batches = len(cu) - 1
    require(world <= batches, "more ranks than requests: shard by token range instead")
    b0, b1 = partition(batches, world)[rank]
    t0, t1 = cu[b0], cu[b1]
    shard = dict(arrays)
    for name in PER_TOKEN:
        if name in arrays:
            shard[name] = arrays[name][t0:t1]
    for name in PER_REQUEST + ("seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv"):
        shard[name] = arrays[name][b0:b1]
    shard["cu_seqlens_q"] = arrays["cu_seqlens_q"][b0 : b1 + 1] - cu[b0]
    return shard, (t0, t1)


def shard_by_token_range(arrays, t0, t1, ratio):
    """Tokens [t0, t1) of the call. Requests cut by the range keep their causal edges."""
    cu = _lengths(arrays)
    batches = len(cu) - 1
    require(0 <= t0 <= t1 <= cu[-1], "token range outside the call")
    touched = [b for b in range(batches) if cu[b] < t1 and cu[b + 1] > t0]
    if not touched:  # empty shard: keep one request with no query so shapes stay legal
        touched = [0]
    b0, b1 = touched[0], touched[-1] + 1
    shard = dict(arrays)
    for name in PER_TOKEN:
        if name in arrays:
            shard[name] = arrays[name][t0:t1]
    for name in PER_REQUEST:
        shard[name] = arrays[name][b0:b1]
    new_cu, raw, completed_rows, residual = [0], [], [], []
    for b in range(b0, b1):
        first, last = max(cu[b], t0), min(cu[b + 1], t1)
        dropped_tail = cu[b + 1] - max(last, first)  # later tokens of the request that left
        if last <= first:
            dropped_tail = cu[b + 1] - cu[b]
        new_cu.append(new_cu[-1] + max(0, last - first))
        length = int(arrays["seqused_ori_kv"][b]) - dropped_tail
        completed = int(arrays["seqused_cmp_kv"][b]) * ratio + int(arrays["cmp_residual_kv"][b]) - dropped_tail
        raw.append(max(0, length))
        completed_rows.append(max(0, completed) // ratio)
        residual.append(max(0, completed) % ratio)
    like = arrays["cu_seqlens_q"]
    shard["cu_seqlens_q"] = _as_like(like, new_cu)
    shard["seqused_ori_kv"] = _as_like(like, raw)
    shard["seqused_cmp_kv"] = _as_like(like, completed_rows)
    shard["cmp_residual_kv"] = _as_like(like, residual)
    return shard, (t0, t1)


def _as_like(like, values):
    try:
        import numpy as np

        if isinstance(like, np.ndarray):
            return np.asarray(values, dtype=like.dtype)
    except ImportError:  # pragma: no cover
        pass
    return like.new_tensor(values)


def sizes_of(shard, ratio):
    """Runtime size parameters (B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE) of a call."""
    return {
        "B": int(shard["ori_block_table"].shape[0]),
        "T": int(shard["q"].shape[0]),
        "PAGES": int(shard["ori_block_table"].shape[1]),
        "ORI_BLOCKS": int(shard["ori_kv"].shape[0]),
        "CMP_BLOCKS": int(shard["cmp_kv"].shape[0]),
        "CMP_PAGE": 128 // ratio,
    }
