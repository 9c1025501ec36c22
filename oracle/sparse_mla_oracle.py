"""NumPy / torch-CPU restatement of the reference's sparse MLA oracle.

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU
baseline. The product package never imports it.

Parity is PINNED: `tests/golden/` holds vectors produced by the reference's own
`benchmarks/attention/sparse_reference.py` (run unmodified through a shim that
only supplies `ascendflow.diagnostics`), and `tests/test_oracle_golden.py`
checks every function here against them, together with the hand-sized
known-answer cases of `tests/operators/test_sparse_attention.py:14-129`.

What follows which reference lines (paths relative to the reference project):

===========================  ==================================================
here                         reference
===========================  ==================================================
`encode_b16`, `decode_b16`   benchmarks/validation/dtypes.py:6-26
`query_counts`               benchmarks/attention/sparse_reference.py:19-26
`token_geometry`             benchmarks/attention/sparse_reference.py:29-42
                             (device form: examples/sparse_attention/gather.py:9-35,
                             examples/sparse_attention/attention.py:339-341)
`resolve_rows`               benchmarks/attention/sparse_reference.py:107-124
`selected_rows`              benchmarks/attention/sparse_reference.py:107-124
`gather_oracle`              benchmarks/attention/sparse_reference.py:174-181
`attend_rows`, `oracle`      benchmarks/attention/sparse_reference.py:127-138
`reference_fp32`             benchmarks/attention/sparse_reference.py:141-171
                             (the "PyTorch numerical reference"; the original
                             hard-codes device="npu", this runs the same FP32
                             bmm / masked softmax with sink / bmm on the CPU)
`validation_inputs`          benchmarks/attention/sparse_reference.py:45-104
`performance_inputs`         benchmarks/attention/sparse_performance.py:27-82
`valid_row_flops`            README.md:38 (effective QK+PV FLOPs, FMA = 2)
===========================  ==================================================
"""

from __future__ import annotations

import numpy as np

CASES = ("empty", "window", "mixed", "ragged", "padding", "duplicates", "replay", "sink")
VALIDATION_SEED = 4102026


# --------------------------------------------------------------------------
# 16-bit storage
# --------------------------------------------------------------------------

def encode_b16(values, dtype):
    """FP32 -> 16-bit storage words (uint16), round to nearest, ties to even."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    if dtype == "f16":
        return values.astype(np.float16).view(np.uint16)
    if dtype != "bf16":
        raise ValueError("oracle requires an explicit b16 dtype")
    word = values.view(np.uint32)
    bias = np.uint32(0x7FFF) + ((word >> np.uint32(16)) & np.uint32(1))
    return ((word + bias) >> np.uint32(16)).astype(np.uint16)


def decode_b16(bits, dtype):
    """16-bit storage words -> FP32."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if dtype == "f16":
        return bits.view(np.float16).astype(np.float32)
    if dtype != "bf16":
        raise ValueError("oracle requires an explicit b16 dtype")
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_b16(values, dtype):
    return decode_b16(encode_b16(values, dtype), dtype).reshape(np.shape(values))


# --------------------------------------------------------------------------
# request / token geometry
# --------------------------------------------------------------------------

def query_counts(policy, ragged=False):
    """Query tokens per request: T spread evenly, the remainder on the first requests."""
    b, t = int(policy["B"]), int(policy["T"])
    counts = np.full(b, t // b, dtype=np.int32)
    counts[: t % b] += 1
    if ragged and b >= 3 and t >= 3:
        head = int(counts[:3].sum())
        counts[:3] = (0, head // 3, head - head // 3)
    return counts


def token_geometry(data, policy):
    """Per-token causal edges, for all T tokens at once.

    Returns int64 arrays of length T: `batch`, `right` (exclusive right edge of
    the raw window), `visible` (window rows kept), `available` (completed
    compressed rows of the request), `cutoff` (exclusive bound on compressed
    indices) and `bound` (number of index ranks examined).
    """
    cu = np.asarray(data["cu_seqlens_q"], dtype=np.int64)
    total = int(cu[-1])
    token = np.arange(total, dtype=np.int64)
    batch = np.searchsorted(cu, token, side="right") - 1
    count = cu[batch + 1] - cu[batch]
    offset = token - cu[batch]
    length = np.asarray(data["seqused_ori_kv"], dtype=np.int64)[batch]
    right = np.maximum(0, length - count + offset + 1)
    visible = np.minimum(int(policy["WINDOW"]), right)
    requested = np.asarray(data["ori_topk_length"], dtype=np.int64).reshape(-1)[:total]
    visible = np.where(requested > 0, np.minimum(visible, requested), visible)
    ratio = int(policy["RATIO"])
    available = np.asarray(data["seqused_cmp_kv"], dtype=np.int64)[batch]
    residual = np.asarray(data["cmp_residual_kv"], dtype=np.int64)[batch]
    cutoff = np.maximum(0, available * ratio + residual - count + offset + 1) // ratio
    bound = np.minimum(np.minimum(int(policy["TOPK"]), available), cutoff)
    return {
        "batch": batch,
        "right": right,
        "visible": visible,
        "available": available,
        "cutoff": cutoff,
        "bound": bound,
    }


def resolve_rows(data, policy, tokens=None):
    """The gathered index set: physical cache row per (token, slot), or -1.

    Slots [0, WINDOW) address rows of `ori_kv` flattened to
    `[ORI_BLOCKS * PAGE, D]`; slots [WINDOW, WINDOW + TOPK) address rows of
    `cmp_kv` flattened to `[CMP_BLOCKS * (PAGE // RATIO), D]`. Window slot s
    holds logical position `right - visible + s`. Compressed slot WINDOW + k
    holds index rank k when it is examined (`k < bound`), lies before the
    first negative index, and is causally complete (`index < cutoff`).
    """
    window, topk = int(policy["WINDOW"]), int(policy["TOPK"])
    page, ratio = int(policy["PAGE"]), int(policy["RATIO"])
    cmp_page = page // ratio
    geometry = token_geometry(data, policy)
    total = len(geometry["batch"])
    tokens = np.arange(total) if tokens is None else np.asarray(tokens, dtype=np.int64)
    batch = geometry["batch"][tokens]
    right, visible = geometry["right"][tokens], geometry["visible"][tokens]
    cutoff, bound = geometry["cutoff"][tokens], geometry["bound"][tokens]
    span = max(int(policy.get("S", window + topk)), window + topk)
    resolved = np.full((len(tokens), span), -1, dtype=np.int64)

    slot = np.arange(window, dtype=np.int64)[None, :]
    position = (right - visible)[:, None] + slot
    live = slot < visible[:, None]
    position = np.where(live, position, 0)
    table = np.asarray(data["ori_block_table"], dtype=np.int64)
    physical = table[batch[:, None], position // page] * page + position % page
    resolved[:, :window] = np.where(live, physical, -1)

    index = np.asarray(data["cmp_sparse_indices"], dtype=np.int64)[tokens, 0, :]
    rank = np.arange(topk, dtype=np.int64)[None, :]
    before_padding = np.cumsum(index < 0, axis=1) == 0
    live = before_padding & (rank < bound[:, None]) & (index < cutoff[:, None])
    index = np.where(live, index, 0)
    table = np.asarray(data["cmp_block_table"], dtype=np.int64)
    physical = table[batch[:, None], index // cmp_page] * cmp_page + index % cmp_page
    resolved[:, window : window + topk] = np.where(live, physical, -1)
    return resolved


def _flat_caches(data, policy):
    d = int(policy["D"])
    return (
        np.asarray(data["ori_kv"], dtype=np.float32).reshape(-1, d),
        np.asarray(data["cmp_kv"], dtype=np.float32).reshape(-1, d),
    )


def selected_rows(data, policy, token):
    """Rows one token attends to, window first then compressed ranks, and their slots."""
    window = int(policy["WINDOW"])
    resolved = resolve_rows(data, policy, [token])[0]
    ori, cmp = _flat_caches(data, policy)
    slots = [int(s) for s in np.flatnonzero(resolved >= 0)]
    rows = [ori[resolved[s]] if s < window else cmp[resolved[s]] for s in slots]
    return np.asarray(rows, dtype=np.float32).reshape(-1, int(policy["D"])), slots


def gather_oracle(data, policy):
    """Dense `[T, S, D]` gathered rows (zeros where unselected) and 0 / -inf bias `[T, S]`."""
    window = int(policy["WINDOW"])
    resolved = resolve_rows(data, policy)
    ori, cmp = _flat_caches(data, policy)
    total, slots = resolved.shape
    kv = np.zeros((total, slots, int(policy["D"])), dtype=np.float32)
    live = resolved >= 0
    head, tail = live[:, :window], live[:, window:]
    kv[:, :window][head] = ori[resolved[:, :window][head]]
    kv[:, window:][tail] = cmp[resolved[:, window:][tail]]
    bias = np.where(live, np.float32(0), np.float32(-np.inf)).astype(np.float32)
    return kv, bias


# --------------------------------------------------------------------------
# attention arithmetic
# --------------------------------------------------------------------------

def attend_rows(q_token, rows, sinks, scale):
    """One token: FP32 joint softmax over `rows` with one sink per head.

    `q_token` is `[H, D]`, `rows` is `[n, D]`. The sink has a zero value row,
    so it adds `exp(sink - max)` to the denominator only. No rows -> zeros.
    """
    q_token = np.asarray(q_token, dtype=np.float32)
    if len(rows) == 0:
        return np.zeros_like(q_token)
    rows = np.asarray(rows, dtype=np.float32)
    sinks = np.asarray(sinks, dtype=np.float32)
    scores = (q_token @ rows.T) * scale
    peak = np.maximum(scores.max(axis=1), sinks)
    weights = np.exp(scores - peak[:, None])
    denominator = weights.sum(axis=1) + np.exp(sinks - peak)
    return (weights @ rows) / denominator[:, None]


def oracle(data, policy, tokens=None):
    """Attention output `[T, H, D]` in FP32 arithmetic, rounded to the storage dtype."""
    q = np.asarray(data["q"], dtype=np.float32)
    window = int(policy["WINDOW"])
    ori, cmp = _flat_caches(data, policy)
    chosen = range(q.shape[0]) if tokens is None else tokens
    resolved = resolve_rows(data, policy, None if tokens is None else list(tokens))
    output = np.zeros((len(resolved),) + q.shape[1:], dtype=np.float32)
    for local, token in enumerate(chosen):
        ids = resolved[local]
        head, tail = ids[:window], ids[window:]
        rows = np.concatenate([ori[head[head >= 0]], cmp[tail[tail >= 0]]], axis=0)
        output[local] = attend_rows(q[token], rows, data["sinks"], policy["SCALE"])
    return round_b16(output, policy["DTYPE"])


def reference_fp32(q, sinks, rows_of, policy, chunk=128, threads=None):
    """FP32 batched QK / masked softmax with sink / PV on the CPU with torch.

    `rows_of(token)` returns that token's `[n, D]` rows. Tokens are processed
    `chunk` at a time against a zero-padded `[chunk, S, D]` cache; the
    probabilities stay FP32 through PV and the result is not rounded.
    """
    import torch

    if threads is not None:
        torch.set_num_threads(int(threads))
    q = np.asarray(q, dtype=np.float32)
    span, width = int(policy["S"]), int(policy["D"])
    sink = torch.from_numpy(np.asarray(sinks, dtype=np.float32))[None, :]
    output = np.empty_like(q)
    with torch.inference_mode():
        for first in range(0, len(q), chunk):
            count = min(chunk, len(q) - first)
            cache = np.zeros((count, span, width), dtype=np.float32)
            live = np.zeros((count, span), dtype=bool)
            for local in range(count):
                rows = rows_of(first + local)
                cache[local, : len(rows)] = rows
                live[local, : len(rows)] = True
            query = torch.from_numpy(q[first : first + count])
            keys = torch.from_numpy(cache)
            mask = torch.from_numpy(live)
            scores = torch.bmm(query, keys.transpose(1, 2)) * float(policy["SCALE"])
            scores.masked_fill_(~mask[:, None, :], float("-inf"))
            peak = torch.maximum(scores.amax(dim=-1), sink)
            weight = torch.exp(scores - peak[:, :, None])
            denominator = weight.sum(dim=-1) + torch.exp(sink - peak)
            output[first : first + count] = (
                torch.bmm(weight, keys) / denominator[:, :, None]
            ).numpy()
    return output


def reference_fp32_from_data(data, policy, chunk=128):
    """`reference_fp32` with rows selected from the paged caches of `data`."""
    return reference_fp32(
        data["q"],
        data["sinks"],
        lambda token: selected_rows(data, policy, token)[0],
        policy,
        chunk=chunk,
    )


# --------------------------------------------------------------------------
# the steps on either side of the operator (no reference implementation exists: the reference
# leaves them to its caller, docs/operators/sparse-mla.md:8, 263-266; their contracts follow from
# what the operator reads, docs/operators/sparse-mla.md:62-87). PARITY UNPINNED for these two:
# there is no golden vector or reference output to pin them against, only the consistency checks
# in tests/test_neighbours.py (the selection is what `resolve_rows` then accepts in full).
# --------------------------------------------------------------------------

def select_topk_indices(scores, data, policy):
    """`cmp_sparse_indices` `[T, 1, TOPK]` from index scores `[T, SPAN]`.

    Per token the candidates are compressed rows `[0, min(available, cutoff))` (what
    `resolve_rows` accepts); the `min(TOPK, candidates)` highest scores win, ties going to the
    lower index; winners in ascending order, then -1.
    """
    scores = np.asarray(scores, dtype=np.float32)
    geometry = token_geometry(dict(data, ori_topk_length=np.zeros((scores.shape[0], 1), np.int32)), policy)
    topk = int(policy["TOPK"])
    out = np.full((scores.shape[0], 1, topk), -1, dtype=np.int32)
    for token in range(scores.shape[0]):
        candidates = int(min(geometry["available"][token], geometry["cutoff"][token], scores.shape[1]))
        take = min(topk, candidates)
        if take == 0:
            continue
        order = np.lexsort((np.arange(candidates), -scores[token, :candidates].astype(np.float64)))
        out[token, 0, :take] = np.sort(order[:take]).astype(np.int32)
    return out


def append_rows(cache, new_rows, block_table, cu_seqlens_q, seqused_kv):
    """A copy of the paged `cache` `[BLOCKS, PAGE_ROWS, 1, D]` with a call's `new_rows` `[T, D]`
    written in: row j of the n of request b at logical position `seqused_kv[b] - n + j`."""
    cache = np.array(cache, copy=True)
    page_rows = cache.shape[1]
    cu = np.asarray(cu_seqlens_q, dtype=np.int64)
    for batch in range(len(cu) - 1):
        count = int(cu[batch + 1] - cu[batch])
        for offset in range(count):
            position = int(seqused_kv[batch]) - count + offset
            page = int(block_table[batch, position // page_rows])
            cache[page, position % page_rows, 0] = new_rows[cu[batch] + offset]
    return cache


# --------------------------------------------------------------------------
# input generators
# --------------------------------------------------------------------------

def validation_inputs(policy, case, query_lens=None):
    """The eight named validation cases, drawn in the reference's order from its seed.

    Draw order matters for bit-identical inputs: q, ori_kv, cmp_kv (normal,
    sigma 0.5), then the two block tables (uniform pages, sharing allowed),
    then one permutation per token that takes indices.
    """
    if case not in CASES:
        raise ValueError(f"unknown sparse attention case: {case}")
    b, t, h, d = (int(policy[k]) for k in ("B", "T", "H", "D"))
    page, ratio, max_seq, topk = (int(policy[k]) for k in ("PAGE", "RATIO", "MAX_SEQ", "TOPK"))
    dtype = policy["DTYPE"]
    rng = np.random.default_rng(VALIDATION_SEED)
    if query_lens is None:
        counts = query_counts(policy, ragged=(case == "ragged"))
    else:
        counts = np.array(query_lens, dtype=np.int32)
    pattern = np.array([page - 1, page + 1, 2 * page + 1, max_seq - 1])
    lengths = np.minimum(max_seq, np.maximum(counts, np.resize(pattern, b))).astype(np.int32)
    if case == "empty":
        lengths[:] = 0

    def draw(shape):
        return round_b16(rng.normal(0, 0.5, shape).astype(np.float32), dtype)

    data = {}
    data["q"] = draw((t, h, d))
    data["ori_kv"] = draw((int(policy["ORI_BLOCKS"]), page, 1, d))
    data["cmp_kv"] = draw((int(policy["CMP_BLOCKS"]), page // ratio, 1, d))
    data["cu_seqlens_q"] = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    data["seqused_ori_kv"] = lengths
    data["seqused_cmp_kv"] = lengths // ratio
    data["cmp_residual_kv"] = lengths % ratio
    data["ori_topk_length"] = np.zeros((t, 1), dtype=np.int32)
    data["cmp_sparse_indices"] = np.full((t, 1, topk), -1, dtype=np.int32)
    data["sinks"] = np.linspace(-2, 2, h, dtype=np.float32)
    for name, blocks in (("ori_block_table", "ORI_BLOCKS"), ("cmp_block_table", "CMP_BLOCKS")):
        data[name] = rng.integers(0, int(policy[blocks]), (b, max_seq // page), dtype=np.int32)

    geometry = token_geometry(data, policy)
    takes_indices = case not in ("empty", "window")
    for token in range(t):
        available = int(geometry["available"][token])
        count = int(geometry["bound"][token])
        if takes_indices and count > 0:
            if case == "padding":
                count = token % (count + 1)
            chosen = rng.permutation(available)[:count]
            if case == "duplicates":
                chosen[:] = 0
            elif case == "mixed":
                # The newest compressed row: early tokens of a request must filter it out.
                chosen[0] = available - 1
            data["cmp_sparse_indices"][token, 0, :count] = chosen
        if case == "replay" and token % 3 != 2:
            data["ori_topk_length"][token, 0] = 1 + token % 7
    if case == "sink":
        data["sinks"][:] = np.resize(np.array([-80, 80, 0, 5], dtype=np.float32), h)
    return data


def performance_inputs(policy, context, seed, query_lens=None, sigma=0.5):
    """Measurement inputs: full-length requests with sorted uniform causal indices.

    Returns `(arrays, rows, valid)`. `arrays` holds every tensor but the two
    caches. `rows` maps "ori_kv" / "cmp_kv" to `(physical_row_ids, values)`:
    only rows some query can touch get values (drawn per request, window union
    first, then the union of its indices); every other cache row is zero.
    `valid` is the `[T, WINDOW + TOPK]` mask of live slots.
    """
    b, t, h, d = (int(policy[k]) for k in ("B", "T", "H", "D"))
    topk, page, ratio = (int(policy[k]) for k in ("TOPK", "PAGE", "RATIO"))
    max_seq, window = int(policy["MAX_SEQ"]), int(policy["WINDOW"])
    counts = query_counts(policy) if query_lens is None else np.array(query_lens, np.int32)
    if len(counts) != b or int(counts.sum()) != t:
        raise ValueError("query lengths differ")
    if not int(counts.max()) <= context <= max_seq:
        raise ValueError("context must contain the query tokens")
    rng = np.random.default_rng(seed)
    pages = max_seq // page
    tables = np.stack([rng.permutation(pages) + r * pages for r in range(b)]).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    indices = np.full((t, 1, topk), -1, dtype=np.int32)
    valid = np.zeros((t, window + topk), dtype=bool)
    for request in range(b):
        n = int(counts[request])
        for offset in range(n):
            token = int(cu[request]) + offset
            right = context - n + offset + 1
            take = min(topk, right // ratio)
            indices[token, 0, :take] = np.sort(rng.choice(right // ratio, take, replace=False))
            valid[token, : min(window, right)] = True
            valid[token, window : window + take] = True
    q = round_b16(rng.normal(0, sigma, (t, h, d)).astype(np.float32), "bf16")
    arrays = {
        "q": q,
        "sinks": np.linspace(-2, 2, h, dtype=np.float32),
        "ori_block_table": tables,
        "cmp_block_table": tables.copy(),
        "cmp_sparse_indices": indices,
        "seqused_ori_kv": np.full(b, context, dtype=np.int32),
        "ori_topk_length": np.zeros((t, 1), dtype=np.int32),
        "cu_seqlens_q": cu,
        "seqused_cmp_kv": np.full(b, context // ratio, dtype=np.int32),
        "cmp_residual_kv": np.full(b, context % ratio, dtype=np.int32),
    }
    rows = {"ori_kv": ([], []), "cmp_kv": ([], [])}
    for request in range(b):
        n = int(counts[request])
        if n == 0:
            continue
        window_union = np.arange(max(0, context - n + 1 - window), context)
        index_union = np.unique(indices[cu[request] : cu[request + 1]])
        index_union = index_union[index_union >= 0]
        for name, positions, block in (
            ("ori_kv", window_union, page),
            ("cmp_kv", index_union, page // ratio),
        ):
            values = round_b16(rng.normal(0, sigma, (len(positions), d)).astype(np.float32), "bf16")
            physical = tables[request, positions // block].astype(np.int64) * block + positions % block
            rows[name][0].append(physical)
            rows[name][1].append(values)
    for name in rows:
        ids, values = rows[name]
        rows[name] = (
            np.concatenate(ids) if ids else np.zeros(0, np.int64),
            np.concatenate(values) if values else np.zeros((0, d), np.float32),
        )
    return arrays, rows, valid


def materialize_caches(policy, rows):
    """Dense zero-background caches from the sparse rows of `performance_inputs`."""
    page, ratio, d = int(policy["PAGE"]), int(policy["RATIO"]), int(policy["D"])
    caches = {}
    for name, blocks, block in (
        ("ori_kv", int(policy["ORI_BLOCKS"]), page),
        ("cmp_kv", int(policy["CMP_BLOCKS"]), page // ratio),
    ):
        dense = np.zeros((blocks * block, d), dtype=np.float32)
        ids, values = rows[name]
        dense[ids] = values
        caches[name] = dense.reshape(blocks, block, 1, d)
    return caches


# --------------------------------------------------------------------------
# work accounting
# --------------------------------------------------------------------------

def valid_row_count(data, policy):
    """Sum over tokens of live window rows + live compressed rows."""
    return int((resolve_rows(data, policy) >= 0).sum())


def valid_row_flops(valid_rows, policy):
    """Effective QK+PV FLOPs with FMA = 2: 4 * H * D per live (token, row) pair."""
    return 4 * int(policy["H"]) * int(policy["D"]) * int(valid_rows)


def make_policy(b, t, *, h=64, d=512, page=128, ratio=2, max_seq=4096, window=128, topk=512,
                dtype="bf16", blocks=None):
    """Policy dictionary with the reference's field names and derived sizes."""
    blocks = b * (max_seq // page) if blocks is None else blocks
    return {
        "B": b, "T": t, "H": h, "D": d, "PAGE": page, "RATIO": ratio, "MAX_SEQ": max_seq,
        "ORI_BLOCKS": blocks, "CMP_BLOCKS": blocks, "WINDOW": window, "TOPK": topk,
        "S": window + topk, "DTYPE": dtype, "SCALE": float(d) ** -0.5,
    }
