"""The steps on either side of the attention call whose output the call's inputs fix.

The reference leaves the indexer, the compressor and the cache writes to its caller
(`docs/operators/sparse-mla.md:8, 263-266`). Two of them have an output format that the
operator dictates and are provided here on the device: `topk_indices` turns index scores into
`cmp_sparse_indices` (sorted, -1 padded, causally cut), `cache_append` puts a step's new raw
rows where the next attention call will look for them. Both launch on torch's current stream.
"""

from __future__ import annotations

import ctypes as ct

import torch

from .build import library_path
from .diagnostics import require
from .runtime.torch import _library


_entry_points = {}


def _entry(name, pointers, sizes):
    """The typed C entry point, looked up once: loading verifies the library file's hash, which
    costs milliseconds on the host."""
    if name not in _entry_points:
        function = getattr(_library(library_path()), name)
        function.argtypes, function.restype = [ct.c_void_p] * pointers + [ct.c_int64] * sizes, ct.c_int
        _entry_points[name] = function
    return _entry_points[name]


def _check(tensor, dtype, name):
    require(tensor.is_cuda and tensor.is_contiguous() and tensor.dtype == dtype,
            f"{name}: expected a contiguous {dtype} CUDA tensor")


def _raise_on(status):
    if status:
        raise RuntimeError(f"kernel launch failed with status {status}; device retries are disabled")


def topk_indices(scores, cu_seqlens_q, seqused_cmp_kv, cmp_residual_kv, *, ratio=2, out=None):
    """`cmp_sparse_indices` `[T, 1, 512]` int32 from index scores `[T, SPAN]` float32."""
    _check(scores, torch.float32, "scores")
    for name, tensor in (("cu_seqlens_q", cu_seqlens_q), ("seqused_cmp_kv", seqused_cmp_kv),
                         ("cmp_residual_kv", cmp_residual_kv)):
        _check(tensor, torch.int32, name)
    require(ratio in (1, 2), "compression ratio must be 1 or 2")
    tokens, span = scores.shape
    batches = seqused_cmp_kv.shape[0]
    require(cu_seqlens_q.shape[0] == batches + 1, "cu_seqlens_q must have one entry more than there are requests")
    if out is None:
        out = torch.empty((tokens, 1, 512), dtype=torch.int32, device=scores.device)
    _check(out, torch.int32, "cmp_sparse_indices")
    require(tuple(out.shape) == (tokens, 1, 512), "cmp_sparse_indices must be [T, 1, 512]")
    launch = _entry("launch_sparse_mla_topk_indices", 6, 4)
    stream = torch.cuda.current_stream(scores.device).cuda_stream
    _raise_on(launch(stream, scores.data_ptr(), cu_seqlens_q.data_ptr(), seqused_cmp_kv.data_ptr(),
                     cmp_residual_kv.data_ptr(), out.data_ptr(), batches, tokens, span, 128 // ratio))
    return out


def cache_append(new_rows, cache, block_table, cu_seqlens_q, seqused_kv):
    """Write `new_rows` `[T, 512]` into the paged `cache` `[BLOCKS, PAGE_ROWS, 1, 512]` in place.

    `seqused_kv` counts the new rows, as it does for the attention call that follows. Returns the
    status block (word 0: 0 ok, 1 a row had no legal page), which synchronises the stream.
    """
    require(new_rows.is_cuda and cache.is_cuda and new_rows.dtype == cache.dtype
            and new_rows.dtype in (torch.bfloat16, torch.float16), "rows and cache must be 16-bit CUDA tensors of one dtype")
    require(new_rows.is_contiguous() and cache.is_contiguous(), "rows and cache must be contiguous")
    require(new_rows.dim() == 2 and new_rows.shape[1] == 512 and cache.dim() == 4 and cache.shape[2:] == (1, 512),
            "expected new_rows [T, 512] and cache [BLOCKS, PAGE_ROWS, 1, 512]")
    for name, tensor in (("block_table", block_table), ("cu_seqlens_q", cu_seqlens_q), ("seqused_kv", seqused_kv)):
        _check(tensor, torch.int32, name)
    library = _library(library_path()) if "library" not in _entry_points else _entry_points["library"]
    _entry_points["library"] = library
    launch = _entry("launch_sparse_mla_cache_append", 7, 5)
    workspace = torch.empty(1024, dtype=torch.uint8, device=cache.device)
    stream = torch.cuda.current_stream(cache.device).cuda_stream
    _raise_on(launch(stream, new_rows.data_ptr(), cache.data_ptr(), block_table.data_ptr(), cu_seqlens_q.data_ptr(),
                     seqused_kv.data_ptr(), workspace.data_ptr(), block_table.shape[0], new_rows.shape[0],
                     block_table.shape[1], cache.shape[0], cache.shape[1]))
    read = library.read_status_sparse_mla
    read.argtypes, read.restype = [ct.c_void_p, ct.c_void_p, ct.POINTER(ct.c_int32)], ct.c_int
    words = (ct.c_int32 * 8)()
    _raise_on(read(stream, workspace.data_ptr(), words))
    return tuple(words)


def measure(repeats=20):
    """Time both kernels at the benchmark configurations' shapes; returns a list of records.

    Algorithmic bytes: the selection reads every visible score once and writes 2 KiB of indices per
    token; the append reads and writes 1 KiB per row. L2 is evicted before every timed launch.
    """
    import numpy as np

    device = torch.device("cuda")
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=device)
    records = []

    def timed(call):
        times = []
        for _ in range(repeats):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            call()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        return float(np.median(times))

    for name, batches, queries, context in (("decode_b128_q6_ctx128k", 128, 6, 131072), ("prefill_q8k_ctx32k", 1, 8192, 32768)):
        tokens, span = batches * queries, context // 2
        scores = torch.randn((tokens, span), dtype=torch.float32, device=device)
        cu = (torch.arange(batches + 1, dtype=torch.int32, device=device) * queries).contiguous()
        lengths = torch.full((batches,), context // 2, dtype=torch.int32, device=device)
        residual = torch.zeros(batches, dtype=torch.int32, device=device)
        out = torch.empty((tokens, 1, 512), dtype=torch.int32, device=device)
        ms = timed(lambda: topk_indices(scores, cu, lengths, residual, out=out))
        offsets = np.arange(queries)
        visible = np.minimum(context // 2, (context - queries + offsets + 1) // 2).sum() * batches
        algorithmic = int(visible) * 4 + tokens * 2048
        records.append({"kernel": "topk_select_kernel", "workload": name, "tokens": tokens, "ms": ms,
                        "algorithmic_bytes": algorithmic, "GB_s": algorithmic / ms / 1e6})
        del scores
    rows = 8192
    new = torch.randn((rows, 512), device=device).to(torch.bfloat16)
    cache = torch.empty((1024, 128, 1, 512), dtype=torch.bfloat16, device=device)
    table = torch.randperm(1024, device=device).to(torch.int32).view(1, 1024).contiguous()
    cu = torch.tensor([0, rows], dtype=torch.int32, device=device)
    lengths = torch.tensor([32768], dtype=torch.int32, device=device)
    launch = _entry("launch_sparse_mla_cache_append", 7, 5)
    workspace = torch.empty(1024, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    ms = timed(lambda: _raise_on(launch(stream, new.data_ptr(), cache.data_ptr(), table.data_ptr(), cu.data_ptr(),
                                        lengths.data_ptr(), workspace.data_ptr(), 1, rows, 1024, 1024, 128)))
    records.append({"kernel": "cache_append_kernel", "workload": "8192 rows into a 32768-token cache", "tokens": rows,
                    "ms": ms, "algorithmic_bytes": rows * 2048, "GB_s": rows * 2048 / ms / 1e6})
    return records


if __name__ == "__main__":
    import json

    for record in measure():
        print(json.dumps(record))
