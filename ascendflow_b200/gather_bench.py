"""Isolated row-gather experiment on B200 (counterpart of the reference's gather study).

    python -m ascendflow_b200.gather_bench [--requests 128] [--queries 4]

The reference measures, apart from attention, how fast TopK=512 rows of a paged 128K-context
cache can be gathered per query, with page-table lookup or pre-resolved physical ids
(`benchmarks/attention/gather_dma.py`, inputs at `:44-55`, row check at `:170-198`, reported as
`logical_kv_read_GB_s` at `:355-359`). This does the same with the attention kernel's gather
mechanism (16-byte cp.async into swizzled shared tiles), checks the rows bit for bit in a
separate pass, and prints one JSON line per variant.
"""

from __future__ import annotations

import argparse
import ctypes as ct
import json
import subprocess
from pathlib import Path

import numpy as np

from .build import FLAGS, PACKAGE, nvcc
from .diagnostics import ErrorKind, require

SOURCE = PACKAGE / "csrc" / "gather_bench.cu"
LIBRARY = PACKAGE / "lib" / "libgather_experiment_sm100a.so"
TOPK, FEATURES, TABLE, PAGE_ROWS = 512, 512, 1024, 64


def build():
    if LIBRARY.exists() and LIBRARY.stat().st_mtime >= SOURCE.stat().st_mtime:
        return LIBRARY
    compiler = nvcc()
    require(compiler is not None, "nvcc not found", kind=ErrorKind.RESOURCE)
    LIBRARY.parent.mkdir(parents=True, exist_ok=True)
    result = subprocess.run([compiler, *FLAGS, "-o", str(LIBRARY), str(SOURCE)], capture_output=True, text=True)
    require(result.returncode == 0, "nvcc failed:\n" + result.stderr[-2000:], kind=ErrorKind.RESOURCE)
    return LIBRARY


def inputs(requests, queries, context=131072, seed=4102026):
    """Per-request page permutations and sorted distinct causal indices, as the reference draws them."""
    rng = np.random.default_rng(seed)
    pages = np.stack([rng.permutation(TABLE) + b * TABLE for b in range(requests)]).astype(np.int32)
    indices = np.stack([
        np.sort(rng.choice((context - queries + token % queries + 1) // 2, TOPK, replace=False))
        for token in range(requests * queries)]).astype(np.int32)
    batch = np.arange(requests * queries) // queries
    physical = pages[batch[:, None], indices // PAGE_ROWS] * PAGE_ROWS + indices % PAGE_ROWS
    return pages, indices, physical.astype(np.int32)


def launcher():
    library = ct.CDLL(str(build()))
    launch = library.launch_gather_experiment
    launch.argtypes = [ct.c_void_p, ct.c_void_p, ct.c_void_p, ct.c_int64, ct.c_int64, ct.c_void_p, ct.c_void_p,
                       ct.c_int64, ct.c_int64, ct.c_void_p, ct.c_int64, ct.c_int64, ct.c_int64]
    launch.restype = ct.c_int
    return launch


def run(requests=128, queries=4, threads=(256, 512), depths=(2, 3), repeats=20):
    import torch

    launch = launcher()
    device = torch.device("cuda")
    pages_h, indices_h, physical_h = inputs(requests, queries)
    rows_total = requests * TABLE * PAGE_ROWS
    source = torch.empty((rows_total, FEATURES), dtype=torch.int16, device=device)
    words = source.view(torch.int32)  # [rows, 256]: every word identifies its row and column
    column = torch.arange(FEATURES // 2, dtype=torch.int32, device=device)[None, :]
    for first in range(0, rows_total, 1 << 20):
        last = min(rows_total, first + (1 << 20))
        words[first:last] = torch.arange(first, last, dtype=torch.int32, device=device)[:, None] * 257 + column
    pages, indices, physical = (torch.from_numpy(a).to(device) for a in (pages_h, indices_h, physical_h))
    tokens = requests * queries
    stream = torch.cuda.current_stream().cuda_stream
    blocks = torch.cuda.get_device_properties(device).multi_processor_count
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=device)
    records = []
    for address in ("lookup", "physical"):
        ids = physical.data_ptr() if address == "physical" else None
        # correctness pass on a slice, separate from timing
        check = min(tokens, 32)
        out = torch.zeros((check, TOPK, FEATURES), dtype=torch.int16, device=device)
        status = launch(stream, source.data_ptr(), pages.data_ptr(), TABLE, PAGE_ROWS, indices.data_ptr(), ids,
                        queries, check, out.data_ptr(), 256, 2, blocks)
        require(status == 0, f"gather launch failed with status {status}")
        expected = source[torch.from_numpy(physical_h[:check].astype(np.int64)).to(device)]
        exact = bool(torch.equal(out, expected))
        for count in threads:
            for depth in depths:
                times = []
                for _ in range(repeats):
                    flush.zero_()
                    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    status = launch(stream, source.data_ptr(), pages.data_ptr(), TABLE, PAGE_ROWS, indices.data_ptr(),
                                    ids, queries, tokens, None, count, depth, blocks)
                    end.record()
                    require(status == 0, f"gather launch failed with status {status}")
                    torch.cuda.synchronize()
                    times.append(start.elapsed_time(end))
                median = float(np.median(times))
                records.append({"address": address, "threads": count, "tiles_in_flight": depth, "rows_exact": exact,
                                "ms": median, "logical_kv_read_GB_s": tokens * TOPK * FEATURES * 2 / median / 1e6,
                                "requests": requests, "queries_per_request": queries})
    return records


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--requests", type=int, default=128)
    parser.add_argument("--queries", type=int, default=4)
    args = parser.parse_args()
    for record in run(args.requests, args.queries):
        print(json.dumps(record))


if __name__ == "__main__":
    main()
