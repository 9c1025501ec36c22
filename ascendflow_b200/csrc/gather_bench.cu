// Stand-alone row-gather experiment: the CUDA counterpart of the reference's isolated gather
// study (benchmarks/attention/gather_dma.py with references/ascendc/ascendc_gather2.asc.in):
// per query token, TopK=512 rows of 512 16-bit features are gathered from a paged cache, either
// through the page table ("lookup") or from pre-resolved physical row ids ("physical"), with
// the same 16-byte cp.async / 128-byte-swizzled shared tiles the attention kernel uses. In check
// mode the gathered rows are written back out so that the host can compare them bit for bit
// (gather_dma.py:170-198); in timing mode the tiles are dropped after landing.
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kTopK = 512, kRowBytes = 1024, kTileRows = 64, kTileBytes = kTileRows * kRowBytes;

__device__ __forceinline__ uint32_t swizzled(int row, int unit) {
  return (unit >> 3) * (kTileRows * 128) + row * 128 + (((unit & 7) ^ (row & 7)) << 4);
}

template <int kDepth>
__global__ void gather_kernel(const char* source, const int32_t* pages, int table_width, int page_rows,
                              const int32_t* indices, const int32_t* physical, int queries_per_request,
                              int tokens, char* out) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ int rows[2][kTopK];
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int unit = threadIdx.x & 63, first_row = threadIdx.x >> 6, row_step = blockDim.x >> 6;
  int local = 0;
  for (int token = blockIdx.x; token < tokens; token += gridDim.x, ++local) {
    int* list = rows[local & 1];
    for (int slot = threadIdx.x; slot < kTopK; slot += blockDim.x) {
      int row;
      if (physical != nullptr) {
        row = physical[(size_t)token * kTopK + slot];
      } else {
        const int index = indices[(size_t)token * kTopK + slot];
        const int request = token / queries_per_request;
        row = index < 0 ? -1 : pages[(size_t)request * table_width + index / page_rows] * page_rows + index % page_rows;
      }
      list[slot] = row;
    }
    __syncthreads();
    constexpr int kTiles = kTopK / kTileRows;
    for (int tile = 0; tile < kTiles + kDepth - 1; ++tile) {
      if (tile < kTiles) {
        const uint32_t stage = base + (tile % kDepth) * kTileBytes;
        for (int r = first_row; r < kTileRows; r += row_step) {
          const int row = list[tile * kTileRows + r];
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(stage + swizzled(r, unit)),
                       "l"(source + (size_t)(row < 0 ? 0 : row) * kRowBytes + unit * 16), "r"(row >= 0 ? 16 : 0));
        }
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
      asm volatile("cp.async.wait_group %0;\n" ::"n"(kDepth - 1) : "memory");
      __syncthreads();
      const int landed = tile - (kDepth - 1);
      if (landed >= 0 && out != nullptr) {
        const unsigned char* stage = smem + (landed % kDepth) * kTileBytes;
        for (int r = first_row; r < kTileRows; r += row_step)
          *reinterpret_cast<uint4*>(out + ((size_t)token * kTopK + landed * kTileRows + r) * kRowBytes + unit * 16) =
              *reinterpret_cast<const uint4*>(stage + swizzled(r, unit));
      }
      __syncthreads();
    }
  }
}

}  // namespace

// Returns 0 on success. `physical` NULL selects page-table lookup. `out` NULL selects timing mode.
// depth: tiles in flight (1..3); threads: 128..1024, a multiple of 64.
extern "C" int launch_gather_experiment(void* stream, const void* source, const void* pages, int64_t table_width,
                                        int64_t page_rows, const void* indices, const void* physical,
                                        int64_t queries_per_request, int64_t tokens, void* out, int64_t threads,
                                        int64_t depth, int64_t blocks) {
  if (tokens <= 0 || threads < 128 || threads > 1024 || threads % 64 || depth < 1 || depth > 3 || blocks <= 0) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto run = [&](auto kernel) -> int {
    cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(depth) * kTileBytes);
    if (error != cudaSuccess) return int(error);
    kernel<<<int(blocks), int(threads), int(depth) * kTileBytes, s>>>(
        static_cast<const char*>(source), static_cast<const int32_t*>(pages), int(table_width), int(page_rows),
        static_cast<const int32_t*>(indices), static_cast<const int32_t*>(physical), int(queries_per_request),
        int(tokens), static_cast<char*>(out));
    return int(cudaGetLastError());
  };
  if (depth == 1) return run(gather_kernel<1>);
  if (depth == 2) return run(gather_kernel<2>);
  return run(gather_kernel<3>);
}
