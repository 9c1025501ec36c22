// The two steps next to the attention operator whose output format the operator fixes: choosing
// each query token's TopK compressed rows from index scores (the producer of
// `cmp_sparse_indices`), and appending a call's new raw rows to the paged cache (the producer
// of `ori_kv`). The reference leaves both to its caller (docs/operators/sparse-mla.md:8,
// 263-266: "indexer, compressor, projections and cache writes are provided by the caller"), so
// there is no reference implementation to match: the contracts below are derived from what the
// operator reads (docs/operators/sparse-mla.md:62-87) and pinned by this repository's oracle.
// Both are byte/integer work bound by memory traffic.

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sparse_mla.h"
#include "sparse_mla_common.cuh"

namespace sparse_mla {
namespace {

constexpr int kSelectThreads = 512;
constexpr int kSelectWarps = kSelectThreads / 32;

// Monotone map of a finite FP32 value to an unsigned key: larger value, larger key.
__device__ __forceinline__ uint32_t score_key(float value) {
  const uint32_t bits = __float_as_uint(value);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// One block per query token (blocks stride over tokens). Candidates are compressed rows
// [0, min(available, cutoff)): the rows the attention kernel would accept for this token. The
// min(TopK, candidates) highest scores win, ties going to the lower index; winners are written in
// ascending index order, the rest of the 512 entries is -1.
//
// More candidates than TopK: an MSB-first radix select over the keys (four 8-bit digits, one
// histogram per warp, one addition per warp and bin, so that the exponent digit's few hot bins
// do not serialise anything)
// finds the key of the TopK-th highest score and how many entries equal to it are taken; one more
// pass in index order writes the winners through a block-wide prefix count.
struct SelectParams {
  const float* scores;       // [T, span]
  const int32_t* cu;         // [B + 1]
  const int32_t* seq_cmp;    // [B]
  const int32_t* residual;   // [B]
  int32_t* out;              // [T, 512]
  int32_t batches, tokens, ratio;
  int64_t span;
};

// Completed compressed rows a token may see: min(C, cutoff), with the attention operator's
// cutoff = max(0, C R + r - n + j + 1) / R (examples/sparse_attention/attention.py:339-341).
__device__ __forceinline__ int visible_compressed_rows(const SelectParams& p, int token) {
  int lo = 0, hi = p.batches;  // invariant: cu[lo] <= token < cu[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(p.cu + mid) <= token) lo = mid; else hi = mid;
  }
  const int begin = __ldg(p.cu + lo), count = __ldg(p.cu + lo + 1) - begin;
  const int available = __ldg(p.seq_cmp + lo);
  const int completed = available * p.ratio + __ldg(p.residual + lo);
  return min(available, max(0, completed - count + (token - begin) + 1) / p.ratio);
}

// Four consecutive scores per thread and step (16-byte loads, two in flight); `span` is a
// multiple of four, so every row starts on a 16-byte boundary.
__device__ __forceinline__ void load_keys(const float* row, int i, int candidates, uint32_t (&key)[4], bool (&valid)[4]) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i < candidates) v = __ldg(reinterpret_cast<const float4*>(row + i));  // may run past `candidates`, never past the row
  key[0] = score_key(v.x); key[1] = score_key(v.y); key[2] = score_key(v.z); key[3] = score_key(v.w);
#pragma unroll
  for (int e = 0; e < 4; ++e) valid[e] = i + e < candidates;
}

__global__ void __launch_bounds__(kSelectThreads) topk_select_kernel(const SelectParams p) {
  __shared__ unsigned histogram[kSelectWarps][256];
  __shared__ unsigned totals[256];
  __shared__ unsigned long long warp_count[kSelectWarps], base_count;
  __shared__ unsigned prefix_key, wanted;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kStep = kSelectThreads * 4;
  constexpr int kInFlight = 2;  // 16-byte loads in flight per thread in the counting passes (four: slower)
  for (int token = blockIdx.x; token < p.tokens; token += gridDim.x) {
    const int candidates = int(min((int64_t)visible_compressed_rows(p, token), p.span));
    const int take = min(kTopK, candidates);
    int32_t* list = p.out + (size_t)token * kTopK;
    const float* row = p.scores + (size_t)token * p.span;
    __syncthreads();  // the shared words of the previous token are no longer read
    if (candidates <= kTopK) {
      for (int i = threadIdx.x; i < kTopK; i += blockDim.x) list[i] = i < candidates ? i : -1;
      continue;
    }
    // ---- radix select: key of the take-th highest score ------------------------------------
    if (threadIdx.x == 0) { prefix_key = 0; wanted = unsigned(take); }
    for (int digit = 3; digit >= 0; --digit) {
      const int shift = digit * 8;
      for (int i = threadIdx.x; i < kSelectWarps * 256; i += blockDim.x) (&histogram[0][0])[i] = 0;
      __syncthreads();
      const unsigned prefix = prefix_key;
      const unsigned mask = digit == 3 ? 0u : (0xffffffffu << (shift + 8));
      // Lanes that fall into the same bin (most of them, for the exponent digit) add once,
      // through their lowest lane.
      for (int first = 0; first < candidates; first += kInFlight * kStep) {
        uint32_t key[kInFlight][4];
        bool valid[kInFlight][4];
#pragma unroll
        for (int h = 0; h < kInFlight; ++h) load_keys(row, first + h * kStep + threadIdx.x * 4, candidates, key[h], valid[h]);
#pragma unroll
        for (int h = 0; h < kInFlight; ++h)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const bool counted = valid[h][e] && (key[h][e] & mask) == prefix;
            // from the second digit on, most warps hold no entry with the prefix: nothing to vote on
            if (__ballot_sync(0xffffffffu, counted) == 0u) continue;
            const unsigned bin = counted ? (key[h][e] >> shift) & 255u : 256u;
            const unsigned peers = __match_any_sync(0xffffffffu, bin);
            if (counted && lane == __ffs(peers) - 1) atomicAdd(&histogram[warp][bin], unsigned(__popc(peers)));
          }
      }
      __syncthreads();
      if (threadIdx.x < 256) {
        unsigned sum = 0;
#pragma unroll
        for (int w = 0; w < kSelectWarps; ++w) sum += histogram[w][threadIdx.x];
        totals[threadIdx.x] = sum;
      }
      __syncthreads();
      if (threadIdx.x == 0) {  // walk down from the highest bin until `wanted` entries are covered
        unsigned above = 0;
        int bin = 255;
        while (bin > 0 && above + totals[bin] < wanted) above += totals[bin--];
        prefix_key = prefix | (unsigned(bin) << shift);
        wanted -= above;  // entries still to take among those that share the longer prefix
      }
      __syncthreads();
    }
    const unsigned threshold = prefix_key, equal_taken = wanted;  // wanted >= 1
    // ---- winners in index order -------------------------------------------------------------
    // Counts are packed: entries above the threshold in the low half, entries equal to it in the
    // high half of a 64-bit word.
    if (threadIdx.x == 0) base_count = 0;
    __syncthreads();
    for (int first = 0; first < candidates; first += kStep) {
      const int i = first + threadIdx.x * 4;
      uint32_t key[4];
      bool valid[4];
      load_keys(row, i, candidates, key, valid);
      unsigned long long mine = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (valid[e]) mine += key[e] > threshold ? 1ull : (key[e] == threshold ? (1ull << 32) : 0ull);
      unsigned long long scan = mine;  // inclusive scan over the warp
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, scan, d);
        if (lane >= d) scan += up;
      }
      if (lane == 31) warp_count[warp] = scan;
      __syncthreads();
      unsigned long long before = base_count + scan - mine;
      for (int w = 0; w < warp; ++w) before += warp_count[w];
      unsigned greater_before = unsigned(before), equal_before = unsigned(before >> 32);
      // An entry equal to the threshold is a winner while fewer than `equal_taken` such entries
      // precede it; every winner's position is the number of winners before it.
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (!valid[e]) continue;
        if (key[e] > threshold) {
          list[greater_before + min(equal_before, equal_taken)] = i + e;
          ++greater_before;
        } else if (key[e] == threshold) {
          if (equal_before < equal_taken) list[greater_before + equal_before] = i + e;
          ++equal_before;
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned long long add = 0;
        for (int w = 0; w < kSelectWarps; ++w) add += warp_count[w];
        base_count += add;
      }
      __syncthreads();
    }
    for (int i = take + threadIdx.x; i < kTopK; i += blockDim.x) list[i] = -1;
  }
}

// One warp per new row: token j of n of request b goes to logical position L_b - n + j of the raw
// cache (L_b includes this call's tokens, as `seqused_ori_kv` does for the attention operator),
// i.e. to row `position % rows_per_page` of page `table[b][position / rows_per_page]`.
__global__ void cache_append_kernel(const char* new_rows, char* cache, const int32_t* table, const int32_t* cu,
                                    const int32_t* lengths, int batches, int tokens, int pages, int blocks,
                                    int page_rows, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int token = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; token < tokens; token += warps) {
    int lo = 0, hi = batches;  // invariant: cu[lo] <= token < cu[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(cu + mid) <= token) lo = mid; else hi = mid;
    }
    const int begin = __ldg(cu + lo), count = __ldg(cu + lo + 1) - begin;
    const int position = __ldg(lengths + lo) - count + (token - begin);
    const int column = position / page_rows;
    const int page = position >= 0 && column < pages ? __ldg(table + (size_t)lo * pages + column) : -1;
    if (position < 0 || (unsigned)page >= (unsigned)blocks) {  // nowhere to put it: reported, not written
      if (lane == 0 && atomicCAS(status, kStatusOk, kStatusBadPage) == kStatusOk) { status[1] = token; status[2] = position; }
      continue;
    }
    const uint4* source = reinterpret_cast<const uint4*>(new_rows + (size_t)token * kRowBytes);
    uint4* target = reinterpret_cast<uint4*>(cache + ((size_t)page * page_rows + position % page_rows) * kRowBytes);
    target[lane] = __ldg(source + lane);
    target[lane + 32] = __ldg(source + lane + 32);
  }
}

}  // namespace
}  // namespace sparse_mla

using namespace sparse_mla;

extern "C" {

int launch_sparse_mla_topk_indices(void* stream, void* arg_scores, void* arg_cu_seqlens_q, void* arg_seqused_cmp_kv,
                                   void* arg_cmp_residual_kv, void* arg_cmp_sparse_indices, int64_t B, int64_t T,
                                   int64_t SPAN, int64_t CMP_PAGE) {
  if (B <= 0 || T <= 0 || SPAN <= 0 || B > INT32_MAX || T > INT32_MAX || SPAN > INT32_MAX - 8192 || SPAN % 4 != 0) return -1;
  if (CMP_PAGE != 64 && CMP_PAGE != 128) return -1;
  SelectParams p = {};
  p.scores = static_cast<const float*>(arg_scores);
  p.cu = static_cast<const int32_t*>(arg_cu_seqlens_q);
  p.seq_cmp = static_cast<const int32_t*>(arg_seqused_cmp_kv);
  p.residual = static_cast<const int32_t*>(arg_cmp_residual_kv);
  p.out = static_cast<int32_t*>(arg_cmp_sparse_indices);
  p.batches = int32_t(B); p.tokens = int32_t(T); p.ratio = int32_t(kPage / CMP_PAGE);
  p.span = SPAN;
  int device = 0, multiprocessors = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&multiprocessors, cudaDevAttrMultiProcessorCount, device);
  const int64_t cap = int64_t(multiprocessors) * 4;
  topk_select_kernel<<<int(T < cap ? T : cap), kSelectThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return int(cudaGetLastError());
}

int launch_sparse_mla_cache_append(void* stream, void* arg_new_rows, void* arg_cache, void* arg_block_table,
                                   void* arg_cu_seqlens_q, void* arg_seqused_kv, void* npu_workspace, int64_t B,
                                   int64_t T, int64_t PAGES, int64_t BLOCKS, int64_t PAGE_ROWS) {
  if (B <= 0 || T <= 0 || PAGES <= 0 || BLOCKS < 0 || npu_workspace == nullptr) return -1;
  if (PAGE_ROWS != 64 && PAGE_ROWS != 128) return -1;
  if (B > INT32_MAX || T > INT32_MAX || PAGES > INT32_MAX || BLOCKS > INT32_MAX / kPage) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int status = int(cudaMemsetAsync(npu_workspace, 0, kWorkspaceBytes, s))) return status;
  const int64_t blocks = (T + 7) / 8;  // eight warps = eight rows per block
  cache_append_kernel<<<int(blocks), 256, 0, s>>>(
      static_cast<const char*>(arg_new_rows), static_cast<char*>(arg_cache), static_cast<const int32_t*>(arg_block_table),
      static_cast<const int32_t*>(arg_cu_seqlens_q), static_cast<const int32_t*>(arg_seqused_kv), int(B), int(T), int(PAGES),
      int(BLOCKS), int(PAGE_ROWS),
      reinterpret_cast<int32_t*>(static_cast<char*>(npu_workspace) + kWorkspaceStatusOffset));
  return int(cudaGetLastError());
}

}  // extern "C"
