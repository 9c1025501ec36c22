// Shared definitions of the sparse MLA kernels: launch parameters, per-token causal
// geometry and the slot -> physical cache row resolution.
//
// Geometry follows the reference's device routine `query_metadata`
// (examples/sparse_attention/gather.py:9-35), its compressed cutoff
// (examples/sparse_attention/attention.py:339-341) and the row selection of its oracle
// (benchmarks/attention/sparse_reference.py:107-124): index ranks [0, min(TOPK, C, cutoff))
// are examined, the list ends at the first negative index, indices >= cutoff are dropped,
// duplicates are kept.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace sparse_mla {

constexpr int kHeads = 64;
constexpr int kFeatures = 512;
constexpr int kWindow = 128;
constexpr int kTopK = 512;
constexpr int kSlots = kWindow + kTopK;  // 640
constexpr int kPage = 128;
constexpr int kRowBytes = kFeatures * 2;  // one latent row, 16-bit elements

constexpr int kStatusWords = 8;
constexpr int kStatusOk = 0;
constexpr int kStatusBadPage = 1;
constexpr int kStatusWaitExpired = 2;

// Workspace layout (bytes): [0, 512) status block; the rest of the 1024 bytes is reserved.
constexpr int kWorkspaceStatusOffset = 0;
constexpr int kWorkspaceBytes = 1024;

struct Params {
  const void* q;             // [T, 64, 512] 16-bit
  const void* ori_kv;        // [ori_rows, 512]
  const void* cmp_kv;        // [cmp_rows, 512]
  const int32_t* indices;    // [T, 512]
  const int32_t* ori_table;  // [B, pages]
  const int32_t* cmp_table;  // [B, pages]
  const int32_t* cu;         // [B + 1]
  const int32_t* seq_ori;    // [B]
  const int32_t* seq_cmp;    // [B]
  const int32_t* residual;   // [B]
  const int32_t* topk_len;   // [T]
  const float* sinks;        // [64]
  void* out;                 // [T, 64, 512] 16-bit
  int32_t* status;           // kStatusWords
  int32_t batches;           // B
  int32_t tokens;            // T
  int32_t pages;             // block-table width
  int32_t cmp_page;          // rows of one compressed page: 128 / ratio
  int32_t ratio;             // 1 or 2
  int32_t ori_blocks;
  int32_t cmp_blocks;
  float scale_log2;          // 512^-0.5 * log2(e)
  int32_t token_group;       // consecutive tokens a persistent block takes per round (>= 1)
};

struct TokenGeometry {
  int batch;
  int right;    // exclusive right edge of the raw window
  int visible;  // raw window rows kept
  int cutoff;   // exclusive bound on compressed indices
  int bound;    // index ranks examined
};

__device__ __forceinline__ TokenGeometry token_geometry(const Params& p, int token) {
  // batch = upper_bound(cu, token) - 1; empty requests (equal neighbours) are skipped over.
  int lo = 0, hi = p.batches;  // invariant: cu[lo] <= token < cu[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (__ldg(p.cu + mid) <= token) lo = mid; else hi = mid;
  }
  TokenGeometry g;
  g.batch = lo;
  const int begin = __ldg(p.cu + lo);
  const int count = __ldg(p.cu + lo + 1) - begin;
  const int offset = token - begin;
  const int length = __ldg(p.seq_ori + lo);
  g.right = max(0, length - count + offset + 1);
  g.visible = min(kWindow, g.right);
  const int requested = __ldg(p.topk_len + token);
  if (requested > 0) g.visible = min(g.visible, requested);
  const int available = __ldg(p.seq_cmp + lo);
  const int completed = available * p.ratio + __ldg(p.residual + lo);
  g.cutoff = max(0, completed - count + offset + 1) / p.ratio;
  g.bound = min(min(kTopK, available), g.cutoff);
  return g;
}

__device__ __forceinline__ void report(const Params& p, int code, int token, int detail) {
  if (atomicCAS(p.status, kStatusOk, code) == kStatusOk) {
    p.status[1] = token;
    p.status[2] = detail;
  }
}

// Raw window slot -> physical row of ori_kv, or -1.
__device__ __forceinline__ int resolve_window_slot(const Params& p, const TokenGeometry& g,
                                                   int token, int slot) {
  if (slot >= g.visible) return -1;
  const int position = g.right - g.visible + slot;
  const int column = position / kPage;
  if (column >= p.pages) { report(p, kStatusBadPage, token, slot); return -1; }
  const int page = __ldg(p.ori_table + (size_t)g.batch * p.pages + column);
  if ((unsigned)page >= (unsigned)p.ori_blocks) { report(p, kStatusBadPage, token, slot); return -1; }
  return page * kPage + position % kPage;
}

// Compressed index rank -> physical row of cmp_kv, or -1. `first_negative` is the rank of the
// first negative entry of this token's index list (kTopK when there is none).
__device__ __forceinline__ int resolve_compressed_rank(const Params& p, const TokenGeometry& g,
                                                       int token, int rank, int index,
                                                       int first_negative) {
  if (rank >= g.bound || rank >= first_negative || index >= g.cutoff) return -1;
  const int column = index / p.cmp_page;
  if (column >= p.pages) { report(p, kStatusBadPage, token, kWindow + rank); return -1; }
  const int page = __ldg(p.cmp_table + (size_t)g.batch * p.pages + column);
  if ((unsigned)page >= (unsigned)p.cmp_blocks) { report(p, kStatusBadPage, token, kWindow + rank); return -1; }
  return page * p.cmp_page + index % p.cmp_page;
}

// Block-wide resolution of all 640 slots of `token` into shared memory `rows[kSlots]`.
// `scratch` is one shared int. Every thread of the block must call it. Returns the geometry.
// Ends with a __syncthreads(), so `rows` is readable by all threads on return.
__device__ __forceinline__ TokenGeometry resolve_token_rows(const Params& p, int token,
                                                            int* rows, int* scratch) {
  const TokenGeometry g = token_geometry(p, token);
  if (threadIdx.x == 0) *scratch = kTopK;
  __syncthreads();
  const int32_t* list = p.indices + (size_t)token * kTopK;
  int local = kTopK;
  for (int rank = threadIdx.x; rank < kTopK; rank += blockDim.x)
    if (__ldg(list + rank) < 0) { local = rank; break; }
  if (local < kTopK) atomicMin(scratch, local);
  __syncthreads();
  const int first_negative = *scratch;
  for (int slot = threadIdx.x; slot < kSlots; slot += blockDim.x) {
    rows[slot] = slot < kWindow
        ? resolve_window_slot(p, g, token, slot)
        : resolve_compressed_rank(p, g, token, slot - kWindow, __ldg(list + slot - kWindow),
                                  first_negative);
  }
  __syncthreads();
  return g;
}

}  // namespace sparse_mla
