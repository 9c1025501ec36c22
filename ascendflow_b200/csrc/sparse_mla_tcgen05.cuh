// Sparse MLA attention on the Blackwell tensor path: tcgen05.mma with operands and accumulators
// in tensor memory, warp-specialised and software-pipelined. BF16 or FP16 storage (template
// parameter kFormat), FP32 accumulation.
//
// One persistent block per SM owns one query token at a time (64 heads x 512 features) and
// walks the token's live 64-row chunks (window rows first, then the compressed ranks in list
// order, as the reference does: examples/sparse_attention/attention.py:42-64, 147-207). The
// chunks of all the block's tokens form one stream; the issue order is QK(c + 1), PV(c).
//
//   resolver warp    resolves slot -> physical row (sparse_mla_common.cuh) up to two tokens ahead.
//   producer warps   gather the token's rows with 16-byte cp.async into a three-stage ring of
//                    128-byte-swizzled shared tiles (a row is fetched once and serves as K and
//                    V), and move the token's Q from global to tensor memory through registers.
//   MMA warp         one thread issues S = Q X^T (Q from tensor memory, X K-major from the tile)
//                    and O += P X (P from a shared tile, X MN-major from the same tile; issued
//                    as tcgen05.mma.ws so that M = 64 does not halve the rate).
//   softmax warps    tcgen05.ld S, joint online softmax with the per-head sink
//                    (examples/sparse_attention/attention.py:398-490: one maximum and one
//                    denominator over window, compressed rows and sink; P rounded to the storage
//                    type before PV, denominator from unrounded FP32), P to shared memory, O
//                    rescaled only when the running maximum moved by more than 2^8, final
//                    normalisation and store (after the next token's first chunk).
//
// Tensor memory (512 columns x 128 lanes), all of it in use:
//   columns   0-255  O: two weight-stationary M = 64, N = 256 accumulators (columns 0-127: features
//                    0-255, columns 128-255: features 256-511). Lane l holds head l % 64 and,
//                    of each accumulator, features 128 (l / 64) .. + 127.
//   columns 256-383  Q as 16-bit pairs, same split: lanes 0-15 hold Q[:, 0:256] of 16 heads, lanes
//                    16-31 hold Q[:, 256:512] of the same heads.
//   columns 384-511  the score buffer of the stacked QK product (see `issue_qk`): a low-half lane
//                    finds its partial scores in columns 0-63, a high-half lane in columns 64-127.
// Thread (lane & 15) + 16 * half of softmax warp w owns head 16 w + (lane & 15) of that half; the
// two lanes of a head add their partial scores with one shuffle per score and split the 64 rows
// of the chunk between them.
//
// Every wait on an mbarrier is bounded (tcgen05_ptx.cuh): on expiry the block records
// kStatusWaitExpired, all roles leave their loops, tensor memory is released, the kernel returns.
#pragma once

#include <cuda_bf16.h>
#include <type_traits>
#include <cuda_fp16.h>

#include "sparse_mla_common.cuh"
#include "tcgen05_ptx.cuh"

namespace sparse_mla {
namespace umma {

using namespace sm100;

constexpr int kSoftmaxWarps = 4;
constexpr int kProducerWarps = 8;
constexpr int kMmaWarp = kSoftmaxWarps;                     // warp index 4
constexpr int kResolverWarp = kSoftmaxWarps + 1;            // warp index 5
constexpr int kFirstProducerWarp = kSoftmaxWarps + 2;
constexpr int kPvWarp = kFirstProducerWarp + kProducerWarps;  // warp index 14
constexpr int kThreads = 32 * (kSoftmaxWarps + 3 + kProducerWarps);
constexpr int kProducerThreads = 32 * kProducerWarps;

constexpr int kChunkRows = 64;
constexpr int kMaxChunks = kSlots / kChunkRows;             // 10
constexpr int kStages = 3;
constexpr int kBlockBytes = kChunkRows * 128;               // one 64-feature block of a tile: 8 KiB
constexpr int kTileBytes = 8 * kBlockBytes;                 // 64 rows x 512 features: 64 KiB

// Shared memory map (bytes from a 1024-aligned base).
constexpr int kSmemKv = 0;
// The P tile (64 heads x 64 rows, 8 KiB) and, per softmax warp, 4 KiB of epilogue staging
// (32 x 128-byte rows). Both 1024-byte aligned like the tiles, because the swizzle is a function
// of the address.
constexpr int kSmemP = kSmemKv + kStages * kTileBytes;
constexpr int kSmemStore = kSmemP + kHeads * 128;
constexpr int kSmemRows = kSmemStore + kSoftmaxWarps * 4096;   // int[2][640]
constexpr int kSmemInfo = kSmemRows + 2 * kSlots * 4;       // TokenInfo[2]
constexpr int kSmemBars = kSmemInfo + 2 * 128;              // mbarriers
constexpr int kSmemMisc = kSmemBars + 32 * 8;               // tmem slot, abort flag
// Per-head factors handed between the softmax warps (float[2][64] each, double-buffered): a
// thread works out the softmax of one head but reads the accumulator of another (see below).
constexpr int kSmemAlpha = kSmemMisc + 64;
constexpr int kSmemInverse = kSmemAlpha + 2 * kHeads * 4;
constexpr int kSmemEnd = kSmemInverse + 2 * kHeads * 4;
constexpr int kSmemBytes = kSmemEnd + 1024;  // + slack for the 1024-byte alignment

constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kTmemO = 0;
constexpr uint32_t kTmemQ = 256;
constexpr uint32_t kTmemS = 384;                             // one 128-column score buffer
constexpr uint32_t kTmemOHalf = 128;                         // columns of one 256-feature accumulator
constexpr uint32_t kHalfLanes = 16u << 16;                   // lane offset of the high-half lanes in a tensor-memory address

struct TokenInfo {
  int token;
  int chunks;                 // live chunks of this token
  unsigned char chunk[kMaxChunks];
  unsigned live[kSlots / 32]; // bit l of word i: slot 32 i + l is live
};
static_assert(sizeof(TokenInfo) <= 128, "the info area holds two 128-byte entries");

enum Bar {
  kTokenReady0 = 0, kTokenReady1, kTokenDone0, kTokenDone1, kQFull, kQFree,
  kKvFree0, kKvFree1, kKvFree2,
  kSFull, kPFull, kOFree,
  kKvFull0, kKvFull1, kKvFull2, kSoftmaxSync, kInfoRead0, kInfoRead1, kBarCount
};
static_assert(kBarCount <= 32, "the barrier area holds 32 mbarriers");

// Storage formats of kind::f16 instructions: 0 = IEEE half, 1 = BF16.
template <int kFormat> constexpr uint32_t kIdescQK = idesc_f16(128, 128, kFormat, 0, 0);
template <int kFormat> constexpr uint32_t kIdescPV = idesc_f16(64, 256, kFormat, 0, 1);  // issued as .ws

// Position of 64-feature block b in a tile: blocks b and b + 4 (the same features of the low
// and the high half of a row) are neighbours, so that a K-major operand of 128 "rows" with
// 8-row groups 1024 bytes apart reads rows 0-63 from block b and rows 64-127 from block b + 4.
__host__ __device__ constexpr int block_position(int b) { return (b & 3) * 2 + (b >> 2); }

// Byte offset of 16-byte unit `unit` (0..63) of row `row` in a K-major 128-byte-swizzled tile
// of 64 rows: eight 64-feature blocks of [64 rows x 128 bytes].
__device__ __forceinline__ uint32_t swizzled(int row, int unit) {
  return block_position(unit >> 3) * kBlockBytes + row * 128 + (((unit & 7) ^ (row & 7)) << 4);
}

// The P tile (64 heads x 64 rows of 16-bit probabilities, K-major, 128-byte swizzle: one
// 128-byte row per head): byte offset of 16-byte unit `unit` (0..7) of head `head` from kSmemP.
__device__ __forceinline__ uint32_t p_offset(int head, int unit) {
  return head * 128 + ((unit ^ (head & 7)) << 4);
}

struct Shared {
  uint32_t base;        // shared-space address of the 1024-aligned region
  unsigned char* ptr;   // generic pointer to the same
  __device__ __forceinline__ uint32_t bar(int which) const { return base + kSmemBars + which * 8; }
  __device__ __forceinline__ int* rows(int buffer) const {
    return reinterpret_cast<int*>(ptr + kSmemRows) + buffer * kSlots;
  }
  __device__ __forceinline__ TokenInfo* info(int buffer) const {
    return reinterpret_cast<TokenInfo*>(ptr + kSmemInfo + buffer * 128);
  }
  __device__ __forceinline__ volatile int* abort_flag() const {
    return reinterpret_cast<volatile int*>(ptr + kSmemMisc + 4);
  }
};

// The tokens of one persistent block, in order. Blocks take `group` consecutive tokens per round
// (round r, block b: tokens (r * grid + b) * group ...), so that a block's successive tokens
// share most of their window rows in L2 while different blocks read different windows at any one
// time. Every role of a block walks the same sequence.
struct TokenWalk {
  int block, grid, group, tokens, k;
  __device__ __forceinline__ explicit TokenWalk(const Params& p)
      : block(blockIdx.x), grid(gridDim.x), group(p.token_group), tokens(p.tokens), k(0) {}
  __device__ __forceinline__ int next() {  // next token of this block, or -1 when done
    while (true) {
      const int round = k / group;
      if ((long long)round * grid * group >= tokens) return -1;
      const long long token = ((long long)round * grid + block) * group + k % group;
      ++k;
      if (token < tokens) return int(token);
    }
  }
  __device__ __forceinline__ int peek() const { TokenWalk copy = *this; return copy.next(); }
  __device__ __forceinline__ int count() const {  // how many tokens next() hands out in all
    const int per_round = grid * group;  // at most the SM count times eight
    const int rounds = tokens / per_round, rest = tokens - rounds * per_round - block * group;
    return rounds * group + (rest < 0 ? 0 : (rest > group ? group : rest));
  }
};

// A wait whose outcome is uniform across the calling warp (all 32 lanes must call it).
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}

// ---- producer warps ---------------------------------------------------------------------------

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool live) {
  // A masked slot is zero-filled (source size 0) so the tile never holds non-finite leftovers.
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(live ? 16 : 0));
}

// Arrive on `bar` once all cp.async copies this thread has issued so far have completed. The
// arrival counts towards the barrier's expected count (no pending-count increment).
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}

// Warp-cooperative form of `token_geometry`: the request search probes 32 positions of
// cu_seqlens_q per step instead of one, and every other per-token scalar is loaded before the
// search so that the loads overlap (a cold block starts with this chain on its critical path).
__device__ __forceinline__ TokenGeometry token_geometry_warp(const Params& p, int token, int lane) {
  const int requested = __ldg(p.topk_len + token);
  int lo = 0, hi = p.batches;  // invariant: cu[lo] <= token < cu[hi]
  while (hi - lo > 1) {
    const int step = (hi - lo + 31) >> 5;
    const int probe = lo + lane * step;
    const bool below = probe < hi && __ldg(p.cu + probe) <= token;
    const unsigned mask = __ballot_sync(0xffffffffu, below);  // lane 0 probes cu[lo]: always set
    const int last = 31 - __clz(mask);
    lo += last * step;
    hi = min(hi, lo + step);
  }
  TokenGeometry g;
  g.batch = lo;
  const int begin = __ldg(p.cu + lo), end = __ldg(p.cu + lo + 1);
  const int length = __ldg(p.seq_ori + lo), available = __ldg(p.seq_cmp + lo), residual = __ldg(p.residual + lo);
  const int count = end - begin, offset = token - begin;
  g.right = max(0, length - count + offset + 1);
  g.visible = min(kWindow, g.right);
  if (requested > 0) g.visible = min(g.visible, requested);
  g.cutoff = max(0, available * p.ratio + residual - count + offset + 1) / p.ratio;
  g.bound = min(min(kTopK, available), g.cutoff);
  return g;
}

// ---- slot -> physical row, one warp per token -------------------------------------------------
// The selection of the reference's oracle (benchmarks/attention/sparse_reference.py:107-124) and
// of its device routines (examples/sparse_attention/gather.py:39-60, 87-131): window slot s is
// position right - visible + s of the raw cache; compressed rank r is kept when r < min(TOPK,
// C, cutoff), no entry before it is negative and its index is below the cutoff; a kept entry
// goes through the request's block table. Lane l returns slots 32 i + l in resolved[i] (the
// physical cache row, or -1). This one routine serves the attention kernel (its resolver warp)
// and the index-set export (`resolve_rows_kernel`), so that the exported set is the gathered set.
__device__ __forceinline__ void resolve_token_warp(const Params& p, int token, int lane,
                                                   int (&resolved)[kSlots / 32]) {
  // The index list does not depend on the geometry: its loads go out first.
  const int32_t* list = p.indices + (size_t)token * kTopK;
  int index[kTopK / 32];
#pragma unroll
  for (int i = 0; i < kTopK / 32; ++i) index[i] = __ldg(list + i * 32 + lane);
  const TokenGeometry g = token_geometry_warp(p, token, lane);
  int first = kTopK;
#pragma unroll
  for (int i = 0; i < kTopK / 32; ++i)
    if (index[i] < 0 && first == kTopK) first = i * 32 + lane;
  const int first_negative = __reduce_min_sync(0xffffffffu, first);
  const int cmp_shift = p.cmp_page == 64 ? 6 : 7;
  // Three passes so that all block-table loads are in flight together (a branch or vote between
  // them would serialise twenty dependent round trips to memory): columns, loads, rows.
  int column[kSlots / 32], within[kSlots / 32];
#pragma unroll
  for (int i = 0; i < kWindow / 32; ++i) {
    const int slot = i * 32 + lane;
    const int position = g.right - g.visible + slot;
    const bool live = slot < g.visible;
    column[i] = live ? position / kPage : -1;
    within[i] = position % kPage;
  }
#pragma unroll
  for (int i = 0; i < kTopK / 32; ++i) {
    const int rank = i * 32 + lane;
    const bool live = rank < g.bound && rank < first_negative && index[i] < g.cutoff;
    // cmp_page is 64 or 128: shift and mask instead of a run-time division
    column[kWindow / 32 + i] = live ? index[i] >> cmp_shift : -1;
    within[kWindow / 32 + i] = index[i] & (p.cmp_page - 1);
  }
#pragma unroll
  for (int i = 0; i < kSlots / 32; ++i) {
    const int32_t* table = (i < kWindow / 32 ? p.ori_table : p.cmp_table) + (size_t)g.batch * p.pages;
    resolved[i] = __ldg(table + min(max(column[i], 0), p.pages - 1));  // the page, for now
  }
  bool bad = false;
#pragma unroll
  for (int i = 0; i < kSlots / 32; ++i) {
    const bool window = i < kWindow / 32;
    const int blocks = window ? p.ori_blocks : p.cmp_blocks, page_rows = window ? kPage : p.cmp_page;
    const bool live = column[i] >= 0;
    const bool legal = column[i] < p.pages && (unsigned)resolved[i] < (unsigned)blocks;
    bad |= live && !legal;
    resolved[i] = live && legal ? resolved[i] * page_rows + within[i] : -1;
  }
  if (bad) report(p, kStatusBadPage, token, lane);
}

// The gathered index set of every token, written out: one warp per token runs the routine the
// attention kernel's resolver warp runs.
__global__ void resolve_rows_kernel(const Params p, int32_t* out) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int token = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; token < p.tokens; token += warps) {
    int resolved[kSlots / 32];
    resolve_token_warp(p, token, lane, resolved);
#pragma unroll
    for (int i = 0; i < kSlots / 32; ++i) out[(size_t)token * kSlots + i * 32 + lane] = resolved[i];
  }
}

// ---- resolver warp ----------------------------------------------------------------------------
// Runs ahead of everybody else: for each token of this block it resolves the 640 slots into row
// buffer `token_count & 1`, lists the live chunks and publishes both.
__device__ void resolver_role(const Params& p, const Shared& sm) {
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = sm.abort_flag();
  uint32_t token_count = 0;
  TokenWalk walk(p);
  for (int token = walk.next(); token >= 0; token = walk.next(), ++token_count) {
    const int buffer = token_count & 1;
    int* rows = sm.rows(buffer);
    TokenInfo* info = sm.info(buffer);
    // The buffer is free once the softmax warps have finished the token that used it two tokens
    // ago. (Barriers that one role may pass without the others keeping up exist once per buffer:
    // a phase parity can only tell two consecutive phases apart.)
    // ... and once the MMA thread and the producer warps have read its chunk count: for a token
    // with nothing to do the softmax warps finish without waiting for anybody, and a role that
    // fell two publications behind could not tell them apart by parity.
    if (token_count >= 2 &&
        (!warp_wait(sm.bar(kTokenDone0 + buffer), ((token_count >> 1) & 1) ^ 1, abort_flag) ||
         !warp_wait(sm.bar(kInfoRead0 + buffer), ((token_count >> 1) & 1) ^ 1, abort_flag))) return;
    int resolved[kSlots / 32];
    resolve_token_warp(p, token, lane, resolved);
    int live_chunks = 0;  // bit c set: chunk c holds a live slot (same in all lanes)
#pragma unroll
    for (int i = 0; i < kSlots / 32; ++i) {
      rows[i * 32 + lane] = resolved[i];
      const unsigned live = __ballot_sync(0xffffffffu, resolved[i] >= 0);
      if (live != 0) live_chunks |= 1 << (i * 32 / kChunkRows);
      if (lane == 0) info->live[i] = live;
    }
    if (lane == 0) {
      int count = 0;
      for (int chunk = 0; chunk < kMaxChunks; ++chunk)
        if (live_chunks >> chunk & 1) info->chunk[count++] = (unsigned char)chunk;
      info->token = token;
      info->chunks = count;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(sm.bar(kTokenReady0 + buffer));
  }
}

// 8 x 8 transpose of 16-byte elements across the eight lanes of an octet: on entry lane a holds
// element (a, b) ... of row b in words[4 b .. 4 b + 3]; on return it holds element (b, a) there,
// i.e. what lane b held at index a. Three butterfly stages, register indices all static.
__device__ __forceinline__ void transpose_octet(uint32_t* words, int lane) {
#pragma unroll
  for (int m = 1; m < 8; m <<= 1) {
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b & m) continue;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t& low = words[4 * b + w];
        uint32_t& high = words[4 * (b | m) + w];
        const uint32_t send = upper ? low : high;
        const uint32_t got = __shfl_xor_sync(0xffffffffu, send, m);
        if (upper) low = got; else high = got;
      }
    }
  }
}

__device__ void producer_role(const Params& p, const Shared& sm, uint32_t tmem) {
  const int tid = threadIdx.x - kFirstProducerWarp * 32;
  const int lane = tid & 31;
  volatile int* abort_flag = sm.abort_flag();
  const char* window_base = static_cast<const char*>(p.ori_kv);
  const char* compressed_base = static_cast<const char*>(p.cmp_kv);
  // Q goes from global memory to tensor memory through registers, never through the ring. A warp
  // reaches the 32 tensor-memory lanes of subpartition (warp index % 4): two producer warps
  // share each subpartition and take 64 columns (256 bytes of every half row) each. Lane l of a
  // subpartition holds head 16 * subpartition + (l & 15), feature half l >> 4.
  const int warp = threadIdx.x >> 5;
  const int subpartition = warp & 3, part = (warp - kFirstProducerWarp) >> 2;
  // Loads are coalesced: in load j the eight lanes of an octet read 128 contiguous bytes of the
  // half row that belongs to the octet's lane (j & 7); an 8 x 8 transpose by shuffles within
  // the octet then gives every lane its own half row (see `transpose_octet`).
  const size_t q_octet_offset = (size_t)(subpartition * 16 + (lane & 8)) * kRowBytes + (lane >> 4) * 512 + part * 256 + (lane & 7) * 16;
  const uint32_t q_tmem = tmem + kTmemQ + part * 64 + (uint32_t(subpartition * 32) << 16);
  // Ring bookkeeping: stage s is free again once the PV of the tile it held has completed
  // (kKvFree0 + s, committed by the MMA thread). A tile is announced without anybody waiting
  // for it: every producer thread attaches the completion of its own copies to the stage's
  // full barrier (cp.async.mbarrier.arrive), so the threads never block on data in flight and
  // the warps need not stay in step with each other.
  uint32_t ring = 0;  // tiles placed so far (all tokens)
  uint32_t token_count = 0, q_loads = 0;
  // Q staging registers: `words` holds (part of) the Q slice of `staged_token`; step s < 4 loads
  // a quarter of it, steps 4 and 5 transpose the two halves.
  constexpr int kQSteps = 6;
  constexpr int kQFirstItem = 2;  // the first two tiles of a token are issued without delay
  uint32_t words[64];
  int staged_token = -1, q_step = kQSteps;
  auto q_advance = [&]() {
    const char* source = static_cast<const char*>(p.q) + (size_t)staged_token * kHeads * kRowBytes + q_octet_offset;
    auto load4 = [&](auto first) {
      constexpr int kFirst = decltype(first)::value;
#pragma unroll
      for (int j = kFirst; j < kFirst + 4; ++j) {  // row (j & 7) of the octet, units 8 (j >> 3) .. + 7
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(source + (size_t)(j & 7) * kRowBytes + (j >> 3) * 128));
        words[4 * j + 0] = v.x; words[4 * j + 1] = v.y; words[4 * j + 2] = v.z; words[4 * j + 3] = v.w;
      }
    };
    switch (q_step) {
      case 0: load4(std::integral_constant<int, 0>{}); break;
      case 1: load4(std::integral_constant<int, 4>{}); break;
      case 2: load4(std::integral_constant<int, 8>{}); break;
      case 3: load4(std::integral_constant<int, 12>{}); break;
      case 4: transpose_octet(words, lane); break;
      default: transpose_octet(words + 32, lane); break;
    }
    ++q_step;
  };
  TokenWalk walk(p);
  // The first token's Q does not depend on the resolver: its loads go out while the token is
  // being resolved (a block that only gets a few tokens spends a good part of its time here).
  staged_token = walk.peek();
  if (staged_token >= 0) {
    q_step = 0;
    while (q_step < kQSteps) q_advance();
  }
  for (int token = walk.next(); token >= 0; token = walk.next(), ++token_count) {
    if (!warp_wait(sm.bar(kTokenReady0 + (token_count & 1)), (token_count >> 1) & 1, abort_flag)) return;
    const int* rows = sm.rows(token_count & 1);
    const TokenInfo* info = sm.info(token_count & 1);
    const int chunks = info->chunks;
    // (for a working token this is said behind the first tile, off the token's critical path)
    if (chunks == 0 && lane == 0) mbar_arrive(sm.bar(kInfoRead0 + (token_count & 1)));
    for (int item = 0; item < chunks; ++item, ++ring) {
      const uint32_t stage = ring % kStages, use = ring / kStages;
      if (use > 0 && !warp_wait(sm.bar(kKvFree0 + stage), (use - 1) & 1, abort_flag)) return;
      const uint32_t tile = sm.base + kSmemKv + stage * kTileBytes;
      const int chunk = info->chunk[item];
      // Sixteen threads per row and quarter: eight 16-byte units of block q, eight of block q + 4.
      const int sub = tid & 15;
      const char* source[kChunkRows / (kProducerThreads / 16)];
      bool live[kChunkRows / (kProducerThreads / 16)];
#pragma unroll
      for (int k = 0; k < kChunkRows / (kProducerThreads / 16); ++k) {
        const int slot = chunk * kChunkRows + (tid >> 4) + k * (kProducerThreads / 16);
        const int row = rows[slot];
        live[k] = row >= 0;
        source[k] = (slot < kWindow ? window_base : compressed_base) + (size_t)(row < 0 ? 0 : row) * kRowBytes;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int unit = (q + 4 * (sub >> 3)) * 8 + (sub & 7);
#pragma unroll
        for (int k = 0; k < kChunkRows / (kProducerThreads / 16); ++k) {
          const int r = (tid >> 4) + k * (kProducerThreads / 16);
          cp_async16(tile + swizzled(r, unit), source[k] + unit * 16, live[k]);
        }
      }
      cp_async_arrive(sm.bar(kKvFull0 + stage));
      if (item == 0 && lane == 0) mbar_arrive(sm.bar(kInfoRead0 + (token_count & 1)));
      if (item == 0) {
        // The token's Q, right behind its first tile. Its registers were filled while the
        // previous token's tiles were being issued, unless this is the block's first working
        // token or the walk skipped an empty one. The wait (the previous working token's last
        // QK has read the old Q) cannot depend on this thread: all its tiles have been issued.
        if (staged_token != token) { staged_token = token; q_step = 0; }
        while (q_step < kQSteps) q_advance();
        if (q_loads > 0 && !warp_wait(sm.bar(kQFree), (q_loads - 1) & 1, abort_flag)) return;
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tmem_st16(q_tmem + j * 16, *reinterpret_cast<uint32_t(*)[16]>(&words[16 * j]));
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar(kQFull));
        ++q_loads;
        staged_token = walk.peek();  // start on the next token's Q
        q_step = staged_token >= 0 ? 0 : kQSteps;
      } else if (item >= kQFirstItem && q_step < kQSteps) {
        q_advance();  // one slice of the next token's Q per tile, so that it never comes as a burst
      }
    }
  }
}

// ---- MMA warp (one thread) --------------------------------------------------------------------

// Compile-time unrolled issue loops: every operand offset and accumulate flag is an immediate,
// so the issuing thread spends a couple of instructions per MMA and stays ahead of the pipe.
constexpr int kQkSteps = kFeatures / 32;  // K = 16 steps over one half of the features
template <int kFormat, int K, int kEnd = kQkSteps>
__device__ __forceinline__ void issue_qk_steps(uint32_t s_tmem, uint32_t q_tmem, uint64_t x_desc) {
  if constexpr (K < kEnd) {
    constexpr uint32_t offset = block_position(K >> 2) * kBlockBytes + (K & 3) * 32;
    mma_ts_c<K != 0>(s_tmem, q_tmem + K * 8, x_desc + (offset >> 4), kIdescQK<kFormat>);
    issue_qk_steps<kFormat, K + 1, kEnd>(s_tmem, q_tmem, x_desc);
  }
}

// S = Q X^T for one 64-row tile as ONE M = 128, N = 128 product per K step. Operand rows
// (tensor-memory lanes) 16-31 of every subpartition hold the high feature half of the heads
// whose low half is in lanes 0-15; operand "rows" 64-127 of B are the tile's rows again, high
// feature half (block b + 4 next to block b). Of the 128 x 128 result a thread's useful scores
// are columns 0-63 in a low-half lane (Q_lo . X_lo) and 64-127 in a high-half lane
// (Q_hi . X_hi); the other two quadrants mix the halves and are ignored. Half the products are
// thrown away, but M = 128 runs at the full rate of the pipe and N = 128 is above its
// per-instruction floor: 16 instructions of 64 cycles replace 32 of about 56.
template <int kFormat, int kBegin = 0, int kEnd = kQkSteps>
__device__ __forceinline__ void issue_qk(const Shared& sm, uint32_t tmem, int stage) {
  const uint64_t x_desc = smem_desc_sw128(sm.base + kSmemKv + stage * kTileBytes, 16, 1024);
  issue_qk_steps<kFormat, kBegin, kEnd>(tmem + kTmemS, tmem + kTmemQ, x_desc);
}

constexpr int kPvSteps = 2 * (kChunkRows / 16);
template <int kFormat, int I, bool kFirst, int kEnd = kPvSteps>
__device__ __forceinline__ void issue_pv_steps(uint32_t o_tmem, uint64_t p_desc, uint64_t x_desc) {
  if constexpr (I < kEnd) {
    constexpr int h = I / (kChunkRows / 16), k = I % (kChunkRows / 16);
    constexpr uint32_t offset = h * kBlockBytes + k * 2048;
    mma_ws_ss_c<!(kFirst && k == 0)>(o_tmem + h * kTmemOHalf, p_desc + ((k * 32) >> 4), x_desc + (offset >> 4), kIdescPV<kFormat>);
    issue_pv_steps<kFormat, I + 1, kFirst, kEnd>(o_tmem, p_desc, x_desc);
  }
}

// O += P X for one 64-row tile as two weight-stationary M = 64, N = 256 products (features 0-255
// and 256-511): with 64 heads a plain M = 64 instruction would leave half of the pipe idle.
// A = P from shared memory (one 128-byte row per head, 32 bytes per K = 16 step); B = X with
// features contiguous: the four 64-feature blocks of a half are two block positions apart,
// 8-row groups 1024 bytes apart.
template <int kFormat, int kBegin = 0, int kEnd = kPvSteps>
__device__ __forceinline__ void issue_pv(const Shared& sm, uint32_t tmem, int stage, bool accumulate) {
  const uint64_t x_desc = smem_desc_sw128(sm.base + kSmemKv + stage * kTileBytes, 2 * kBlockBytes, 1024);
  const uint64_t p_desc = smem_desc_sw128(sm.base + kSmemP, 16, 1024);
  if (accumulate) issue_pv_steps<kFormat, kBegin, false, kEnd>(tmem + kTmemO, p_desc, x_desc);
  else issue_pv_steps<kFormat, kBegin, true, kEnd>(tmem + kTmemO, p_desc, x_desc);
}

// Two issuing threads in two warps, one per product. Each follows its own data: the QK thread
// goes on as soon as a tile has landed and the score buffer is free, the PV thread as soon as a P
// is complete. The tensor pipe executes what arrives in the order it arrives, so the
// non-MMA instructions of one thread (barrier waits, commits, fences: a hundred cycles and more
// each, far beyond what the pipe's short queue covers) run while the other thread's product
// executes. Both walk the same token and chunk sequence as everybody else.

// S = Q X^T: chunk c of the block's chunk stream uses ring stage c % kStages and the c-th phase of
// the score barrier.
template <int kFormat>
__device__ void qk_role(const Params& p, const Shared& sm, uint32_t tmem) {
  volatile int* abort_flag = sm.abort_flag();
  uint32_t chunk_count = 0, working_tokens = 0;
  const uint32_t my_tokens = uint32_t(TokenWalk(p).count());  // closed form: no walk on this thread
  for (uint32_t token_count = 0; token_count < my_tokens; ++token_count) {
    if (!mbar_wait(sm.bar(kTokenReady0 + (token_count & 1)), (token_count >> 1) & 1, abort_flag)) return;
    const int chunks = sm.info(token_count & 1)->chunks;
    if (chunks == 0) {
      mbar_arrive(sm.bar(kInfoRead0 + (token_count & 1)));
      continue;
    }
    // the token's Q is in tensor memory
    if (!mbar_wait(sm.bar(kQFull), working_tokens & 1, abort_flag)) return;
    for (int i = 0; i < chunks; ++i, ++chunk_count) {
      const uint32_t stage = chunk_count % kStages;
      // One barrier says both that the tile has landed and that the single score buffer is free
      // (the softmax warps have read the previous chunk out of it).
      if (!mbar_wait(sm.bar(kKvFull0 + stage), (chunk_count / kStages) & 1, abort_flag)) return;
      tc_fence_after_sync();
      issue_qk<kFormat>(sm, tmem, stage);
      mma_commit(sm.bar(kSFull));
      if (i + 1 == chunks) mma_commit(sm.bar(kQFree));  // the last QK that reads this token's Q
      if (i == 0) mbar_arrive(sm.bar(kInfoRead0 + (token_count & 1)));  // chunk count read (see resolver)
    }
    ++working_tokens;
  }
}

// O += P X (O = P X for a token's first chunk, once the previous token's O has been read out).
template <int kFormat>
__device__ void pv_role(const Params& p, const Shared& sm, uint32_t tmem) {
  volatile int* abort_flag = sm.abort_flag();
  uint32_t chunk_count = 0, working_tokens = 0;
  const uint32_t my_tokens = uint32_t(TokenWalk(p).count());
  for (uint32_t token_count = 0; token_count < my_tokens; ++token_count) {
    if (!mbar_wait(sm.bar(kTokenReady0 + (token_count & 1)), (token_count >> 1) & 1, abort_flag)) return;
    const int chunks = sm.info(token_count & 1)->chunks;
    mbar_arrive(sm.bar(kInfoRead0 + (token_count & 1)));
    if (chunks == 0) continue;
    for (int i = 0; i < chunks; ++i, ++chunk_count) {
      const uint32_t stage = chunk_count % kStages;
      if (!mbar_wait(sm.bar(kPFull), chunk_count & 1, abort_flag)) return;
      if (i == 0 && !mbar_wait(sm.bar(kOFree), (working_tokens & 1) ^ 1, abort_flag)) return;
      tc_fence_after_sync();
      issue_pv<kFormat>(sm, tmem, stage, i != 0);
      mma_commit(sm.bar(kKvFree0 + stage));  // frees the ring stage for the producers
      mma_commit(sm.bar(kSoftmaxSync));      // and counts towards the softmax warps' step c + 1
    }
    ++working_tokens;
  }
}

// ---- softmax / correction / epilogue warps ----------------------------------------------------

template <int kFormat>
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {  // two FP32 -> two storage words
  if constexpr (kFormat == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

__device__ __forceinline__ float max3(float a, float b, float c) {  // one instruction on sm_100
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int kFormat>
__device__ void softmax_role(const Params& p, const Shared& sm, uint32_t tmem) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane >> 4;
  const int head = warp * 16 + (lane & 15);
  const uint32_t lane_base = uint32_t(warp * 32) << 16;
  volatile int* abort_flag = sm.abort_flag();
  const float sink = __ldg(p.sinks + head) * 1.4426950408889634f;  // log2 domain
  uint32_t chunk_count = 0, token_count = 0;
  // The accumulator's layout is that of the weight-stationary PV (lane = head for lanes 0-63, the
  // same heads again for lanes 64-127 with the next 128 features), not that of the scores: this
  // thread reads O of head `o_head`, features o_feature .. + 127 of each 256-feature half.
  const int o_head = (warp & 1) * 32 + lane, o_feature = (warp >> 1) * 128;
  float* alpha_exchange = reinterpret_cast<float*>(sm.ptr + kSmemAlpha);
  float* inverse_exchange = reinterpret_cast<float*>(sm.ptr + kSmemInverse);
  __nv_bfloat16* out_base = static_cast<__nv_bfloat16*>(p.out);
  const uint32_t s_addr = tmem + kTmemS + lane_base;

  if (lane == 0) mbar_arrive(sm.bar(kKvFull0));  // the score buffer starts out free (first chunk, stage 0)
  // Step c (c >= 1) of this block's chunk stream is one phase of one barrier: it completes once
  // all four softmax warps have published what they hand each other for chunk c (rescale factors,
  // or the finished token's reciprocal denominators) AND the PV of chunk c - 1 has completed
  // (the MMA thread commits every PV to it). A warp arrives as early as it can and waits, once,
  // right before it needs the others' values, O, or the P tile: one wait per chunk for all three.
  uint32_t steps_arrived = 0, steps_waited = 0;  // steps 1 .. n are done
  auto step_arrive = [&](uint32_t step) {
    if (steps_arrived >= step) return;
    __syncwarp();
    if (lane == 0) mbar_arrive(sm.bar(kSoftmaxSync));
    steps_arrived = step;
  };
  auto step_wait = [&](uint32_t step) -> bool {
    if (steps_waited >= step) return true;
    if (!warp_wait(sm.bar(kSoftmaxSync), (step - 1) & 1, abort_flag)) return false;
    steps_waited = step;
    return true;
  };

  // A finished token waits for its epilogue until the first chunk of the next working token has
  // been through the softmax, so that the MMA thread has a P to go on with while O is written out.
  int done_token = -1;          // token whose O is complete (or about to be) and not yet stored
  uint32_t done_count = 0;      // its index in this block's walk

  // O / denominator -> 16-bit -> global for `done_token`: 64 columns per pass, tensor memory ->
  // registers -> a swizzled per-warp staging tile -> global, so that every store instruction
  // writes four complete 128-byte lines.
  auto epilogue = [&]() -> bool {
    // The token's last PV and everybody's reciprocal denominators: step `chunk_count`. After the
    // next token's first chunk that step has been waited for already.
    step_arrive(chunk_count);
    if (!step_wait(chunk_count)) return false;
    tc_fence_after_sync();
    const float inverse = inverse_exchange[(done_count & 1) * kHeads + o_head];
    unsigned char* staging = sm.ptr + kSmemStore + warp * 4096;
    __nv_bfloat16* token_out = out_base + (size_t)done_token * kHeads * kFeatures;
#pragma unroll 1
    for (int c = 0; c < 256; c += 64) {
      uint32_t o[64];
#pragma unroll
      for (int q = 0; q < 64; q += 16)
        tmem_ld16(tmem + kTmemO + c + q + lane_base, *reinterpret_cast<uint32_t(*)[16]>(&o[q]));
      tmem_wait_ld();
      if (c == 192) {  // O has been read completely: the next token's first PV may overwrite it
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar(kOFree));
      }
#pragma unroll
      for (int unit = 0; unit < 8; ++unit) {
        uint4 v;
        v.x = pack_pair<kFormat>(__uint_as_float(o[unit * 8 + 0]) * inverse, __uint_as_float(o[unit * 8 + 1]) * inverse);
        v.y = pack_pair<kFormat>(__uint_as_float(o[unit * 8 + 2]) * inverse, __uint_as_float(o[unit * 8 + 3]) * inverse);
        v.z = pack_pair<kFormat>(__uint_as_float(o[unit * 8 + 4]) * inverse, __uint_as_float(o[unit * 8 + 5]) * inverse);
        v.w = pack_pair<kFormat>(__uint_as_float(o[unit * 8 + 6]) * inverse, __uint_as_float(o[unit * 8 + 7]) * inverse);
        *reinterpret_cast<uint4*>(staging + lane * 128 + ((unit ^ (lane & 7)) << 4)) = v;
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = i * 4 + (lane >> 3), unit = lane & 7;  // staging row = owning lane
        const uint4 v = *reinterpret_cast<const uint4*>(staging + row * 128 + ((unit ^ (row & 7)) << 4));
        // accumulator columns 0-127: features 0-255 (this warp's 128 of them), 128-255: 256-511
        __nv_bfloat16* dst = token_out + (size_t)((warp & 1) * 32 + row) * kFeatures + (c >> 7) * 256 + o_feature + (c & 127) + unit * 8;
        __stcs(reinterpret_cast<uint4*>(dst), v);  // written once, read by nobody here
      }
      __syncwarp();
    }
    if (lane == 0) mbar_arrive(sm.bar(kTokenDone0 + (done_count & 1)));
    done_token = -1;
    return true;
  };

  TokenWalk walk(p);
  for (int token = walk.next(); token >= 0; token = walk.next(), ++token_count) {
    if (!warp_wait(sm.bar(kTokenReady0 + (token_count & 1)), (token_count >> 1) & 1, abort_flag)) return;
    const TokenInfo* info = sm.info(token_count & 1);
    const int chunks = info->chunks;
    if (chunks == 0) {  // nothing visible: the output row is zero whatever the sink
      // The resolver needs the finished token's row buffer back before it can publish the token
      // after this one: no point in holding its epilogue any longer.
      if (done_token >= 0 && !epilogue()) return;
      __nv_bfloat16* out = out_base + ((size_t)token * kHeads + head) * kFeatures + half * 256;
      for (int i = 0; i < 256; i += 8) *reinterpret_cast<uint4*>(out + i) = make_uint4(0, 0, 0, 0);
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar(kTokenDone0 + (token_count & 1)));
      continue;
    }
    // `run_sum` is this lane's share of the denominator; the low lane's share includes the
    // sink's own weight exp2(sink - run_max) = 1.
    float run_max = sink, run_sum = half ? 0.f : 1.f;
    for (int i = 0; i < chunks; ++i, ++chunk_count) {
      const int chunk = info->chunk[i];
      const unsigned live_lo = info->live[2 * chunk], live_hi = info->live[2 * chunk + 1];

      if (!warp_wait(sm.bar(kSFull), chunk_count & 1, abort_flag)) return;
      tc_fence_after_sync();
      // Lane (head, low half) holds Q_lo . X_lo in columns 0-63, lane (head, high half) holds
      // Q_hi . X_hi in columns 64-127. The two threads of a head share the softmax work: the low
      // thread owns tile rows 0-31, the high thread rows 32-63. Both partial scores of a row come
      // straight to the thread that owns it: a load over the 16 low lanes gives threads 0-15
      // columns j and threads 16-31 columns 32 + j of the low partials; a load over the 16 high
      // lanes gives them columns 64 + j and 96 + j of the high partials. No exchange between lanes.
      const unsigned live = half ? live_hi : live_lo;
      const bool all_live = (live_lo & live_hi) == 0xffffffffu;  // the usual case: nothing to mask
      float mine[32];  // unscaled scores: the scale goes into the exponent's FMA
      {
        uint32_t low_a[16], low_b[16], high_a[16], high_b[16];
        tmem_ld16_halves<32>(s_addr, low_a);                       // rows 0-15 | 32-47, low partial
        tmem_ld16_halves<32>(s_addr + 16, low_b);                  // rows 16-31 | 48-63
        tmem_ld16_halves<32>(s_addr + kHalfLanes + 64, high_a);    // the same rows, high partial
        tmem_ld16_halves<32>(s_addr + kHalfLanes + 80, high_b);
        tmem_wait_ld();
        // The scores are in registers: the next QK may overwrite the buffer. Its tile's full
        // barrier counts this as well as the copies.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar(kKvFull0 + (chunk_count + 1) % kStages));
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          mine[e] = __uint_as_float(low_a[e]) + __uint_as_float(high_a[e]);
          mine[16 + e] = __uint_as_float(low_b[e]) + __uint_as_float(high_b[e]);
        }
      }
      if (!all_live) {
#pragma unroll
        for (int j = 0; j < 32; ++j) mine[j] = ((live >> j) & 1u) ? mine[j] : -INFINITY;
      }
      float partial_max[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) partial_max[j] = max3(mine[j], mine[j + 4], mine[j + 8]);
#pragma unroll
      for (int j = 12; j < 32; j += 8)
#pragma unroll
        for (int k = 0; k < 4; ++k) partial_max[k] = max3(partial_max[k], mine[j + k], mine[j + 4 + k]);
      partial_max[0] = max3(partial_max[0], mine[28], mine[29]);
      partial_max[1] = max3(partial_max[1], mine[30], mine[31]);
      float chunk_max = fmaxf(fmaxf(partial_max[0], partial_max[1]), fmaxf(partial_max[2], partial_max[3]));
      chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, 16)) * p.scale_log2;  // scale > 0
      // The running maximum only moves when it is exceeded by more than 8 (a factor 256), so the
      // accumulator is rescaled rarely; probabilities stay below 2^8 and all terms of one head
      // share the same reference, which cancels in the final division.
      float alpha = 1.f;
      if (chunk_max > run_max + 8.f) {
        alpha = exp2f(run_max - chunk_max);
        run_max = chunk_max;
      }
      if (i > 0) {
        // O holds earlier chunks. The factor of a head is known to the thread that has its scores;
        // the head's accumulator rows are in other threads' lanes: hand the factors over.
        // They are picked up after the exponentials, when everybody's have long been written.
        if (half == 0) alpha_exchange[(chunk_count & 1) * kHeads + head] = alpha;
      }
      if (chunk_count > 0) step_arrive(chunk_count);
      float partial_sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 32; ++j) { mine[j] = exp2f(fmaf(mine[j], p.scale_log2, -run_max)); partial_sum[j & 3] += mine[j]; }
      run_sum = run_sum * alpha + ((partial_sum[0] + partial_sum[1]) + (partial_sum[2] + partial_sum[3]));
      // There is one P tile: the previous chunk's PV must have finished reading it. (In step, that
      // PV ran right behind the QK whose scores this chunk started from.)
      if (chunk_count > 0 && !step_wait(chunk_count)) return;
      if (i > 0) {
        const float o_alpha = alpha_exchange[(chunk_count & 1) * kHeads + o_head];
        if (__any_sync(0xffffffffu, o_alpha != 1.f)) {  // the previous PV has landed (wait above)
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 256; c += 16) {
            uint32_t o[16];
            tmem_ld16(tmem + kTmemO + c + lane_base, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * o_alpha);
            tmem_st16(tmem + kTmemO + c + lane_base, o);
          }
          tmem_wait_st();
        }
      }
      // P to shared memory, one 128-byte row per head; this lane writes its 32 rows (64 bytes).
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 v;
        v.x = pack_pair<kFormat>(mine[8 * u + 0], mine[8 * u + 1]); v.y = pack_pair<kFormat>(mine[8 * u + 2], mine[8 * u + 3]);
        v.z = pack_pair<kFormat>(mine[8 * u + 4], mine[8 * u + 5]); v.w = pack_pair<kFormat>(mine[8 * u + 6], mine[8 * u + 7]);
        *reinterpret_cast<uint4*>(sm.ptr + kSmemP + p_offset(head, half * 4 + u)) = v;
      }
      fence_proxy_async();  // the PV reads the tile through the async proxy
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar(kPFull));
      // The previous token's output, now that the MMA thread has this token's first P to go on with.
      if (done_token >= 0 && !epilogue()) return;
    }
    done_token = token;
    done_count = token_count;
    // Hand the reciprocal denominators over now; the epilogue picks them up a chunk later.
    const float own_inverse = 1.f / (run_sum + __shfl_xor_sync(0xffffffffu, run_sum, 16));
    if (half == 0) inverse_exchange[(done_count & 1) * kHeads + head] = own_inverse;
  }
  if (done_token >= 0 && !epilogue()) return;
}

// ---- kernel and launch ------------------------------------------------------------------------

template <int kFormat>
__global__ void __launch_bounds__(kThreads, 1) attention_kernel(const Params p) {
  extern __shared__ unsigned char smem_raw[];
  Shared sm;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  sm.base = raw + pad;
  sm.ptr = smem_raw + pad;
  const int warp = threadIdx.x >> 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm.ptr + kSmemMisc);

  if (threadIdx.x == 0) {
    const int P = kProducerWarps, S = kSoftmaxWarps, T = kProducerThreads;
    const int counts[kBarCount] = {1, 1, S, S, P, 1, 1, 1, 1, 1, S, S, T + S, T + S, T + S, S + 1, P + 2, P + 2};
    for (int i = 0; i < kBarCount; ++i) mbar_init(sm.bar(i), counts[i]);
    mbar_fence_init();
    *sm.abort_flag() = 0;
  }
  if (warp == kMmaWarp) { tmem_alloc(smem_u32(tmem_slot), kTmemColumns); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp < kSoftmaxWarps) {
    softmax_role<kFormat>(p, sm, tmem);
  } else if (warp == kMmaWarp) {
    if ((threadIdx.x & 31) == 0) qk_role<kFormat>(p, sm, tmem);
    __syncwarp();
  } else if (warp == kPvWarp) {
    if ((threadIdx.x & 31) == 0) pv_role<kFormat>(p, sm, tmem);
    __syncwarp();
  } else if (warp == kResolverWarp) {
    resolver_role(p, sm);
  } else {
    producer_role(p, sm, tmem);
    asm volatile("cp.async.wait_all;\n" ::: "memory");
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *sm.abort_flag() != 0) report(p, kStatusWaitExpired, blockIdx.x, 0);
  if (warp == kMmaWarp) tmem_dealloc(tmem, kTmemColumns);
}

template <int kFormat>
inline int launch(const Params& p, cudaStream_t stream, int multiprocessors) {
  static bool configured[64] = {false};
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return int(error);
  if (device < 0 || device >= 64) return -1;
  if (!configured[device]) {
    error = cudaFuncSetAttribute(attention_kernel<kFormat>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (error != cudaSuccess) return int(error);
    configured[device] = true;
  }
  const int grid = p.tokens < multiprocessors ? p.tokens : multiprocessors;
  Params launch_params = p;
  const int per_block = p.tokens / (grid * 4);
  launch_params.token_group = per_block < 1 ? 1 : (per_block > 8 ? 8 : per_block);
  attention_kernel<kFormat><<<grid, kThreads, kSmemBytes, stream>>>(launch_params);
  return int(cudaGetLastError());
}

}  // namespace umma
}  // namespace sparse_mla
