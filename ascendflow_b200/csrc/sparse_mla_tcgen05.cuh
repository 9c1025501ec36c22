// Sparse MLA attention on the Blackwell tensor path: tcgen05.mma with accumulators in tensor
// memory, warp-specialised and software-pipelined. BF16 storage, FP32 accumulation and softmax.
//
// One persistent block per SM owns one query token at a time (64 heads x 512 features) and
// walks the token's live 64-row chunks (window rows first, then the compressed ranks in list
// order, as the reference does: examples/sparse_attention/attention.py:42-64, 147-207):
//
//   producer warps   resolve slot -> physical row (sparse_mla_common.cuh), then gather the rows
//                    with 16-byte cp.async into 128-byte-swizzled shared tiles (a row is fetched
//                    once and serves as K and as V); they also stage the token's Q tile.
//   MMA warp         one thread issues S = Q X^T (M64 N64 K512, both operands K-major) into a
//                    double-buffered S tile in tensor memory, and O += P X (M64 N256 x 2 halves,
//                    X read MN-major from the same tile) into the O accumulator.
//   softmax warps    tcgen05.ld S, joint online softmax with the per-head sink
//                    (examples/sparse_attention/attention.py:398-490: one maximum and one
//                    denominator over window, compressed rows and sink; P rounded to BF16 before
//                    PV, denominator from unrounded FP32), P to shared memory, O rescaled in
//                    tensor memory only when the running maximum moved by more than 2^8, final
//                    normalisation and store.
//
// Tensor memory (512 columns): an M=64 accumulator occupies lanes 0-15 of each 32-lane
// subpartition; a second one can live in lanes 16-31 of the same columns. O[:, 0:256] and
// O[:, 256:512] share columns 0-255 that way; S buffers 0 / 1 sit at columns 256 / 320 with
// lane offsets 0 / 16, so that thread (lane & 15) + 16 * parity of each softmax warp owns one
// head row of the chunk with that parity.
//
// Every wait on an mbarrier is bounded (tcgen05_ptx.cuh): on expiry the block records
// kStatusWaitExpired, all roles leave their loops, tensor memory is released, the kernel returns.
#pragma once

#include <cuda_bf16.h>

#include "sparse_mla_common.cuh"
#include "tcgen05_ptx.cuh"

namespace sparse_mla {
namespace umma {

using namespace sm100;

constexpr int kSoftmaxWarps = 4;
constexpr int kProducerWarps = 4;
constexpr int kMmaWarp = kSoftmaxWarps;                    // warp index 4
constexpr int kFirstProducerWarp = kSoftmaxWarps + 1;       // warps 5..8
constexpr int kThreads = 32 * (kSoftmaxWarps + 1 + kProducerWarps);
constexpr int kProducerThreads = 32 * kProducerWarps;

constexpr int kChunkRows = 64;
constexpr int kMaxChunks = kSlots / kChunkRows;             // 10
constexpr int kStages = 2;
constexpr int kBlockBytes = kChunkRows * 128;               // one 64-feature block of a tile: 8 KiB
constexpr int kTileBytes = 8 * kBlockBytes;                 // 64 rows x 512 features: 64 KiB

// Shared memory map (bytes from a 1024-aligned base).
constexpr int kSmemQ = 0;
constexpr int kSmemKv = kSmemQ + kTileBytes;
constexpr int kSmemP = kSmemKv + kStages * kTileBytes;      // two [64 x 64] BF16 tiles
constexpr int kSmemRows = kSmemP + 2 * kBlockBytes;         // int[2][640]
constexpr int kSmemInfo = kSmemRows + 2 * kSlots * 4;       // TokenInfo[2]
constexpr int kSmemBars = kSmemInfo + 2 * 64;               // mbarriers
constexpr int kSmemMisc = kSmemBars + 32 * 8;               // tmem slot, abort flag, scratch
constexpr int kSmemBytes = kSmemMisc + 64 + 1024;           // + slack for the 1024-byte alignment

constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kTmemO = 0;
constexpr uint32_t kTmemS = 256;                             // buffer b at column 256 + 64 b, lane offset 16 b

struct TokenInfo {
  int token;
  int chunks;                 // live chunks of this token
  unsigned char chunk[kMaxChunks];
};

enum Bar {
  kQFull0 = 0, kQFull1, kQFree, kKvFull0, kKvFull1, kKvFree0, kKvFree1, kSFull0, kSFull1, kSFree0,
  kSFree1, kPFull0, kPFull1, kPFree0, kPFree1, kODone, kOFree, kTokenDone0, kTokenDone1, kBarCount
};

constexpr uint32_t kIdescQK = idesc_f16(64, 64, 1, 0, 0);
constexpr uint32_t kIdescPV = idesc_f16(64, 256, 1, 0, 1);

// Byte offset of 16-byte unit `unit` (0..63) of row `row` in a K-major 128-byte-swizzled tile
// of 64 rows: eight 64-feature blocks of [64 rows x 128 bytes].
__device__ __forceinline__ uint32_t swizzled(int row, int unit) {
  return (unit >> 3) * kBlockBytes + row * 128 + (((unit & 7) ^ (row & 7)) << 4);
}

__device__ __forceinline__ void producer_sync() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(kProducerThreads) : "memory");
}

struct Shared {
  uint32_t base;        // shared-space address of the 1024-aligned region
  unsigned char* ptr;   // generic pointer to the same
  __device__ __forceinline__ uint32_t bar(int which) const { return base + kSmemBars + which * 8; }
  __device__ __forceinline__ int* rows(int buffer) const {
    return reinterpret_cast<int*>(ptr + kSmemRows) + buffer * kSlots;
  }
  __device__ __forceinline__ TokenInfo* info(int buffer) const {
    return reinterpret_cast<TokenInfo*>(ptr + kSmemInfo + buffer * 64);
  }
  __device__ __forceinline__ volatile int* abort_flag() const {
    return reinterpret_cast<volatile int*>(ptr + kSmemMisc + 4);
  }
  __device__ __forceinline__ int* scratch() const { return reinterpret_cast<int*>(ptr + kSmemMisc + 8); }
};

// ---- producer warps ---------------------------------------------------------------------------

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool live) {
  // A masked slot is zero-filled (source size 0) so the tile never holds non-finite leftovers.
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(live ? 16 : 0));
}

// A producer wait whose outcome is the same for all producer threads: if any of them gave up,
// all of them leave (a thread that returned alone would strand the others at the next bar.sync).
__device__ __forceinline__ bool producer_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t ok = mbar_wait(bar, parity, abort_flag) ? 1u : 0u;
  uint32_t failed;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.eq.u32 q, %1, 0;\n"
      "bar.red.or.pred p, 1, %2, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n" : "=r"(failed) : "r"(ok), "n"(kProducerThreads) : "memory");
  return failed == 0;
}

// A wait whose outcome is uniform across the calling warp (all 32 lanes must call it).
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}

__device__ void producer_role(const Params& p, const Shared& sm) {
  const int tid = threadIdx.x - kFirstProducerWarp * 32;  // 0..127
  const int lane = tid & 31;
  volatile int* abort_flag = sm.abort_flag();
  uint32_t chunk_count = 0;  // live chunks handed to the MMA warp so far (all tokens)
  uint32_t token_count = 0;
  for (int token = blockIdx.x; token < p.tokens; token += gridDim.x, ++token_count) {
    const int buffer = token_count & 1;
    int* rows = sm.rows(buffer);
    TokenInfo* info = sm.info(buffer);
    int* scratch = sm.scratch();

    // Resolve the 640 slots once the softmax warps have finished the token that used this
    // buffer two tokens ago. (Barriers that a role may pass without the others keeping up are
    // kept per buffer: a phase parity can only tell apart two consecutive phases.)
    if (token_count >= 2 &&
        !producer_wait(sm.bar(kTokenDone0 + buffer), ((token_count >> 1) & 1) ^ 1, abort_flag)) return;
    const TokenGeometry g = token_geometry(p, token);
    if (tid == 0) *scratch = kTopK;
    producer_sync();
    const int32_t* list = p.indices + (size_t)token * kTopK;
    {
      int first = kTopK;
      for (int rank = tid; rank < kTopK; rank += kProducerThreads)
        if (__ldg(list + rank) < 0) { first = rank; break; }
      if (first < kTopK) atomicMin(scratch, first);
    }
    producer_sync();
    const int first_negative = *scratch;
    for (int slot = tid; slot < kSlots; slot += kProducerThreads)
      rows[slot] = slot < kWindow
          ? resolve_window_slot(p, g, token, slot)
          : resolve_compressed_rank(p, g, token, slot - kWindow, __ldg(list + slot - kWindow), first_negative);
    producer_sync();
    if (tid < 32) {  // one warp lists the chunks that hold at least one live slot
      int count = 0;
      for (int chunk = 0; chunk < kMaxChunks; ++chunk) {
        const bool live = rows[chunk * kChunkRows + lane] >= 0 || rows[chunk * kChunkRows + 32 + lane] >= 0;
        if (__any_sync(0xffffffffu, live)) {
          if (lane == 0) info->chunk[count] = (unsigned char)chunk;
          ++count;
        }
      }
      if (lane == 0) { info->token = token; info->chunks = count; }
    }
    producer_sync();
    const int chunks = info->chunks;

    // Q tile: wait until the previous token's last QK has read it.
    if (!producer_wait(sm.bar(kQFree), (token_count & 1) ^ 1, abort_flag)) return;
    if (chunks > 0) {
      const char* q = static_cast<const char*>(p.q) + (size_t)token * kHeads * kRowBytes;
      const int unit = tid & 63;
      for (int r = tid >> 6; r < kHeads; r += kProducerThreads / 64)
        cp_async16(sm.base + kSmemQ + swizzled(r, unit), q + (size_t)r * kRowBytes + unit * 16, true);
      asm volatile("cp.async.commit_group;\n" ::: "memory");
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      fence_proxy_async();
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(sm.bar(kQFull0 + buffer));

    const char* window_base = static_cast<const char*>(p.ori_kv);
    const char* compressed_base = static_cast<const char*>(p.cmp_kv);
    for (int i = 0; i < chunks; ++i, ++chunk_count) {
      const int stage = chunk_count & 1;
      if (!producer_wait(sm.bar(kKvFree0 + stage), ((chunk_count >> 1) & 1) ^ 1, abort_flag)) return;
      const int chunk = info->chunk[i];
      const uint32_t tile = sm.base + kSmemKv + stage * kTileBytes;
      const int unit = tid & 63;
      for (int r = tid >> 6; r < kChunkRows; r += kProducerThreads / 64) {
        const int slot = chunk * kChunkRows + r;
        const int row = rows[slot];
        const char* base = slot < kWindow ? window_base : compressed_base;
        cp_async16(tile + swizzled(r, unit), base + (size_t)(row < 0 ? 0 : row) * kRowBytes + unit * 16, row >= 0);
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar(kKvFull0 + stage));
    }
  }
}

// ---- MMA warp (one thread) --------------------------------------------------------------------

__device__ __forceinline__ void issue_qk(const Shared& sm, uint32_t tmem, int stage, int s_buffer) {
  const uint32_t d = tmem + kTmemS + s_buffer * 64 + (uint32_t(16 * s_buffer) << 16);
  const uint32_t q = sm.base + kSmemQ, x = sm.base + kSmemKv + stage * kTileBytes;
#pragma unroll
  for (int k = 0; k < kFeatures / 16; ++k) {
    const uint32_t offset = (k >> 2) * kBlockBytes + (k & 3) * 32;
    mma_ss(d, smem_desc_sw128(q + offset, 16, 1024), smem_desc_sw128(x + offset, 16, 1024), kIdescQK, k > 0);
  }
}

__device__ __forceinline__ void issue_pv(const Shared& sm, uint32_t tmem, int stage, int p_buffer, bool accumulate) {
  const uint32_t prob = sm.base + kSmemP + p_buffer * kBlockBytes, x = sm.base + kSmemKv + stage * kTileBytes;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint32_t d = tmem + kTmemO + (uint32_t(16 * half) << 16);
#pragma unroll
    for (int k = 0; k < kChunkRows / 16; ++k) {
      // A: P[64 heads x 16 rows], K-major. B: X[16 rows x 256 features], features contiguous:
      // four 64-feature blocks kBlockBytes apart, 8-row groups 1024 bytes apart.
      mma_ss(d, smem_desc_sw128(prob + k * 32, 16, 1024),
             smem_desc_sw128(x + half * 4 * kBlockBytes + k * 2048, kBlockBytes, 1024), kIdescPV,
             accumulate || k > 0);
    }
  }
}

__device__ void mma_role(const Params& p, const Shared& sm, uint32_t tmem) {
  volatile int* abort_flag = sm.abort_flag();
  uint32_t chunk_count = 0, token_count = 0, working_tokens = 0;
  for (int token = blockIdx.x; token < p.tokens; token += gridDim.x, ++token_count) {
    if (!mbar_wait(sm.bar(kQFull0 + (token_count & 1)), (token_count >> 1) & 1, abort_flag)) return;
    const int chunks = sm.info(token_count & 1)->chunks;
    if (chunks == 0) { mbar_arrive(sm.bar(kQFree)); continue; }
    tc_fence_after_sync();
    // First QK of the token.
    {
      const uint32_t n = chunk_count, slot = n & 1, use = (n >> 1) & 1;
      if (!mbar_wait(sm.bar(kKvFull0 + slot), use, abort_flag)) return;
      if (!mbar_wait(sm.bar(kSFree0 + slot), use ^ 1, abort_flag)) return;
      tc_fence_after_sync();
      issue_qk(sm, tmem, slot, slot);
      mma_commit(sm.bar(kSFull0 + slot));
      if (chunks == 1) mma_commit(sm.bar(kQFree));
    }
    for (int i = 0; i < chunks; ++i, ++chunk_count) {
      if (i + 1 < chunks) {  // QK of the next chunk runs while the softmax warps work on this one
        const uint32_t n = chunk_count + 1, slot = n & 1, use = (n >> 1) & 1;
        if (!mbar_wait(sm.bar(kKvFull0 + slot), use, abort_flag)) return;
        if (!mbar_wait(sm.bar(kSFree0 + slot), use ^ 1, abort_flag)) return;
        tc_fence_after_sync();
        issue_qk(sm, tmem, slot, slot);
        mma_commit(sm.bar(kSFull0 + slot));
        if (i + 2 == chunks) mma_commit(sm.bar(kQFree));
      }
      const uint32_t slot = chunk_count & 1, use = (chunk_count >> 1) & 1;
      if (i == 0) {  // the previous token's epilogue must have read O
        if (!mbar_wait(sm.bar(kOFree), (working_tokens & 1) ^ 1, abort_flag)) return;
      }
      if (!mbar_wait(sm.bar(kPFull0 + slot), use, abort_flag)) return;
      tc_fence_after_sync();
      issue_pv(sm, tmem, slot, slot, i > 0);
      mma_commit(sm.bar(kKvFree0 + slot));
      mma_commit(sm.bar(kPFree0 + slot));
      mma_commit(sm.bar(kODone));
    }
    ++working_tokens;
  }
}

// ---- softmax / correction / epilogue warps ----------------------------------------------------

__device__ void softmax_role(const Params& p, const Shared& sm, uint32_t tmem) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int parity = lane >> 4;                 // which S buffer / which half of O this lane owns
  const int head = warp * 16 + (lane & 15);
  const uint32_t lane_base = uint32_t(warp * 32) << 16;
  volatile int* abort_flag = sm.abort_flag();
  const float sink = __ldg(p.sinks + head) * 1.4426950408889634f;  // log2 domain
  uint32_t chunk_count = 0, token_count = 0, pv_waited = 0;
  __nv_bfloat16* out_base = static_cast<__nv_bfloat16*>(p.out);

  for (int token = blockIdx.x; token < p.tokens; token += gridDim.x, ++token_count) {
    if (!warp_wait(sm.bar(kQFull0 + (token_count & 1)), (token_count >> 1) & 1, abort_flag)) return;
    const TokenInfo* info = sm.info(token_count & 1);
    const int* rows = sm.rows(token_count & 1);
    const int chunks = info->chunks;
    __nv_bfloat16* out = out_base + ((size_t)token * kHeads + head) * kFeatures + parity * 256;
    if (chunks == 0) {  // nothing visible: the output row is zero whatever the sink
      for (int i = 0; i < 256; i += 8) *reinterpret_cast<uint4*>(out + i) = make_uint4(0, 0, 0, 0);
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar(kTokenDone0 + (token_count & 1)));
      continue;
    }
    float run_max = sink, run_sum = 1.f;  // the sink's own weight exp2(sink - run_max)
    for (int i = 0; i < chunks; ++i, ++chunk_count) {
      const uint32_t slot = chunk_count & 1, use = (chunk_count >> 1) & 1;
      const bool owner = parity == int(slot);
      const int chunk = info->chunk[i];
      const unsigned live_lo = __ballot_sync(0xffffffffu, rows[chunk * kChunkRows + lane] >= 0);
      const unsigned live_hi = __ballot_sync(0xffffffffu, rows[chunk * kChunkRows + 32 + lane] >= 0);

      if (!warp_wait(sm.bar(kSFull0 + slot), use, abort_flag)) return;
      tc_fence_after_sync();
      uint32_t raw[64];
#pragma unroll
      for (int c = 0; c < 64; c += 16)
        tmem_ld16(tmem + kTmemS + slot * 64 + c + lane_base, *reinterpret_cast<uint32_t(*)[16]>(&raw[c]));
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar(kSFree0 + slot));

      float s[64];
      float chunk_max = -INFINITY;
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const bool live = ((j < 32 ? live_lo : live_hi) >> (j & 31)) & 1u;
        s[j] = (owner && live) ? __uint_as_float(raw[j]) * p.scale_log2 : -INFINITY;
        chunk_max = fmaxf(chunk_max, s[j]);
      }
      chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, 16));
      // The running maximum only moves when it is exceeded by more than 8 (a factor 256), so the
      // accumulator is rescaled rarely; probabilities stay below 2^8 and all terms of one head
      // share the same reference, which cancels in the final division.
      float alpha = 1.f;
      if (chunk_max > run_max + 8.f) {
        alpha = exp2f(run_max - chunk_max);
        run_max = chunk_max;
      }
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
        if (i > 0) {  // O holds earlier chunks: the previous PV must have landed
          while (pv_waited < chunk_count) {
            if (!warp_wait(sm.bar(kODone), pv_waited & 1, abort_flag)) return;
            ++pv_waited;
          }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 256; c += 16) {
            uint32_t o[16];
            tmem_ld16(tmem + kTmemO + c + lane_base, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st16(tmem + kTmemO + c + lane_base, o);
          }
          tmem_wait_st();
          tc_fence_before_sync();
        }
      }
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 64; ++j) { s[j] = exp2f(s[j] - run_max); sum += s[j]; }
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      run_sum = run_sum * alpha + sum;

      if (!warp_wait(sm.bar(kPFree0 + slot), use ^ 1, abort_flag)) return;
      if (owner) {
        unsigned char* row = sm.ptr + kSmemP + slot * kBlockBytes + head * 128;
#pragma unroll
        for (int unit = 0; unit < 8; ++unit) {
          uint4 packed;
          __nv_bfloat162 v;
          v = __floats2bfloat162_rn(s[unit * 8 + 0], s[unit * 8 + 1]); packed.x = *reinterpret_cast<uint32_t*>(&v);
          v = __floats2bfloat162_rn(s[unit * 8 + 2], s[unit * 8 + 3]); packed.y = *reinterpret_cast<uint32_t*>(&v);
          v = __floats2bfloat162_rn(s[unit * 8 + 4], s[unit * 8 + 5]); packed.z = *reinterpret_cast<uint32_t*>(&v);
          v = __floats2bfloat162_rn(s[unit * 8 + 6], s[unit * 8 + 7]); packed.w = *reinterpret_cast<uint32_t*>(&v);
          *reinterpret_cast<uint4*>(row + ((unit ^ (head & 7)) << 4)) = packed;
        }
        fence_proxy_async();
      }
      // Observe the previous chunk's PV completion before releasing this P: the PV barrier then
      // never runs more than one phase ahead of this warp.
      while (pv_waited < chunk_count) {
        if (!warp_wait(sm.bar(kODone), pv_waited & 1, abort_flag)) return;
        ++pv_waited;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar(kPFull0 + slot));
    }
    // ---- epilogue: O / denominator -> BF16 -> global ------------------------------------------
    while (pv_waited < chunk_count) {
      if (!warp_wait(sm.bar(kODone), pv_waited & 1, abort_flag)) return;
      ++pv_waited;
    }
    tc_fence_after_sync();
    const float inverse = 1.f / run_sum;
#pragma unroll 1
    for (int c = 0; c < 256; c += 16) {
      uint32_t o[16];
      tmem_ld16(tmem + kTmemO + c + lane_base, o);
      tmem_wait_ld();
      uint4 lo, hi;
      __nv_bfloat162 v;
      v = __floats2bfloat162_rn(__uint_as_float(o[0]) * inverse, __uint_as_float(o[1]) * inverse); lo.x = *reinterpret_cast<uint32_t*>(&v);
      v = __floats2bfloat162_rn(__uint_as_float(o[2]) * inverse, __uint_as_float(o[3]) * inverse); lo.y = *reinterpret_cast<uint32_t*>(&v);
      v = __floats2bfloat162_rn(__uint_as_float(o[4]) * inverse, __uint_as_float(o[5]) * inverse); lo.z = *reinterpret_cast<uint32_t*>(&v);
      v = __floats2bfloat162_rn(__uint_as_float(o[6]) * inverse, __uint_as_float(o[7]) * inverse); lo.w = *reinterpret_cast<uint32_t*>(&v);
      v = __floats2bfloat162_rn(__uint_as_float(o[8]) * inverse, __uint_as_float(o[9]) * inverse); hi.x = *reinterpret_cast<uint32_t*>(&v);
      v = __floats2bfloat162_rn(__uint_as_float(o[10]) * inverse, __uint_as_float(o[11]) * inverse); hi.y = *reinterpret_cast<uint32_t*>(&v);
      v = __floats2bfloat162_rn(__uint_as_float(o[12]) * inverse, __uint_as_float(o[13]) * inverse); hi.z = *reinterpret_cast<uint32_t*>(&v);
      v = __floats2bfloat162_rn(__uint_as_float(o[14]) * inverse, __uint_as_float(o[15]) * inverse); hi.w = *reinterpret_cast<uint32_t*>(&v);
      *reinterpret_cast<uint4*>(out + c) = lo;
      *reinterpret_cast<uint4*>(out + c + 8) = hi;
    }
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(sm.bar(kOFree));
      mbar_arrive(sm.bar(kTokenDone0 + (token_count & 1)));
    }
  }
}

// ---- kernel and launch ------------------------------------------------------------------------

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
    const int counts[kBarCount] = {kProducerWarps, kProducerWarps, 1, kProducerWarps, kProducerWarps, 1, 1,
                                   1, 1, kSoftmaxWarps, kSoftmaxWarps, kSoftmaxWarps, kSoftmaxWarps, 1, 1,
                                   1, kSoftmaxWarps, kSoftmaxWarps, kSoftmaxWarps};
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
    softmax_role(p, sm, tmem);
  } else if (warp == kMmaWarp) {
    if ((threadIdx.x & 31) == 0) mma_role(p, sm, tmem);
    __syncwarp();
  } else {
    producer_role(p, sm);
    asm volatile("cp.async.wait_all;\n" ::: "memory");
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *sm.abort_flag() != 0) report(p, kStatusWaitExpired, blockIdx.x, 0);
  if (warp == kMmaWarp) tmem_dealloc(tmem, kTmemColumns);
}

inline int launch(const Params& p, cudaStream_t stream, int multiprocessors) {
  static bool configured[64] = {false};
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return int(error);
  if (device < 0 || device >= 64) return -1;
  if (!configured[device]) {
    error = cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (error != cudaSuccess) return int(error);
    configured[device] = true;
  }
  const int grid = p.tokens < multiprocessors ? p.tokens : multiprocessors;
  attention_kernel<<<grid, kThreads, kSmemBytes, stream>>>(p);
  return int(cudaGetLastError());
}

}  // namespace umma
}  // namespace sparse_mla
