// Sparse MLA attention on the warp-level tensor path (ldmatrix + mma.sync m16n8k16).
//
// One block of 8 warps owns one query token at a time (64 heads x 512 features) and walks its
// 640 slots in ten 64-row chunks: window rows first, then the compressed ranks in list order,
// as the reference does (examples/sparse_attention/attention.py:42-64, 147-207). Rows of a chunk
// are fetched with 16-byte cp.async into a double-buffered shared tile and serve as K for
// S = Q X^T and as V for O += P X. The softmax is the joint one of the reference
// (examples/sparse_attention/attention.py:398-490): one running maximum and one denominator
// over window, compressed rows and the per-head sink, with P rounded to the storage type
// before PV and the denominator kept in unrounded FP32.
//
// This kernel is the portable-instruction implementation; it is used for the FP16
// specialisation and as the cross-check of the tcgen05 kernel on full-size inputs.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sparse_mla_common.cuh"

namespace sparse_mla {
namespace warp_mma {

constexpr int kThreads = 256;
constexpr int kChunkRows = 64;
constexpr int kChunks = kSlots / kChunkRows;           // 10
constexpr int kTileBytes = kChunkRows * kRowBytes;     // 64 KiB: Q tile and each KV stage
constexpr int kProbBytes = kHeads * kChunkRows * 2;    // 8 KiB
constexpr int kSmemQ = 0;
constexpr int kSmemKv = kSmemQ + kTileBytes;           // two stages
constexpr int kSmemP = kSmemKv + 2 * kTileBytes;
constexpr int kSmemRows = kSmemP + kProbBytes;         // int[640]
constexpr int kSmemMax = kSmemRows + kSlots * 4;       // float[2][64]
constexpr int kSmemSum = kSmemMax + 2 * kHeads * 4;    // float[2][64]
constexpr int kSmemScratch = kSmemSum + 2 * kHeads * 4;
constexpr int kSmemBytes = kSmemScratch + 16;

template <typename T> struct Storage;
template <> struct Storage<__nv_bfloat16> {
  using Pair = __nv_bfloat162;
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct Storage<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Byte offset of 16-byte unit `unit` of row `row` in a tile of 1 KiB rows (64 units per row).
// The low three unit bits are XORed with the row so that eight consecutive rows of one unit
// column fall into eight different bank groups.
__device__ __forceinline__ uint32_t tile_offset(int row, int unit) {
  return row * kRowBytes + ((unit ^ (row & 7)) << 4);
}
// Same for the probability tile: rows of 128 bytes (8 units).
__device__ __forceinline__ uint32_t prob_offset(int row, int unit) {
  return row * 128 + ((unit ^ (row & 7)) << 4);
}

// Fetch one 64-row chunk of the token's slots into `stage`; masked slots are zero-filled so the
// tile never holds non-finite leftovers.
__device__ __forceinline__ void fetch_chunk(const Params& p, const int* rows, int chunk,
                                            uint32_t stage) {
  const char* window_base = static_cast<const char*>(p.ori_kv);
  const char* compressed_base = static_cast<const char*>(p.cmp_kv);
  const int unit = threadIdx.x & 63;
  for (int r = threadIdx.x >> 6; r < kChunkRows; r += kThreads / 64) {
    const int slot = chunk * kChunkRows + r;
    const int row = rows[slot];
    const uint32_t dst = stage + tile_offset(r, unit);
    if (row >= 0) {
      const char* base = slot < kWindow ? window_base : compressed_base;
      cp_async16(dst, base + (size_t)row * kRowBytes + unit * 16);
    } else {
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(dst), "r"(0));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) attention_kernel(const Params p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);
  int* rows = reinterpret_cast<int*>(smem + kSmemRows);
  float* chunk_max = reinterpret_cast<float*>(smem + kSmemMax);
  float* chunk_sum = reinterpret_cast<float*>(smem + kSmemSum);
  int* scratch = reinterpret_cast<int*>(smem + kSmemScratch);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head_group = warp & 3;   // heads [16*head_group, +16)
  const int half = warp >> 2;        // QK: kv rows [32*half, +32) of a chunk; PV: features [256*half, +256)
  const int quad_row = lane >> 2, quad_col = lane & 3;
  const int head0 = head_group * 16 + quad_row, head1 = head0 + 8;

  for (int token = blockIdx.x; token < p.tokens; token += gridDim.x) {
    __syncthreads();  // previous token's readers of rows / tiles are done
    resolve_token_rows(p, token, rows, scratch);

    // Q tile and the first chunk.
    {
      const char* q = static_cast<const char*>(p.q) + (size_t)token * kHeads * kRowBytes;
      const int unit = threadIdx.x & 63;
      for (int r = threadIdx.x >> 6; r < kHeads; r += kThreads / 64)
        cp_async16(smem_base + kSmemQ + tile_offset(r, unit), q + (size_t)r * kRowBytes + unit * 16);
    }
    fetch_chunk(p, rows, 0, smem_base + kSmemKv);
    cp_async_commit();

    float acc[32][4];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    // Running maximum starts at the sink (log2 domain); the sink's own weight exp2(0) = 1 is
    // carried by the first half-warp pair only, so that it enters the denominator once.
    const float sink0 = __ldg(p.sinks + head0) * 1.4426950408889634f;
    const float sink1 = __ldg(p.sinks + head1) * 1.4426950408889634f;
    float run_max0 = sink0, run_max1 = sink1;
    float run_sum0 = half == 0 ? 1.f : 0.f, run_sum1 = run_sum0;
    int live_rows = 0;

    for (int chunk = 0; chunk < kChunks; ++chunk) {
      const uint32_t stage = smem_base + kSmemKv + (chunk & 1) * kTileBytes;
      if (chunk + 1 < kChunks) {
        fetch_chunk(p, rows, chunk + 1, smem_base + kSmemKv + ((chunk + 1) & 1) * kTileBytes);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();

      // ---- S = Q X^T for 16 heads x 32 rows per warp -------------------------------------
      float s[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 4
      for (int k = 0; k < kFeatures / 16; ++k) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, smem_base + kSmemQ + tile_offset(head_group * 16 + (lane & 15), 2 * k + (lane >> 4)));
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
          const int row = half * 32 + pair * 16 + (lane & 7) + ((lane >> 4) << 3);
          ldmatrix_x4(b, stage + tile_offset(row, 2 * k + ((lane >> 3) & 1)));
          Storage<T>::mma(s[2 * pair], a, b[0], b[1]);
          Storage<T>::mma(s[2 * pair + 1], a, b[2], b[3]);
        }
      }

      // ---- mask, scale, chunk maximum -----------------------------------------------------
      float max0 = -INFINITY, max1 = -INFINITY;
#pragma unroll
      for (int tile = 0; tile < 4; ++tile) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int slot = chunk * kChunkRows + half * 32 + tile * 8 + quad_col * 2 + e;
          const bool live = rows[slot] >= 0;
          live_rows += live;
          s[tile][e] = live ? s[tile][e] * p.scale_log2 : -INFINITY;
          s[tile][2 + e] = live ? s[tile][2 + e] * p.scale_log2 : -INFINITY;
          max0 = fmaxf(max0, s[tile][e]);
          max1 = fmaxf(max1, s[tile][2 + e]);
        }
      }
      max0 = fmaxf(max0, __shfl_xor_sync(0xffffffffu, max0, 1));
      max0 = fmaxf(max0, __shfl_xor_sync(0xffffffffu, max0, 2));
      max1 = fmaxf(max1, __shfl_xor_sync(0xffffffffu, max1, 1));
      max1 = fmaxf(max1, __shfl_xor_sync(0xffffffffu, max1, 2));
      if (quad_col == 0) {
        chunk_max[half * kHeads + head0] = max0;
        chunk_max[half * kHeads + head1] = max1;
      }
      __syncthreads();
      const float new_max0 = fmaxf(run_max0, fmaxf(chunk_max[head0], chunk_max[kHeads + head0]));
      const float new_max1 = fmaxf(run_max1, fmaxf(chunk_max[head1], chunk_max[kHeads + head1]));
      const float alpha0 = exp2f(run_max0 - new_max0), alpha1 = exp2f(run_max1 - new_max1);
      run_max0 = new_max0;
      run_max1 = new_max1;

      // ---- probabilities: FP32 sums, storage-type P tile ---------------------------------
      float sum0 = 0.f, sum1 = 0.f;
      unsigned char* prob = smem + kSmemP;
#pragma unroll
      for (int tile = 0; tile < 4; ++tile) {
        const float p00 = exp2f(s[tile][0] - new_max0), p01 = exp2f(s[tile][1] - new_max0);
        const float p10 = exp2f(s[tile][2] - new_max1), p11 = exp2f(s[tile][3] - new_max1);
        sum0 += p00 + p01;
        sum1 += p10 + p11;
        const int unit = half * 4 + tile;  // 8 kv rows = one 16-byte unit
        *reinterpret_cast<uint32_t*>(prob + prob_offset(head0, unit) + quad_col * 4) = Storage<T>::pack(p00, p01);
        *reinterpret_cast<uint32_t*>(prob + prob_offset(head1, unit) + quad_col * 4) = Storage<T>::pack(p10, p11);
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      run_sum0 = run_sum0 * alpha0 + sum0;
      run_sum1 = run_sum1 * alpha1 + sum1;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        acc[i][0] *= alpha0; acc[i][1] *= alpha0;
        acc[i][2] *= alpha1; acc[i][3] *= alpha1;
      }
      __syncthreads();

      // ---- O += P X for 16 heads x 256 features per warp -----------------------------------
#pragma unroll
      for (int k = 0; k < kChunkRows / 16; ++k) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, smem_base + kSmemP + prob_offset(head_group * 16 + (lane & 15), 2 * k + (lane >> 4)));
        const int row = k * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int pair = 0; pair < 16; ++pair) {
          ldmatrix_x4_trans(b, stage + tile_offset(row, half * 32 + pair * 2 + (lane >> 4)));
          Storage<T>::mma(acc[2 * pair], a, b[0], b[1]);
          Storage<T>::mma(acc[2 * pair + 1], a, b[2], b[3]);
        }
      }
      __syncthreads();  // tile, P and chunk_max are free for the next chunk
    }

    // ---- one denominator per head, normalise, store ---------------------------------------
    if (quad_col == 0) {
      chunk_sum[half * kHeads + head0] = run_sum0;
      chunk_sum[half * kHeads + head1] = run_sum1;
    }
    const int any_live = __syncthreads_or(live_rows);
    // No visible row at all: the output row is zero whatever the sink.
    const float inv0 = any_live ? 1.f / (chunk_sum[head0] + chunk_sum[kHeads + head0]) : 0.f;
    const float inv1 = any_live ? 1.f / (chunk_sum[head1] + chunk_sum[kHeads + head1]) : 0.f;
    char* out = static_cast<char*>(p.out) + (size_t)token * kHeads * kRowBytes;
#pragma unroll
    for (int tile = 0; tile < 32; ++tile) {
      const int column = half * 256 + tile * 8 + quad_col * 2;
      *reinterpret_cast<uint32_t*>(out + (size_t)head0 * kRowBytes + column * 2) =
          Storage<T>::pack(acc[tile][0] * inv0, acc[tile][1] * inv0);
      *reinterpret_cast<uint32_t*>(out + (size_t)head1 * kRowBytes + column * 2) =
          Storage<T>::pack(acc[tile][2] * inv1, acc[tile][3] * inv1);
    }
  }
}

}  // namespace warp_mma
}  // namespace sparse_mla
