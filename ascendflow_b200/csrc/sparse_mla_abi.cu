// C ABI of the sparse MLA operator: the four per-kernel host symbols of the reference's
// generated launcher (src/backend/structured.py:573-649, src/backend/workspace.py:93-130 of the
// reference) re-exported over hand-written sm_100a kernels. Declarations and the full contract
// are in include/sparse_mla.h.
//
// Like the reference launcher, `launch_*` forwards and enqueues only: no device
// synchronisation, no input validation (that is the host binding's job).

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sparse_mla.h"
#include "sparse_mla_common.cuh"
#include "sparse_mla_mma_sync.cuh"
#include "sparse_mla_tcgen05.cuh"

namespace sparse_mla {
namespace {

// Self-test of the bounded wait every role of the attention kernel uses: one warp waits on a
// barrier that nobody arrives on; the wait must give up after `limit` clocks, record
// kStatusWaitExpired and let the kernel return normally.
__global__ void wait_expiry_kernel(int32_t* status, long long limit) {
  __shared__ uint64_t barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(sm100::smem_u32(&barrier), 1);
    sm100::mbar_fence_init();
    abort_flag = 0;
  }
  __syncthreads();
  const bool arrived = sm100::mbar_wait(sm100::smem_u32(&barrier), 0, &abort_flag, limit);
  __syncthreads();
  if (threadIdx.x == 0 && !arrived && atomicCAS(status, kStatusOk, kStatusWaitExpired) == kStatusOk) {
    status[1] = -1;
    status[2] = abort_flag;
  }
}

#define SPARSE_MLA_METADATA(NAME, DTYPE)                                                          \
  "{\"version\":1,\"name\":\"" NAME "\",\"target\":\"sm_100a\",\"kind\":\"mixed\",\"groups\":148," \
  "\"disjoint_external\":true,\"device_resources\":null,\"tensors\":["                            \
  "{\"name\":\"q\",\"dtype\":\"" DTYPE "\",\"shape\":[\"T\",64,512],\"layout\":\"linear\",\"access\":\"read\"},"  \
  "{\"name\":\"ori_kv\",\"dtype\":\"" DTYPE "\",\"shape\":[\"ORI_BLOCKS\",128,1,512],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"cmp_kv\",\"dtype\":\"" DTYPE "\",\"shape\":[\"CMP_BLOCKS\",\"CMP_PAGE\",1,512],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"cmp_sparse_indices\",\"dtype\":\"i32\",\"shape\":[\"T\",1,512],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"ori_block_table\",\"dtype\":\"i32\",\"shape\":[\"B\",\"PAGES\"],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"cmp_block_table\",\"dtype\":\"i32\",\"shape\":[\"B\",\"PAGES\"],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"cu_seqlens_q\",\"dtype\":\"i32\",\"shape\":[{\"add\":[\"B\",1]}],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"seqused_ori_kv\",\"dtype\":\"i32\",\"shape\":[\"B\"],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"seqused_cmp_kv\",\"dtype\":\"i32\",\"shape\":[\"B\"],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"cmp_residual_kv\",\"dtype\":\"i32\",\"shape\":[\"B\"],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"ori_topk_length\",\"dtype\":\"i32\",\"shape\":[\"T\",1],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"sinks\",\"dtype\":\"f32\",\"shape\":[64],\"layout\":\"linear\",\"access\":\"read\"}," \
  "{\"name\":\"attention_out\",\"dtype\":\"" DTYPE "\",\"shape\":[\"T\",64,512],\"layout\":\"linear\",\"access\":\"write\"}]," \
  "\"parameters\":["                                                                             \
  "{\"name\":\"B\",\"minimum\":1,\"multiple\":1},{\"name\":\"T\",\"minimum\":1,\"multiple\":1},"  \
  "{\"name\":\"PAGES\",\"minimum\":1,\"multiple\":1},{\"name\":\"ORI_BLOCKS\",\"minimum\":1,\"multiple\":1}," \
  "{\"name\":\"CMP_BLOCKS\",\"minimum\":1,\"multiple\":1},{\"name\":\"CMP_PAGE\",\"minimum\":64,\"multiple\":64}]," \
  "\"workspace\":true}"

int config(int64_t* cfg) {
  if (cfg == nullptr) return -1;
  cfg[0] = SPARSE_MLA_TENSORS;
  cfg[1] = SPARSE_MLA_PARAMETERS;
  cfg[2] = 1;
  cfg[3] = 0;
  cfg[4] = 0;
  return 0;
}

int workspace_size(uint64_t* bytes, int64_t B, int64_t T, int64_t PAGES, int64_t ORI_BLOCKS,
                   int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  if (bytes == nullptr) return -1;
  *bytes = 0;
  if (B < 0 || T < 0 || PAGES < 0 || ORI_BLOCKS < 0 || CMP_BLOCKS < 0 || CMP_PAGE < 0) return -1;
  // The extents the kernels index with must fit int64 byte offsets and int32 row numbers.
  const uint64_t limit = uint64_t(INT64_MAX);
  const uint64_t row_bytes = uint64_t(kRowBytes);
  auto product_fits = [&](uint64_t a, uint64_t b, uint64_t bound) { return b == 0 || a <= bound / b; };
  if (!product_fits(uint64_t(T), uint64_t(kHeads) * row_bytes, limit)) return -1;
  if (!product_fits(uint64_t(ORI_BLOCKS), uint64_t(kPage) * row_bytes, limit)) return -1;
  if (!product_fits(uint64_t(CMP_BLOCKS), uint64_t(kPage) * row_bytes, limit)) return -1;
  if (!product_fits(uint64_t(B), uint64_t(PAGES) * 4u + 4u, limit)) return -1;
  if (!product_fits(uint64_t(T), uint64_t(kSlots) * 4u, limit)) return -1;
  *bytes = (uint64_t(kWorkspaceBytes) + 511u) / 512u * 512u;
  return 0;
}

bool fill(Params& p, void* q, void* ori_kv, void* cmp_kv, void* indices, void* ori_table,
          void* cmp_table, void* cu, void* seq_ori, void* seq_cmp, void* residual, void* topk_len,
          void* sinks, void* out, void* workspace, int64_t B, int64_t T, int64_t PAGES,
          int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  if (B <= 0 || T <= 0 || PAGES <= 0 || workspace == nullptr) return false;
  if (CMP_PAGE != 64 && CMP_PAGE != 128) return false;
  if (B > INT32_MAX || T > INT32_MAX || PAGES > INT32_MAX) return false;
  if (ORI_BLOCKS < 0 || CMP_BLOCKS < 0) return false;  // the kernels' page check is unsigned
  if (ORI_BLOCKS > INT32_MAX / kPage || CMP_BLOCKS > INT32_MAX / kPage) return false;
  p.q = q; p.ori_kv = ori_kv; p.cmp_kv = cmp_kv;
  p.indices = static_cast<const int32_t*>(indices);
  p.ori_table = static_cast<const int32_t*>(ori_table);
  p.cmp_table = static_cast<const int32_t*>(cmp_table);
  p.cu = static_cast<const int32_t*>(cu);
  p.seq_ori = static_cast<const int32_t*>(seq_ori);
  p.seq_cmp = static_cast<const int32_t*>(seq_cmp);
  p.residual = static_cast<const int32_t*>(residual);
  p.topk_len = static_cast<const int32_t*>(topk_len);
  p.sinks = static_cast<const float*>(sinks);
  p.out = out;
  p.status = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + kWorkspaceStatusOffset);
  p.batches = int32_t(B); p.tokens = int32_t(T); p.pages = int32_t(PAGES);
  p.cmp_page = int32_t(CMP_PAGE); p.ratio = int32_t(kPage / CMP_PAGE);
  p.ori_blocks = int32_t(ORI_BLOCKS); p.cmp_blocks = int32_t(CMP_BLOCKS);
  p.scale_log2 = 0.044194173824159216f * 1.4426950408889634f;  // 512^-0.5 * log2(e)
  p.token_group = 1;
  return true;
}

int multiprocessors() {
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    cached[device] = count;
  }
  return cached[device];
}

// The shared-memory attribute of a kernel is a per-device setting: one flag per device. (The
// per-device caches of this file are plain words written with the same value by whoever gets
// there first: concurrent first calls repeat the set-up, nothing else.)
template <typename Kernel>
int configure_once(Kernel kernel, int bytes, bool (&done)[64]) {
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return int(error);
  if (device < 0 || device >= 64) return -1;
  if (done[device]) return 0;
  error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (error != cudaSuccess) return int(error);
  done[device] = true;
  return 0;
}

int clear_workspace(cudaStream_t stream, void* workspace) {
  return int(cudaMemsetAsync(workspace, 0, kWorkspaceBytes, stream));
}

// Scratch of the entry point that allocates nothing: the workspace of one attention launch
// (the status block) as a file-scope device array. Every GPU that loads this
// library holds these bytes until the process exits. In host code the name below is only a
// host-side stand-in for the device array, never a device address: the address a kernel can use
// comes from cudaGetSymbolAddress, once per device, with that device current.
constexpr size_t kStaticWorkspaceBytes = SPARSE_MLA_STATIC_WORKSPACE_BYTES;
static_assert(kStaticWorkspaceBytes >= size_t(kWorkspaceBytes),
              "the static array must hold the workspace of one attention launch");
static __device__ __align__(256) unsigned char static_workspace[kStaticWorkspaceBytes];

// Device address of `static_workspace` on the current device; nullptr (and *error set) on failure.
void* static_workspace_address(int* error) {
  static void* cached[64] = {nullptr};
  int device = 0;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) { *error = int(status); return nullptr; }
  if (device < 0 || device >= 64) { *error = -1; return nullptr; }
  if (cached[device] == nullptr) {
    void* address = nullptr;
    status = cudaGetSymbolAddress(&address, static_workspace);
    if (status != cudaSuccess || address == nullptr) { *error = status != cudaSuccess ? int(status) : -1; return nullptr; }
    cached[device] = address;
  }
  *error = 0;
  return cached[device];
}

}  // namespace
}  // namespace sparse_mla

using namespace sparse_mla;

extern "C" {

int kernel_config_sparse_mla(int64_t cfg[5]) { return config(cfg); }
int kernel_config_sparse_mla_f16(int64_t cfg[5]) { return config(cfg); }

const char* kernel_metadata_sparse_mla(void) { return SPARSE_MLA_METADATA("sparse_mla", "bf16"); }
const char* kernel_metadata_sparse_mla_f16(void) { return SPARSE_MLA_METADATA("sparse_mla_f16", "f16"); }

int workspace_size_sparse_mla(uint64_t* bytes, int64_t B, int64_t T, int64_t PAGES,
                              int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  return workspace_size(bytes, B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE);
}
int workspace_size_sparse_mla_f16(uint64_t* bytes, int64_t B, int64_t T, int64_t PAGES,
                                  int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  return workspace_size(bytes, B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE);
}

int launch_sparse_mla(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                      void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                      void* arg_cmp_block_table, void* arg_cu_seqlens_q, void* arg_seqused_ori_kv,
                      void* arg_seqused_cmp_kv, void* arg_cmp_residual_kv,
                      void* arg_ori_topk_length, void* arg_sinks, void* arg_attention_out,
                      void* npu_workspace, int64_t B, int64_t T, int64_t PAGES,
                      int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  Params p;
  if (!fill(p, arg_q, arg_ori_kv, arg_cmp_kv, arg_cmp_sparse_indices, arg_ori_block_table,
            arg_cmp_block_table, arg_cu_seqlens_q, arg_seqused_ori_kv, arg_seqused_cmp_kv,
            arg_cmp_residual_kv, arg_ori_topk_length, arg_sinks, arg_attention_out, npu_workspace,
            B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE))
    return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int status = clear_workspace(s, npu_workspace)) return status;
  return umma::launch<1>(p, s, multiprocessors());
}

int launch_sparse_mla_f16(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                          void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                          void* arg_cmp_block_table, void* arg_cu_seqlens_q,
                          void* arg_seqused_ori_kv, void* arg_seqused_cmp_kv,
                          void* arg_cmp_residual_kv, void* arg_ori_topk_length, void* arg_sinks,
                          void* arg_attention_out, void* npu_workspace, int64_t B, int64_t T,
                          int64_t PAGES, int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  Params p;
  if (!fill(p, arg_q, arg_ori_kv, arg_cmp_kv, arg_cmp_sparse_indices, arg_ori_block_table,
            arg_cmp_block_table, arg_cu_seqlens_q, arg_seqused_ori_kv, arg_seqused_cmp_kv,
            arg_cmp_residual_kv, arg_ori_topk_length, arg_sinks, arg_attention_out, npu_workspace,
            B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE))
    return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int status = clear_workspace(s, npu_workspace)) return status;
  return umma::launch<0>(p, s, multiprocessors());
}

// The portable-instruction BF16 kernel under its own name: the cross-check of the tcgen05 kernel.
int launch_sparse_mla_warp_mma(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                               void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                               void* arg_cmp_block_table, void* arg_cu_seqlens_q,
                               void* arg_seqused_ori_kv, void* arg_seqused_cmp_kv,
                               void* arg_cmp_residual_kv, void* arg_ori_topk_length,
                               void* arg_sinks, void* arg_attention_out, void* npu_workspace,
                               int64_t B, int64_t T, int64_t PAGES, int64_t ORI_BLOCKS,
                               int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  Params p;
  if (!fill(p, arg_q, arg_ori_kv, arg_cmp_kv, arg_cmp_sparse_indices, arg_ori_block_table,
            arg_cmp_block_table, arg_cu_seqlens_q, arg_seqused_ori_kv, arg_seqused_cmp_kv,
            arg_cmp_residual_kv, arg_ori_topk_length, arg_sinks, arg_attention_out, npu_workspace,
            B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE))
    return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  static bool configured[64] = {false};
  if (int status = configure_once(warp_mma::attention_kernel<__nv_bfloat16>, warp_mma::kSmemBytes, configured))
    return status;
  if (int status = clear_workspace(s, npu_workspace)) return status;
  const int grid = int(T < int64_t(multiprocessors()) ? T : multiprocessors());
  warp_mma::attention_kernel<__nv_bfloat16><<<grid, warp_mma::kThreads, warp_mma::kSmemBytes, s>>>(p);
  return int(cudaGetLastError());
}

int launch_sparse_mla_resolve_rows(void* stream, void* arg_cmp_sparse_indices,
                                   void* arg_ori_block_table, void* arg_cmp_block_table,
                                   void* arg_cu_seqlens_q, void* arg_seqused_ori_kv,
                                   void* arg_seqused_cmp_kv, void* arg_cmp_residual_kv,
                                   void* arg_ori_topk_length, void* arg_resolved_rows,
                                   void* npu_workspace, int64_t B, int64_t T, int64_t PAGES,
                                   int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE) {
  Params p;
  if (!fill(p, nullptr, nullptr, nullptr, arg_cmp_sparse_indices, arg_ori_block_table,
            arg_cmp_block_table, arg_cu_seqlens_q, arg_seqused_ori_kv, arg_seqused_cmp_kv,
            arg_cmp_residual_kv, arg_ori_topk_length, nullptr, nullptr, npu_workspace, B, T, PAGES,
            ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE))
    return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int status = clear_workspace(s, npu_workspace)) return status;
  const int64_t blocks = (T + 3) / 4, cap = int64_t(multiprocessors()) * 8;  // four warps = four tokens per block
  umma::resolve_rows_kernel<<<int(blocks < cap ? blocks : cap), 128, 0, s>>>(p, static_cast<int32_t*>(arg_resolved_rows));
  return int(cudaGetLastError());
}

int launch_sparse_mla_static_workspace(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                                       void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                                       void* arg_cmp_block_table, void* arg_cu_seqlens_q,
                                       void* arg_seqused_ori_kv, void* arg_seqused_cmp_kv,
                                       void* arg_cmp_residual_kv, void* arg_ori_topk_length,
                                       void* arg_sinks, void* arg_attention_out, int64_t B, int64_t T,
                                       int64_t PAGES, int64_t ORI_BLOCKS, int64_t CMP_BLOCKS,
                                       int64_t CMP_PAGE) {
  uint64_t needed = 0;
  if (workspace_size(&needed, B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE) != 0) return -1;
  if (needed > kStaticWorkspaceBytes) return SPARSE_MLA_STATIC_WORKSPACE_TOO_SMALL;
  int error = 0;
  void* workspace = static_workspace_address(&error);  // first call on a device: symbol look-up
  if (workspace == nullptr) return error;
  Params p;
  if (!fill(p, arg_q, arg_ori_kv, arg_cmp_kv, arg_cmp_sparse_indices, arg_ori_block_table,
            arg_cmp_block_table, arg_cu_seqlens_q, arg_seqused_ori_kv, arg_seqused_cmp_kv,
            arg_cmp_residual_kv, arg_ori_topk_length, arg_sinks, arg_attention_out, workspace,
            B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE))
    return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: the status block must start at zero.
  if (int status = int(cudaMemsetAsync(workspace, 0, kStaticWorkspaceBytes, s))) return status;
  return umma::launch<1>(p, s, multiprocessors());
}

int launch_sparse_mla_wait_expiry_selftest(void* stream, void* npu_workspace, int64_t limit_cycles) {
  if (npu_workspace == nullptr || limit_cycles <= 0 || limit_cycles > (int64_t(1) << 31)) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int status = clear_workspace(s, npu_workspace)) return status;
  wait_expiry_kernel<<<1, 32, 0, s>>>(reinterpret_cast<int32_t*>(static_cast<char*>(npu_workspace) + kWorkspaceStatusOffset),
                                      (long long)limit_cycles);
  return int(cudaGetLastError());
}

int read_status_sparse_mla(void* stream, void* npu_workspace, int32_t* host_words) {
  if (host_words == nullptr) return -1;
  if (npu_workspace == nullptr) {  // the static array of the current device (address already cached
                                   // after the first launch_sparse_mla_static_workspace: no allocation)
    int error = 0;
    npu_workspace = static_workspace_address(&error);
    if (npu_workspace == nullptr) return error;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t error = cudaMemcpyAsync(host_words, static_cast<char*>(npu_workspace) + kWorkspaceStatusOffset,
                                      kStatusWords * sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (error != cudaSuccess) return int(error);
  return int(cudaStreamSynchronize(s));
}

}  // extern "C"
