/*
 * C ABI of the B200 (sm_100a) sparse MLA attention operator.
 *
 * The four per-kernel symbols are the ones the reference's generated launcher
 * exports for its `sparse_mla` entry and that its host runtime binds:
 *   emitted by   src/backend/structured.py:573-649  (launch_, kernel_config_, kernel_metadata_)
 *                src/backend/workspace.py:93-130    (workspace_size_)
 *   consumed by  src/runtime/kernel.py:12-63        (KernelLaunch)
 *                src/runtime/torch.py:63-88         (TensorKernel reads the metadata JSON)
 * Tensor order, names, layouts and dtypes follow the operator signature at
 * examples/sparse_attention/attention.py:210-224.
 *
 * Differences from the reference launcher, all inside what its ABI allows:
 *  - The reference bakes every size in at compile time and so has no scalar
 *    parameters. Here H=64, D=512, WINDOW=128, TOPK=512, PAGE=128 are fixed and
 *    B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE are the trailing int64
 *    "runtime size" parameters the ABI provides (src/backend/structured.py:586,
 *    src/runtime/torch.py:133-159), so one library serves every request shape.
 *    PAGES = MAX_SEQ / 128 is the block-table width; CMP_PAGE = 128 / RATIO is
 *    the row count of a compressed page (64 for C2, 128 for C1).
 *  - `target` in the metadata is "sm_100a" (the reference writes "dav-2201").
 *  - The workspace is small: a status block (the rest of its 1024 bytes is reserved).
 *
 * Every function returns 0 on success. `launch_*` only enqueues work on the
 * given CUDA stream and never synchronises; a non-zero value is the CUDA error
 * code of the failed enqueue. Input legality (monotone cu_seqlens_q, in-range
 * indices, finite data) is the caller's contract, as in the reference
 * (docs/operators/sparse-mla.md:83-87); out-of-range page or row numbers are
 * nevertheless masked instead of dereferenced and reported in the status block.
 *
 * All pointers are device pointers valid on the current device, except
 * `stream` (a cudaStream_t) and where a comment says "host".
 */
#ifndef ASCENDFLOW_B200_SPARSE_MLA_H_
#define ASCENDFLOW_B200_SPARSE_MLA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPARSE_MLA_HEADS 64
#define SPARSE_MLA_FEATURES 512
#define SPARSE_MLA_WINDOW 128
#define SPARSE_MLA_TOPK 512
#define SPARSE_MLA_SLOTS 640 /* WINDOW + TOPK */
#define SPARSE_MLA_PAGE 128
#define SPARSE_MLA_TENSORS 13
#define SPARSE_MLA_PARAMETERS 6

/* Status block: the first SPARSE_MLA_STATUS_WORDS int32 words of the workspace. */
#define SPARSE_MLA_STATUS_WORDS 8
#define SPARSE_MLA_STATUS_OK 0
#define SPARSE_MLA_STATUS_BAD_PAGE 1    /* block-table entry outside [0, blocks): slot masked   */
#define SPARSE_MLA_STATUS_WAIT_EXPIRED 2 /* a bounded on-chip wait gave up: output is not valid  */

/* ---- BF16 kernel "sparse_mla" ------------------------------------------------------------- */

/* cfg = {tensors = 13, parameters = 6, has_workspace = 1, 0, 0}; -1 when cfg is NULL.
 * The last two words are the reference's cube/vector core counts used to match a build to a
 * device (src/runtime/kernel.py:32-38); 0 means "any device of the target".
 * Replaces: kernel_config_sparse_mla (src/backend/structured.py:626-631). */
int kernel_config_sparse_mla(int64_t cfg[5]);

/* Static JSON, ABI version 1, same keys as src/backend/abi.py:43-59. Shape entries are integers,
 * parameter names, {"mul":[a,b]} or {"add":[a,b]} (the latter only for cu_seqlens_q = B + 1).
 * Replaces: kernel_metadata_sparse_mla (src/backend/structured.py:633-635). */
const char* kernel_metadata_sparse_mla(void);

/* Workspace bytes for the given sizes, a multiple of 512. -1 when `bytes` (host) is NULL, a size is
 * negative, or a product would overflow int64.
 * Replaces: workspace_size_sparse_mla (src/backend/workspace.py:93-130). */
int workspace_size_sparse_mla(uint64_t* bytes, int64_t B, int64_t T, int64_t PAGES,
                              int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE);

/* Enqueue one attention call. Argument order: stream, the 13 tensors in signature order, the
 * workspace, then the runtime sizes (docs/guide/workspace.md:74-76 of the reference).
 *   q                  [T, 64, 512]               bf16   read
 *   ori_kv             [ORI_BLOCKS, 128, 1, 512]  bf16   read
 *   cmp_kv             [CMP_BLOCKS, CMP_PAGE, 1, 512] bf16 read
 *   cmp_sparse_indices [T, 1, 512]                int32  read
 *   ori_block_table    [B, PAGES]                 int32  read
 *   cmp_block_table    [B, PAGES]                 int32  read
 *   cu_seqlens_q       [B + 1]                    int32  read
 *   seqused_ori_kv     [B]                        int32  read
 *   seqused_cmp_kv     [B]                        int32  read
 *   cmp_residual_kv    [B]                        int32  read
 *   ori_topk_length    [T, 1]                     int32  read
 *   sinks              [64]                       f32    read
 *   attention_out      [T, 64, 512]               bf16   write, disjoint from every input
 * The softmax scale is 512^-0.5.
 * Replaces: launch_sparse_mla (src/backend/structured.py:637-648). */
int launch_sparse_mla(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                      void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                      void* arg_cmp_block_table, void* arg_cu_seqlens_q, void* arg_seqused_ori_kv,
                      void* arg_seqused_cmp_kv, void* arg_cmp_residual_kv,
                      void* arg_ori_topk_length, void* arg_sinks, void* arg_attention_out,
                      void* npu_workspace, int64_t B, int64_t T, int64_t PAGES,
                      int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE);

/* ---- FP16 kernel "sparse_mla_f16": same contract with q / caches / output in IEEE half.
 * The reference builds this as the DTYPE=f16 specialisation of the same entry
 * (examples/sparse_attention/attention.py:244, benchmarks/attention/run_sparse.py:373-374). */
int kernel_config_sparse_mla_f16(int64_t cfg[5]);
const char* kernel_metadata_sparse_mla_f16(void);
int workspace_size_sparse_mla_f16(uint64_t* bytes, int64_t B, int64_t T, int64_t PAGES,
                                  int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE);
int launch_sparse_mla_f16(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                          void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                          void* arg_cmp_block_table, void* arg_cu_seqlens_q,
                          void* arg_seqused_ori_kv, void* arg_seqused_cmp_kv,
                          void* arg_cmp_residual_kv, void* arg_ori_topk_length, void* arg_sinks,
                          void* arg_attention_out, void* npu_workspace, int64_t B, int64_t T,
                          int64_t PAGES, int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE);

/* ---- BF16 cross-check kernel: the same operator on the warp-level tensor instructions
 * (ldmatrix + mma.sync) instead of tcgen05. Same arguments and contract as launch_sparse_mla.
 * It has no counterpart in the reference; tests compare the two implementations on full-size
 * inputs where the CPU oracle can only afford a sample. */
int launch_sparse_mla_warp_mma(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                               void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                               void* arg_cmp_block_table, void* arg_cu_seqlens_q,
                               void* arg_seqused_ori_kv, void* arg_seqused_cmp_kv,
                               void* arg_cmp_residual_kv, void* arg_ori_topk_length,
                               void* arg_sinks, void* arg_attention_out, void* npu_workspace,
                               int64_t B, int64_t T, int64_t PAGES, int64_t ORI_BLOCKS,
                               int64_t CMP_BLOCKS, int64_t CMP_PAGE);

/* ---- Gathered index set export -------------------------------------------------------------
 * Writes, for every token and slot 0..639, the physical cache row the attention kernel gathers
 * (a row of ori_kv viewed as [ORI_BLOCKS*128, 512] for slots < 128, a row of cmp_kv viewed as
 * [CMP_BLOCKS*CMP_PAGE, 512] for the rest) or -1 for a masked slot. One warp per token runs
 * `resolve_token_warp`, the device routine that the resolver warp of the tcgen05 attention
 * kernels (launch_sparse_mla, launch_sparse_mla_f16) runs for every token it gathers; the
 * warp-MMA cross-check kernel keeps its own block-wide routine. The reference checks the same fact by
 * reading back its gather workspace (benchmarks/attention/run_sparse.py:111-130, 253-262);
 * this kernel keeps gathered rows on chip, so the set is exported instead.
 *   resolved_rows [T, 640] int32 write */
int launch_sparse_mla_resolve_rows(void* stream, void* arg_cmp_sparse_indices,
                                   void* arg_ori_block_table, void* arg_cmp_block_table,
                                   void* arg_cu_seqlens_q, void* arg_seqused_ori_kv,
                                   void* arg_seqused_cmp_kv, void* arg_cmp_residual_kv,
                                   void* arg_ori_topk_length, void* arg_resolved_rows,
                                   void* npu_workspace, int64_t B, int64_t T, int64_t PAGES,
                                   int64_t ORI_BLOCKS, int64_t CMP_BLOCKS, int64_t CMP_PAGE);

/* ---- Attention launch that allocates nothing ---------------------------------------------------
 * No counterpart in the reference (its runtime always owns a malloc'ed workspace arena,
 * src/runtime/kernel.py:39-49). Same operator, kernel and tensor contract as launch_sparse_mla,
 * for callers that must not or cannot allocate device memory around the call: code running
 * under an allocator freeze (inside a serving engine's memory-planned step, a plugin whose
 * host hands it a fixed arena, a process that has already given the whole GPU to a pool) and
 * has no workspace to pass. The workspace lives in a static device array inside this library
 * instead: SPARSE_MLA_STATIC_WORKSPACE_BYTES per GPU, held from library load until the
 * process exits.
 *  - The function calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - The first call on each device looks the array's device address up (cudaGetSymbolAddress);
 *    make that first call outside any stream capture.
 *  - Sizes whose workspace would exceed the array are refused with
 *    SPARSE_MLA_STATIC_WORKSPACE_TOO_SMALL (today every legal size needs 1024 bytes and fits);
 *    invalid sizes return -1 as in launch_sparse_mla.
 *  - All calls on a device share the one array. It is cleared on the stream before each launch,
 *    so calls on the same stream are safe back to back; calls that overlap on the GPU
 *    (different streams, different threads) race on it and must not be made.
 *  - The status block of the last such call is read with read_status_sparse_mla(stream, NULL, ..). */
#define SPARSE_MLA_STATIC_WORKSPACE_BYTES 1024
#define SPARSE_MLA_STATIC_WORKSPACE_TOO_SMALL (-2)
int launch_sparse_mla_static_workspace(void* stream, void* arg_q, void* arg_ori_kv, void* arg_cmp_kv,
                                       void* arg_cmp_sparse_indices, void* arg_ori_block_table,
                                       void* arg_cmp_block_table, void* arg_cu_seqlens_q,
                                       void* arg_seqused_ori_kv, void* arg_seqused_cmp_kv,
                                       void* arg_cmp_residual_kv, void* arg_ori_topk_length,
                                       void* arg_sinks, void* arg_attention_out, int64_t B, int64_t T,
                                       int64_t PAGES, int64_t ORI_BLOCKS, int64_t CMP_BLOCKS,
                                       int64_t CMP_PAGE);

/* ---- The steps on either side of the operator whose output the operator's inputs fix ----------
 * No counterpart in the reference: it leaves the indexer, the compressor and the cache writes
 * to its caller (docs/operators/sparse-mla.md:8, 263-266). These two produce, on the device,
 * the two inputs of the attention call that change with every step, in the format it reads
 * (docs/operators/sparse-mla.md:62-87).
 *
 * launch_sparse_mla_topk_indices: for every query token, the indices of the TopK = 512 highest
 * scores among the compressed rows the token may see, i.e. rows [0, min(C, cutoff)) with the
 * operator's cutoff = max(0, C R + r - n + j + 1) / R; fewer visible rows than 512: all of them.
 * Ties go to the lower index. Winners are written in ascending order, the rest is -1: exactly
 * what `cmp_sparse_indices` is. Scores must be finite.
 *   scores               [T, SPAN]   f32  read  (row stride SPAN, a multiple of 4;
 *                                                 columns beyond a token's visible rows are ignored)
 *   cu_seqlens_q         [B + 1]     i32  read
 *   seqused_cmp_kv       [B]         i32  read
 *   cmp_residual_kv      [B]         i32  read
 *   cmp_sparse_indices   [T, 1, 512] i32  write
 * Returns -1 for sizes out of range (B, T >= 1; SPAN as above; CMP_PAGE 64 or 128, which gives R). */
int launch_sparse_mla_topk_indices(void* stream, void* arg_scores, void* arg_cu_seqlens_q,
                                   void* arg_seqused_cmp_kv, void* arg_cmp_residual_kv,
                                   void* arg_cmp_sparse_indices, int64_t B, int64_t T, int64_t SPAN,
                                   int64_t CMP_PAGE);

/* launch_sparse_mla_cache_append: writes a call's T new rows into a paged cache: row j of the n
 * of request b goes to logical position L_b - n + j, L_b = seqused_kv[b] INCLUDING the new rows
 * (the convention of the attention call that follows), through the request's block table.
 * A position without a legal page is not written and is reported in the status block of
 * `npu_workspace` (SPARSE_MLA_STATUS_BAD_PAGE, token, position).
 *   new_rows      [T, 512]                    b16  read
 *   cache         [BLOCKS, PAGE_ROWS, 1, 512] b16  write (rows not addressed keep their contents)
 *   block_table   [B, PAGES]                  i32  read
 *   cu_seqlens_q  [B + 1]                     i32  read
 *   seqused_kv    [B]                         i32  read
 * `npu_workspace`: workspace_size_sparse_mla bytes. PAGE_ROWS 128 (raw cache) or 64. */
int launch_sparse_mla_cache_append(void* stream, void* arg_new_rows, void* arg_cache,
                                   void* arg_block_table, void* arg_cu_seqlens_q, void* arg_seqused_kv,
                                   void* npu_workspace, int64_t B, int64_t T, int64_t PAGES,
                                   int64_t BLOCKS, int64_t PAGE_ROWS);

/* Self-test of the bounded on-chip wait (no counterpart in the reference, whose synchronisation
 * is proven at compile time): one warp waits on a barrier nobody signals; after `limit_cycles`
 * SM clocks (<= 2^31) it gives up, writes SPARSE_MLA_STATUS_WAIT_EXPIRED to the status block of
 * `npu_workspace` and returns normally, leaving the context usable. The attention kernels use
 * the same wait for every barrier, with a limit of 2^31 clocks (about a second). */
int launch_sparse_mla_wait_expiry_selftest(void* stream, void* npu_workspace, int64_t limit_cycles);

/* Copies the status block of a workspace to `host_words` (host, SPARSE_MLA_STATUS_WORDS int32)
 * after synchronising `stream`. word 0: a SPARSE_MLA_STATUS_* code, word 1: token, word 2: detail.
 * `npu_workspace` == NULL reads the static array of launch_sparse_mla_static_workspace on the
 * current device (no allocation: the array's address is looked up once per device). */
int read_status_sparse_mla(void* stream, void* npu_workspace, int32_t* host_words);

#ifdef __cplusplus
}
#endif
#endif /* ASCENDFLOW_B200_SPARSE_MLA_H_ */
