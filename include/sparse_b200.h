/* libsparse_b200.so -- C ABI of the B200 block-sparse attention hot path.
 *
 * Plain pointers and sizes only. Every pointer is a DEVICE pointer unless the
 * comment says otherwise; `stream` is a cudaStream_t passed as void*. Calls are
 * asynchronous on that stream, never synchronise, never throw. Return value:
 * 0 on success, negative on error (SPARSE_B200_ERR_*), with a message from
 * sparse_b200_last_error(). The device that is current when a function is
 * called is the device it launches on.
 *
 * Layouts (d = 128, bf16 unless stated, all contiguous):
 *   q, out        [B, Hq, Sq, 128]
 *   k, v          [B, Hkv, Skv, 128]
 *   block_idx     [B, Hkv, Sq/128, TopK] int32: KV-block ids chosen for a query
 *                 block, shared by the Hq/Hkv query heads of the KV-head group
 *   block_count   [B, Hkv, Sq/128] int32 or NULL: live entries per list
 *   lse           [B, Hq, Sq] fp32, natural log, or NULL
 */
#ifndef SPARSE_B200_H
#define SPARSE_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPARSE_B200_OK 0
#define SPARSE_B200_ERR_INVALID (-1)
#define SPARSE_B200_ERR_CUDA (-2)
#define SPARSE_B200_ERR_TIMEOUT (-3)

/* Text of the last error raised on the calling thread (host pointer). */
const char* sparse_b200_last_error(void);

/* Reads (and with reset != 0 clears) the device status word. 0 = healthy;
 * a positive value names the bounded wait a kernel abandoned. Synchronises the
 * device; meant for tests and post-mortems, not for the hot path. */
int sparse_b200_device_status(int reset);

/* The same check as a return code: synchronises the device, clears the status word and
 * returns SPARSE_B200_ERR_TIMEOUT (message: the code of the abandoned wait) when a
 * kernel gave up a bounded wait since the last check, else 0. The reference's waits
 * have no limit (attention/q_centric/common.cuh:38-52: a protocol error hangs the GPU);
 * here every wait ends after ~0.8 s at the latest and the outputs of that launch are
 * incomplete. */
int sparse_b200_check_status(void);

/* Exercises that give-up path on purpose, harmlessly: one small CTA waits on an
 * mbarrier nobody arrives on (nothing in flight, no tensor memory held) for at most
 * limit_cycles (<= 1e8) clock cycles, records code 0x7e57 in the status word, raises
 * its abort flag, and exits. observed (2 device ints, may be NULL): [0] = 0 when the
 * wait gave up, [1] = 1 when the CTA's other warp saw the abort flag. No counterpart
 * in the reference. */
int sparse_b200_selftest_bounded_wait(int64_t limit_cycles, int32_t* observed, void* stream);

/* Q-centric block-sparse attention forward.
 * Replaces the launch functions behind xomtention_progression::attention_out
 * (attention/q_centric/progression_attention.cpp:11-15, 96-108:
 * dense14_sparse_two_q_launch / dense14_sparse_gqa_launch), same argument
 * order with block_count and lse added. Group sizes Hq/Hkv that are even share
 * each selected K/V tile between two heads; others pair neighbouring query
 * blocks. A list with count 0 yields out = 0 and lse = -inf. */
int sparse_b200_q_centric(const void* q, const void* k, const void* v, const int32_t* block_idx,
                          const int32_t* block_count, void* out, float* lse, int batch, int hq, int hkv,
                          int sq, int skv, int topk, void* stream);

/* sparse_b200_q_centric with a caller-provided scratch buffer (sparse_b200_q_centric_workspace_bytes()
 * bytes on the current device, 16-byte aligned, private to the call while it runs). With it the kernel
 * balances its last round of work items: when a launch is a few rounds of (query block, head pair)
 * items per SM and the last round would keep at most half of the SMs busy, the items of that round are
 * cut into 2-4 pieces of their lists, the pieces write normalised partials into the workspace and a small
 * kernel merges them (the log-sum-exp merge of sparse_b200_combine). Results of those rows may differ
 * from the unbalanced call in the last bf16 bit; everything else is identical. workspace == NULL is
 * sparse_b200_q_centric. No counterpart in the reference (its kernels take no workspace). */
int64_t sparse_b200_q_centric_workspace_bytes(void);
int sparse_b200_q_centric_ws(const void* q, const void* k, const void* v, const int32_t* block_idx,
                             const int32_t* block_count, void* out, float* lse, void* workspace,
                             int64_t workspace_bytes, int batch, int hq, int hkv, int sq, int skv, int topk,
                             void* stream);

/* Same kernel over `nseg` list sets at once, writing normalised partial
 * outputs [nseg, B, Hq, Sq, 128] (bf16, or fp32 when partial_is_f32) and
 * partial LSE [nseg, B, Hq, Sq]. seg_block_idx is [nseg, B, Hkv, Sq/128, TopK],
 * seg_block_count [nseg, B, Hkv, Sq/128]. This is the "main" stage of the
 * KV-centric operator (role of kv11_launch,
 * attention/kv_centric/optimization_round11/tma11_kernel.cu:439-452): segment
 * s holds the ids of one KV range, segments run KV-range-outer. */
int sparse_b200_q_centric_partial(const void* q, const void* k, const void* v, const int32_t* seg_block_idx,
                                  const int32_t* seg_block_count, void* partial_out, float* partial_lse,
                                  int nseg, int partial_is_f32, int batch, int hq, int hkv, int sq, int skv,
                                  int topk, void* stream);

/* Log-sum-exp merge of `ranks` normalised partial outputs per row:
 * out[row] = sum_r exp(L_r - L) O_r, out_lse[row] = L = logsumexp_r L_r, ranks
 * accumulated in order. rank_major != 0: partial [ranks, rows, 128] and
 * partial_lse [ranks, rows] (what sparse_b200_q_centric_partial writes);
 * rank_major == 0: partial [rows, ranks, 128], partial_lse [rows, ranks] (the
 * layout of kv11_launch_combine_f32 / _bf16,
 * attention/kv_centric/optimization_round11/combine11.cu:63-72, which this
 * replaces for any rank count). A rank with LSE = -inf is ignored. out is bf16
 * [rows, 128]; out_lse may be NULL. Also merges the partials of a KV split
 * across GPUs once they are in local memory. */
int sparse_b200_combine(const void* partial, int partial_is_f32, const float* partial_lse, void* out, float* out_lse,
                        int64_t rows, int ranks, int rank_major, void* stream);

/* Scheduling metadata of the KV-centric operator: cut every selection list into
 * nseg KV ranges of ceil(kv_blocks/nseg) blocks. seg_block_idx
 * [nseg, B, Hkv, q_blocks, TopK], seg_block_count [nseg, B, Hkv, q_blocks];
 * error_word gets bit 1 if an id lies outside [0, kv_blocks) (the caller zeroes
 * it). Role of kv4_build_metadata
 * (attention/kv_centric/optimization_round4/gpu_metadata.cu:82-108). */
int sparse_b200_split_kv_segments(const int32_t* block_idx, const int32_t* block_count, int32_t* seg_block_idx,
                                  int32_t* seg_block_count, int32_t* error_word, int batch, int hkv, int q_blocks,
                                  int topk, int kv_blocks, int nseg, void* stream);

/* Whole KV-centric operator = metadata + main + combine on one stream, the
 * sequence of Prepared.run() (attention/kv_centric/optimization_round11/api11.py:85-92).
 * KV ranges are processed outer; each (query block, KV range) yields one partial
 * (O, LSE), merged per query. `workspace` (device, 256-byte aligned) must hold
 * sparse_b200_kv_centric_workspace_bytes(...) bytes; nothing is allocated. */
int64_t sparse_b200_kv_centric_workspace_bytes(int batch, int hq, int hkv, int sq, int topk, int nseg,
                                               int partial_is_f32);
int sparse_b200_kv_centric(const void* q, const void* k, const void* v, const int32_t* block_idx,
                           const int32_t* block_count, void* out, float* lse, void* workspace,
                           int64_t workspace_bytes, int nseg, int partial_is_f32, int batch, int hq, int hkv, int sq,
                           int skv, int topk, void* stream);

/* KV-centric operator for per-TOKEN selection lists, the reference's own KV-centric
 * contract with a free TopK: selected [B, Hkv, Sq, TopK] int32 (any Sq >= 1).
 * kv_token_metadata builds the reverse index on the GPU: rows = (b*Hkv + kvh)*kv_blocks
 * + block; row_ptr [rows+1], query_ids / ranks [B*Hkv*Sq*TopK] (edge order inside a row
 * is arbitrary), task_ptr [rows+1] (task_ptr[rows] = task count), tasks [max_tasks, 4] =
 * (group, block, first edge, edge count <= 128/group_size); counts and cursors are
 * scratch of rows+1 ints; error_word bit 1 = id out of range. Replaces
 * kv4_build_metadata (attention/kv_centric/optimization_round4/gpu_metadata.cu:82-108).
 * kv_token_main gathers the queries of every task, runs QK / softmax over the one
 * block / PV on the tensor cores and scatters normalised partials [B, Hq, Sq, TopK, 128]
 * bf16 and partial_lse [B, Hq, Sq, TopK]; q is [B, Hq, Sq, 128]. Replaces kv11_launch
 * (attention/kv_centric/optimization_round11/tma11_kernel.cu:439-452). Merge with
 * sparse_b200_combine(partial, 0, partial_lse, out, lse, B*Hq*Sq, TopK, rank_major = 0).
 * An id outside [0, kv_blocks) only raises error_word: its edge is dropped and its
 * (query, rank) slot of partial / partial_lse is NOT written. A caller that cannot rule
 * such ids out fills partial_lse with -inf before kv_token_main (Combine ignores -inf
 * ranks) or reads error_word before merging. */
int64_t sparse_b200_kv_token_max_tasks(int batch, int hkv, int sq, int topk, int kv_blocks, int group_size);
int sparse_b200_kv_token_metadata(const int32_t* selected, int32_t* counts, int32_t* cursors, int32_t* row_ptr,
                                  int32_t* query_ids, int32_t* ranks, int32_t* task_ptr, int32_t* tasks,
                                  int32_t* error_word, int batch, int hkv, int sq, int topk, int kv_blocks,
                                  int group_size, void* stream);
int sparse_b200_kv_token_main(const void* q, const void* k, const void* v, const int32_t* tasks,
                              const int32_t* task_ptr, const int32_t* query_ids, const int32_t* ranks, void* partial,
                              float* partial_lse, int batch, int hq, int hkv, int sq, int skv, int topk,
                              void* stream);
/* The same with q in the token-major layout [B, Sq, Hq, 128] of the reference's TMA variants
 * (main_tm_out, attention/kv_centric/optimization_round11/api11.py:1-7,85-87): the heads of a
 * token are one dense block, which the gather fetches faster. Hq / Hkv of 8 or 16 only. The
 * partials keep the head-major layout [B, Hq, Sq, TopK, 128]. */
int sparse_b200_kv_token_main_tm(const void* q_token_major, const void* k, const void* v, const int32_t* tasks,
                                 const int32_t* task_ptr, const int32_t* query_ids, const int32_t* ranks,
                                 void* partial, float* partial_lse, int batch, int hq, int hkv, int sq, int skv,
                                 int topk, void* stream);
/* The reference's token-major pair as it stands (main_tm_out + combine_tm_out,
 * attention/kv_centric/optimization_round11/wrapper11.cpp:94-133): q [B, Sq, Hq, 128], partials
 * token-major too, [B, Sq, TopK, Hq, 128] bf16; partial_lse stays [B, Hq, Sq, TopK] and the merged
 * output head-major [B, Hq, Sq, 128], as in the reference. Hq / Hkv of 8 or 16; any TopK.
 * Same arithmetic as the head-major entries: the merged output is bit-identical. */
int sparse_b200_kv_token_main_tm_partial_tm(const void* q_token_major, const void* k, const void* v,
                                            const int32_t* tasks, const int32_t* task_ptr, const int32_t* query_ids,
                                            const int32_t* ranks, void* partial_token_major, float* partial_lse,
                                            int batch, int hq, int hkv, int sq, int skv, int topk, void* stream);
/* All layouts of the main stage behind one entry. layout is a mask: bit 0 = q token-major
 * [B, Sq, Hq, 128], bit 1 = partials token-major [B, Sq, TopK, Hq, 128] (needs bit 0), bit 2 =
 * fp32 partials instead of bf16. 0, 1 and 3 are the three entries above; 4 and 7 are the
 * reference's fp32 controls (variants -2 and 0, attention/kv_centric/optimization_round11/
 * api11.py:22-25, wrapper11.cpp:66-70,97-100), merged by sparse_b200_combine /
 * sparse_b200_combine_tm with partial_is_f32 = 1. Token-major layouts: Hq / Hkv of 8 or 16. */
int sparse_b200_kv_token_main_layout(const void* q, const void* k, const void* v, const int32_t* tasks,
                                     const int32_t* task_ptr, const int32_t* query_ids, const int32_t* ranks,
                                     void* partial, float* partial_lse, int batch, int hq, int hkv, int sq, int skv,
                                     int topk, int layout, void* stream);
int sparse_b200_combine_tm(const void* partial_token_major, int partial_is_f32, const float* partial_lse, void* out,
                           float* out_lse, int batch, int hq, int sq, int ranks, void* stream);

/* Cross-GPU merge of the KV-range split over peer memory (one process per GPU, one machine). The
 * reference has no multi-GPU path; this is the fused form of "exchange the (O, LSE) partials, then
 * Combine" for the 1 Mi-token configuration: the merge kernel reads the other ranks' partials with
 * plain loads over NVLink. No multicast, no library kernel on peer memory; every wait on a flag
 * another GPU writes gives up after wait_ms and records a status code (sparse_b200_device_status).
 * peer_alloc: `bytes` of zeroed device memory on the current device and a 64-byte handle that
 * another process turns into a pointer with peer_open (CUDA IPC; the open enables peer access).
 * peer_signal: after everything earlier on the stream, stores `value` into each of `count` (<= 16)
 * flag words (host array of device pointers, usually one word in every rank's memory).
 * peer_wait: a one-thread kernel that returns when each of `count` LOCAL flag words is >= value.
 * combine_peer: rows [rows, 128] bf16 + LSE [rows] from `ranks` (1, 2, 4, 8) sources given as host
 * arrays of device pointers (each already at the caller's first row), merged in rank order with the
 * arithmetic of sparse_b200_combine (bit-identical rows); ready_flags (LOCAL, `ranks` words, or NULL)
 * are awaited >= value before the first load.
 * q_centric_scatter: the attention kernel with its output rows cut into `owners` (1..4) equal slices
 * of the flattened [B*Hq*Sq] axis (whole 128-row tiles), slice j stored to outs[j] ([rows/owners, 128]
 * bf16) and lses[j] ([rows/owners] fp32, required) - host arrays of device pointers that may lie in
 * other GPUs' memory (peer_open): the kernel's TMA stores then carry every finished tile straight to
 * the rank that merges it, under the remaining computation, and the merge reads local memory only. */
int sparse_b200_q_centric_scatter(const void* q, const void* k, const void* v, const int32_t* block_idx,
                                  const int32_t* block_count, void* const* outs, float* const* lses, int owners,
                                  int batch, int hq, int hkv, int sq, int skv, int topk, void* stream);
int sparse_b200_peer_alloc(int64_t bytes, void** ptr, void* handle64);
int sparse_b200_peer_open(const void* handle64, void** ptr);
int sparse_b200_peer_close(void* ptr);
int sparse_b200_peer_free(void* ptr);
int sparse_b200_peer_signal(int32_t* const* flags, int count, int value, void* stream);
int sparse_b200_peer_wait(const int32_t* flags, int count, int value, int wait_ms, void* stream);
int sparse_b200_combine_peer(const void* const* partials, const float* const* partial_lses, const int32_t* ready_flags,
                             int value, int wait_ms, void* out, float* out_lse, int64_t rows, int ranks,
                             void* stream);

/* R1 / R4 block-summary indexer (indexers/r1_r4/gpu_ops.py:6-49,
 * indexers/r1_r4/block_selectors.py:9-45), any Hkv, group size x R <= 64, any TopK.
 * pool_blocks: x [B, H, S, 128] bf16 -> desc [B, H, S/128, R, 128] bf16, the
 * fp32 mean of 128/R consecutive tokens summed in token order.
 * summary_select: score[b, kvh, qb, kb] = 128^-0.5 * max over (heads of the
 * group, R x R representatives) of the descriptor dot product (fp32, feature
 * order); block_idx [B, Hkv, q_blocks, TopK] = top-k by (score descending, id
 * ascending); scores [B, Hkv, q_blocks, kv_blocks] fp32 is optional (NULL).
 * indexer_summary = pool(q), pool(k), select: the whole SummarySelector.run(). */
int sparse_b200_pool_blocks(const void* x, void* desc, int batch, int heads, int seq, int representatives,
                            void* stream);
int sparse_b200_summary_select(const void* q_desc, const void* k_desc, float* scores, int32_t* block_idx, int batch,
                               int hq, int hkv, int q_blocks, int kv_blocks, int representatives, int topk,
                               void* stream);
int sparse_b200_indexer_summary(const void* q, const void* k, void* q_desc, void* k_desc, float* scores,
                                int32_t* block_idx, int batch, int hq, int hkv, int sq, int skv, int representatives,
                                int topk, void* stream);

/* Same block ids as sparse_b200_indexer_summary, bit for bit, computed with a
 * tensor-core pre-filter (tcgen05 MMA on the pooled descriptors) followed by exact
 * re-scoring of the surviving candidates and an exact fallback per list when the
 * pre-filter cannot be proven safe. No scores output. `aux` is a device workspace
 * of sparse_b200_indexer_summary_aux_bytes(B, Hkv) bytes (layout below). Shapes the
 * tensor-core path does not cover run the exact kernel. Replaces descriptor_dot +
 * reduce_topk (indexers/r1_r4/gpu_ops.py:19-49).
 * aux: 2*B*Hkv floats of key statistics, then three words written by every call: lists that
 * took the exact fallback (int), re-scored candidates whose tensor-core score differed from
 * the exact one by more than the error bound (int; such a list takes the fallback, so the ids
 * stay exact), largest observed difference as a fraction of the bound (float). */
int64_t sparse_b200_indexer_summary_aux_bytes(int batch, int hkv);
int sparse_b200_indexer_summary_fast(const void* q, const void* k, void* q_desc, void* k_desc, void* aux,
                                     int32_t* block_idx, int batch, int hq, int hkv, int sq, int skv,
                                     int representatives, int topk, void* stream);

/* Indexer -> attention on one stream with no host synchronisation: R1/R4 indexer (tensor-core
 * path) writes block_idx, the Q-centric kernel consumes it. The shape of indexed_attention()
 * (indexers/fp4/pipeline.py:49-65) for the summary indexers; capturable in a CUDA graph after
 * one eager call. Workspaces as in sparse_b200_indexer_summary_fast. */
int sparse_b200_indexed_attention_summary(const void* q, const void* k, const void* v, void* q_desc, void* k_desc,
                                          void* aux, int32_t* block_idx, void* out, float* lse, int batch, int hq,
                                          int hkv, int sq, int skv, int representatives, int topk, void* stream);

/* NVFP4 indexer. Index vectors: 64 bytes of e2m1 codes (low nibble first) + 8
 * e4m3 scales per 128 features (contract of prepare_fp4_inputs,
 * indexers/fp4/fp4.py:37-60). q_codes [B*Sq, Hidx, 64], q_scales [B*Sq, Hidx, 8],
 * k_codes [B*Skv/128, Hk, 128, 64], k_scales [B*Skv/128, Hk, 128, 8], Hk = 1 or Hidx.
 * nvfp4_quantize: x [B, heads_out*group, S, 128] bf16 -> codes and scales of the
 * mean over each `group` of heads; paged = 0 writes the query layout, 1 the key
 * page layout. (No counterpart in the reference, which feeds random bytes.)
 * fp4_scores: query_scores [Hidx, Skv/128, B*Sq] = max over the keys of a page
 * (what fp4_indexer_block_scores returns, indexers/fp4/fp4.py:122-134) and / or
 * tile_scores [B, Hidx, Sq/128, Skv/128] = max over the queries of a tile too.
 * tile_topk: query_scores -> block_idx [B, H, Sq/128, TopK]
 * (fp4_tile_topk_launch, indexers/fp4/tile_topk.cu:130-153, any TopK).
 * row_topk: tile_scores [rows, kv_tiles] -> block_idx [rows, TopK].
 * indexer_fp4 = fp4_scores(tile) + row_topk: fp4_indexer() of fp4.py:137-146
 * without materialising per-query scores. */
int sparse_b200_nvfp4_quantize(const void* x, void* packed, void* scales, int batch, int heads_out, int group,
                               int seq, int paged, void* stream);
int sparse_b200_fp4_scores(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                           float* query_scores, float* tile_scores, int batch, int hidx, int hk, int len_q, int len_kv,
                           void* stream);
/* Ragged batches over a paged key cache, optionally causal: the contract of
 * fp4_indexer_block_scores (indexers/fp4/vendor_minimax_msa/fp4_indexer_interface.py:745-811).
 * q_codes [total_q, Hq, 64], q_scales [total_q, Hq, 8]; k_codes [total_pages, Hk, 128, 64],
 * k_scales [total_pages, Hk, 128, 8]; cu_seqlens_q / cu_seqlens_k / cu_page_offsets [B + 1] and
 * kv_indices [sum of pages] int32 device arrays; qo_offset [B] int32 or NULL (causal only: key j
 * is visible to query i when j <= i + offset, offset = k_len - q_len unless given).
 * query_scores [Hq, ceil(max_seqlen_k / 128), total_q] fp32 is written completely: -inf where a
 * query sees no key of a page. Query head h reads key head h / (Hq / Hk). Same exact arithmetic
 * as sparse_b200_fp4_scores. */
int sparse_b200_fp4_scores_varlen(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                  const int32_t* cu_page_offsets, const int32_t* kv_indices, const int32_t* qo_offset,
                                  float* query_scores, int batch, int hq, int hk, int total_q, int total_pages,
                                  int max_seqlen_q, int max_seqlen_k, int causal, void* stream);
/* Same arguments and output, computed straight off the NVFP4 tensor cores (tcgen05 block-scaled MMAs on the
 * codes and scales as they are, query tile as the M operand, maximum over the keys of a page along a
 * tensor-memory lane): what the reference's scorer itself returns
 * (indexers/fp4/vendor_minimax_msa/src/sm100/fp4_indexer.py:201-1108, decode form :1110-1229). The eight scaled
 * group sums of a dot are added in the tensor core's own order, so finite scores are within the reference's gate
 * (rtol 1e-4, atol 1e-3, benchmarks/ch4_selectors/harness.py:33-42) of sparse_b200_fp4_scores_varlen, not bit-equal;
 * the -inf pattern is identical. Use the exact entry where block ids must be reproducible bit for bit. */
int sparse_b200_fp4_scores_varlen_fast(const void* q_codes, const void* q_scales, const void* k_codes,
                                       const void* k_scales, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                       const int32_t* cu_page_offsets, const int32_t* kv_indices,
                                       const int32_t* qo_offset, float* query_scores, int batch, int hq, int hk,
                                       int total_q, int total_pages, int max_seqlen_q, int max_seqlen_k, int causal,
                                       void* stream);
int sparse_b200_tile_topk(const float* query_scores, int32_t* block_idx, int batch, int heads, int len_q, int kv_tiles,
                          int topk, void* stream);
int sparse_b200_row_topk(const float* tile_scores, int32_t* block_idx, int64_t rows, int kv_tiles, int topk,
                         void* stream);
int sparse_b200_indexer_fp4(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                            float* tile_scores, int32_t* block_idx, int batch, int hidx, int hk, int len_q, int len_kv,
                            int topk, void* stream);

/* Same block ids as sparse_b200_indexer_fp4, bit for bit, with the scoring on the NVFP4
 * tensor cores: tcgen05 block-scaled MMAs (e2m1 codes, ue4m3 scale per 16 features) read
 * the codes and scales as they are, so every dot product comes within a known bound of
 * its exact value and nothing is dequantised. With many pages per top-k they pre-filter
 * the pages of every query tile, the candidates whose order the approximate scores do not
 * settle are re-scored with the exact group-ordered arithmetic, and a tile whose
 * pre-filter cannot be proven safe is scored exactly in full; with few pages they prune
 * every (query tile, page) pair to the few elements that can hold its exact maximum,
 * which are then evaluated exactly. `workspace` (256-byte aligned device memory of
 * sparse_b200_indexer_fp4_workspace_bytes(...) bytes) starts with five words that the
 * owner zeroes ONCE (no call clears them; they accumulate over calls): [0] CTAs of the
 * tensor-core kernels that ran (int), [1] tiles that took the exact path (int), [2]
 * unused, [3] scores whose tensor-core value and exact value differed by more than the
 * bound (int; each sends its tile or pair to the exact path, so ids stay exact),
 * [4] largest such difference seen, as a fraction of the bound (float); tile scores follow
 * at byte 256 when the pruning path ran.
 * Role of fp4_indexer() (indexers/fp4/fp4.py:137-146) with the scorer of
 * indexers/fp4/vendor_minimax_msa/src/sm100/fp4_indexer.py:201-1108. */
int64_t sparse_b200_indexer_fp4_workspace_bytes(int batch, int hidx, int hk, int len_q, int len_kv);
int sparse_b200_indexer_fp4_fast(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                                 void* workspace, int64_t workspace_bytes, int32_t* block_idx, int batch, int hidx,
                                 int hk, int len_q, int len_kv, int topk, void* stream);

/* NVFP4 indexer -> attention on one stream with no host synchronisation, the whole of
 * indexed_attention() (indexers/fp4/pipeline.py:49-65) as one call: [quantise ->] score
 * on the NVFP4 tensor cores -> top-k -> Q-centric attention. One index head per KV head:
 * q_codes [B*Sq, Hkv, 64], q_scales [B*Sq, Hkv, 8], k_codes [B*Skv/128, Hkv, 128, 64],
 * k_scales [B*Skv/128, Hkv, 128, 8]. quantize != 0: the four buffers are OUTPUTS, filled
 * from q (mean over the Hq/Hkv heads of a group) and k first, the preparation the reference
 * leaves outside its timing (indexers/fp4/fp4.py:37-119); quantize == 0: they are inputs
 * prepared earlier. workspace as in sparse_b200_indexer_fp4_fast(B, Hkv, Hkv, Sq, Skv).
 * block_idx [B, Hkv, Sq/128, TopK] is written and consumed. Nothing is allocated;
 * capturable in a CUDA graph after one eager call. */
int sparse_b200_indexed_attention_fp4(const void* q, const void* k, const void* v, void* q_codes, void* q_scales,
                                      void* k_codes, void* k_scales, void* workspace, int64_t workspace_bytes,
                                      int32_t* block_idx, void* out, float* lse, int batch, int hq, int hkv, int sq,
                                      int skv, int topk, int quantize, void* stream);

/* R1 / R4 summary indexer that allocates nothing and takes no workspace: same
 * inputs, outputs, arithmetic and results as sparse_b200_indexer_summary, with
 * the pooled descriptors kept in an 8 MiB array built into the library. It has
 * no counterpart in the reference. It is for callers that cannot allocate
 * device memory where they need block ids (under a memory pool that owns the
 * whole device, inside a serving loop with a fixed memory budget, behind a
 * plugin interface that passes only inputs and outputs). Limits: (B*Hq*Sq/128 + B*Hkv*Skv/128) * R <= 32768
 * descriptors, group size x R <= 16, Skv/128 <= 4096; anything larger returns
 * SPARSE_B200_ERR_INVALID. Every GPU that loads the library holds the 8 MiB
 * until exit. All calls on a device share the array: calls that overlap on the
 * GPU race, so keep them on one stream or order them yourself. The first call on
 * a device resolves the array's address; make it before any stream capture. */
int sparse_b200_indexer_summary_noalloc(const void* q, const void* k, float* scores, int32_t* block_idx, int batch,
                                        int hq, int hkv, int sq, int skv, int representatives, int topk,
                                        void* stream);

#ifdef __cplusplus
}
#endif
#endif
