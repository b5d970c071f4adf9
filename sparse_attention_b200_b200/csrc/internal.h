// Declarations shared by the translation units of libsparse_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#define SB_OK 0
#define SB_ERR_INVALID (-1)   // rejected argument (shape, alignment, null pointer ...)
#define SB_ERR_CUDA (-2)      // a CUDA runtime / driver call failed
#define SB_ERR_TIMEOUT (-3)   // a kernel gave up a bounded wait (see sparse_b200_device_status)

namespace sb {

// Per-device state created on first use (device current at that time).
struct DeviceCtx {
  int device = -1;
  int sm_count = 0;
  int* status = nullptr;      // device word written by kernels that abort a wait
  int qc_attr_bf16 = 0, qc_attr_f32 = 0;
  int misc_attr[8] = {0};
  int tc_attr = 0;
  int small_attr = 0;
};
DeviceCtx* device_ctx();

int set_error(int code, const char* message);   // stores a thread-local message, returns code

int encode_tiled(CUtensorMap* map, CUtensorMapDataType type, int rank, void* ptr, const cuuint64_t* dims,
                 const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* steps,
                 CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo);

struct QCentricArgs {
  const void *q, *k, *v;
  const int32_t* block_idx;
  const int32_t* block_count;
  void* out;
  float* lse;
  int batch, hq, hkv, sq, skv, topk, nseg, out_f32;
  void* tail_ws = nullptr;      // optional workspace for balancing the last round of items (q_centric.cu)
  long long tail_bytes = 0;
  // scatter launch: the flattened rows are cut into `owners` equal slices; slice 0 goes to (out, lse), slice j to
  // (owner_out[j], owner_lse[j]) - host arrays of device pointers, possibly in other GPUs' memory
  int owners = 1;
  void* const* owner_out = nullptr;
  float* const* owner_lse = nullptr;
};
int launch_q_centric(const QCentricArgs& a, cudaStream_t stream);

int launch_combine(const void* partial, int partial_is_f32, const float* lses, void* out, float* out_lse,
                   long long rows, int ranks, long long p_stride_rank, long long p_stride_row,
                   long long l_stride_rank, long long l_stride_row, cudaStream_t stream, int tm_h = 0, int tm_s = 0);
int launch_split_segments(const int32_t* ids, const int32_t* counts, int32_t* seg_ids, int32_t* seg_counts,
                          int* error, long long lists, int topk, int kv_blocks, int nseg, cudaStream_t stream);
int launch_pool(const void* x, void* desc, long long num_desc, int tokens_per_desc, cudaStream_t stream);
// small problems (indexer_summary_small.cu)
bool pool_small_eligible(long long num_desc);
int launch_pool_small(const void* x, void* desc, long long num_desc, int tokens_per_desc, cudaStream_t stream);
int launch_pool_small_pair(const void* x, void* desc, long long num_desc, const void* x2, void* desc2,
                           long long num_desc2, int tokens_per_desc, cudaStream_t stream);
// returns 1 when the problem is not small; fallback_counter (may be null) is reset to 0
int launch_summary_small(const void* qd, const void* kd, float* scores, int32_t* ids, int32_t* fallback_counter,
                         int batch, int hq, int hkv, int qt, int nt, int r, int topk, cudaStream_t stream);
// flagged_only: re-do only the lists whose first id is -1 (second pass after a pre-filter kernel)
int launch_summary_score_topk(const void* qd, const void* kd, float* scores, int32_t* ids, int batch, int hq, int hkv,
                              int qt, int nt, int r, int topk, cudaStream_t stream, int flagged_only = 0);
int launch_summary_select_tc(const void* qd, const void* kd, void* aux, int32_t* ids, int batch, int hq, int hkv,
                             int qt, int nt, int r, int topk, cudaStream_t stream);
int launch_fp4_indexer_tc(const void* qp, const void* qs, const void* kp, const void* ks, void* aux, int32_t* ids,
                          int batch, int hidx, int hk, int len_q, int len_kv, int topk, cudaStream_t stream);
int launch_token_metadata(const int32_t* selected, int32_t* counts, int32_t* cursors, int32_t* row_ptr,
                          int32_t* qids, int32_t* ranks, int32_t* task_ptr, int32_t* tasks, int32_t* error,
                          int groups, int sq, int topk, int kv_blocks, int group_size, cudaStream_t stream);
int launch_kv_token_main(const void* q, const void* k, const void* v, const int32_t* tasks, const int32_t* task_count,
                         const int32_t* qids, const int32_t* ranks, void* partial, float* lses, int batch, int hq,
                         int hkv, int sq, int skv, int topk, int partial_f32, cudaStream_t stream);
int launch_kv_token_pipe(const void* q, const void* k, const void* v, const int32_t* tasks, const int32_t* task_count,
                         const int32_t* qids, const int32_t* ranks, void* partial, float* lses, int batch, int hq,
                         int hkv, int sq, int skv, int topk, int q_token_major, cudaStream_t stream);
// peer_exchange.cu: exchange memory other processes of the machine can map, flag signalling, merge over peer loads
int peer_alloc(long long bytes, void** ptr, void* handle64);
int peer_open(const void* handle64, void** ptr);
int peer_close(void* ptr);
int peer_free(void* ptr);
int launch_peer_signal(int32_t* const* flags, int n, int value, cudaStream_t stream);
int launch_peer_wait(const int32_t* flags, int n, int value, int wait_ms, cudaStream_t stream);
int launch_combine_peer(const void* const* partials, const float* const* lses, const int32_t* ready, int value,
                        int wait_ms, void* out, float* out_lse, long long rows, int ranks, cudaStream_t stream);
int launch_quantize(const void* x, void* packed, void* scales, int batch, int heads_out, int group, int seq,
                    int paged, cudaStream_t stream);
int launch_fp4_scores_prune(const void* qp, const void* qs, const void* kp, const void* ks, void* aux, float* tile_scores,
                            int batch, int hidx, int hk, int len_q, int len_kv, cudaStream_t stream);
int launch_fp4_scores_varlen(const void* qp, const void* qs, const void* kp, const void* ks, const int32_t* cu_q,
                             const int32_t* cu_k, const int32_t* cu_pages, const int32_t* kv_indices,
                             const int32_t* qo_offset, float* out, int batch, int hq, int hk, int total_q,
                             int total_pages, int max_seqlen_q, int max_seqlen_k, int causal, cudaStream_t stream);
int launch_fp4_scores_varlen_nv(const void* qp, const void* qs, const void* kp, const void* ks, const int32_t* cu_q,
                                const int32_t* cu_k, const int32_t* cu_pages, const int32_t* kv_indices,
                                const int32_t* qo_offset, float* out, int batch, int hq, int hk, int total_q,
                                int total_pages, int max_seqlen_q, int max_seqlen_k, int causal, cudaStream_t stream);
int launch_fp4_scores(const void* qp, const void* qs, const void* kp, const void* ks, float* query_scores,
                      float* tile_scores, int batch, int hidx, int hk, int len_q, int len_kv, cudaStream_t stream);
int launch_tile_max_topk(const float* query_scores, int32_t* ids, int batch, int heads, int len_q, int tiles, int topk,
                         cudaStream_t stream);
int launch_row_topk(const float* tile_scores, int32_t* ids, long long rows, int tiles, int topk, cudaStream_t stream,
                    bool after_scorer = false);
int launch_bounded_wait_selftest(long long limit_cycles, int* observed, cudaStream_t stream);

}  // namespace sb
