// C-ABI of libsparse_b200.so: argument checks, per-device state, error text.
// No entry point throws, synchronises the device or allocates on the stream
// path (the only allocation is a 4-byte status word per device, on first use).
#include "internal.h"
#include "../../include/sparse_b200.h"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace sb {

static thread_local char g_error[512] = "";

int set_error(int code, const char* message) {
  snprintf(g_error, sizeof(g_error), "%s", message ? message : "");
  return code;
}

static const size_t STATUS_BYTES = sizeof(int);
static std::mutex g_mutex;
static DeviceCtx g_ctx[64];
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn g_encode = nullptr;

DeviceCtx* device_ctx() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error(SB_ERR_CUDA, "no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceCtx& c = g_ctx[dev];
  if (c.device == dev) return &c;
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
      set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
      return nullptr;
    }
    g_encode = reinterpret_cast<EncodeFn>(fn);
  }
  if (cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaMalloc(&c.status, STATUS_BYTES) != cudaSuccess ||
      cudaMemset(c.status, 0, STATUS_BYTES) != cudaSuccess) {
    set_error(SB_ERR_CUDA, "device state initialisation failed");
    return nullptr;
  }
  c.device = dev;
  return &c;
}

int encode_tiled(CUtensorMap* map, CUtensorMapDataType type, int rank, void* ptr, const cuuint64_t* dims,
                 const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* steps,
                 CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo) {
  if (!g_encode) return 1;
  CUresult r = g_encode(map, type, rank, ptr, dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace sb

using namespace sb;

#define REQUIRE(cond, msg) \
  do {                     \
    if (!(cond)) return set_error(SB_ERR_INVALID, msg); \
  } while (0)

extern "C" {

const char* sparse_b200_last_error(void) { return g_error; }

int sparse_b200_device_status(int reset) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  int value = 0;
  if (cudaMemcpy(&value, ctx->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return set_error(SB_ERR_CUDA, "status read failed");
  if (reset && value != 0) cudaMemset(ctx->status, 0, sizeof(int));
  return value;
}

int sparse_b200_check_status(void) {
  const int value = sparse_b200_device_status(1);
  if (value < 0) return value;
  if (value == 0) return SB_OK;
  char msg[160];
  snprintf(msg, sizeof(msg), "a kernel abandoned a bounded wait (code 0x%x); its outputs are incomplete", value);
  return set_error(SB_ERR_TIMEOUT, msg);
}

int sparse_b200_selftest_bounded_wait(int64_t limit_cycles, int32_t* observed, void* stream) {
  REQUIRE(limit_cycles > 0 && limit_cycles <= 100000000LL, "limit must be in (0, 1e8] cycles");
  return launch_bounded_wait_selftest(limit_cycles, observed, static_cast<cudaStream_t>(stream));
}

static int check_attention(const void* q, const void* k, const void* v, const int32_t* block_idx,
                           const void* out, int batch, int hq, int hkv, int sq, int skv, int topk, int nseg) {
  REQUIRE(q && k && v && block_idx && out, "q, k, v, block_idx and out must be non-null device pointers");
  REQUIRE(batch > 0 && hkv > 0, "batch and KV heads must be positive");
  REQUIRE(hq >= hkv && hq % hkv == 0, "Hq must be a multiple of and at least Hkv");
  REQUIRE(sq >= 128 && sq % 128 == 0, "Sq must be a positive multiple of 128");
  REQUIRE(skv >= 128 && skv % 128 == 0, "Skv must be a positive multiple of 128");
  REQUIRE(topk > 0, "selected_count must be positive");
  REQUIRE(topk <= skv / 128, "selected_count cannot exceed the number of KV tiles");
  REQUIRE(nseg >= 1, "segment count must be positive");
  REQUIRE(static_cast<long long>(nseg) * batch * hq * sq < (1LL << 31) &&
              static_cast<long long>(batch) * hkv * skv < (1LL << 31),
          "flattened Q / KV row counts must fit int32 (TMA row coordinates)");
  REQUIRE(static_cast<long long>(nseg) * batch * hkv * (sq / 128) * topk < (1LL << 40), "block_idx too large");
  REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), "q, k, v, out must be 16-byte aligned");
  REQUIRE(out != q && out != k && out != v && out != static_cast<const void*>(block_idx),
          "output must not alias inputs");
  return SB_OK;
}

int sparse_b200_q_centric(const void* q, const void* k, const void* v, const int32_t* block_idx,
                          const int32_t* block_count, void* out, float* lse, int batch, int hq, int hkv,
                          int sq, int skv, int topk, void* stream) {
  int rc = check_attention(q, k, v, block_idx, out, batch, hq, hkv, sq, skv, topk, 1);
  if (rc) return rc;
  QCentricArgs a{q, k, v, block_idx, block_count, out, lse, batch, hq, hkv, sq, skv, topk, 1, 0};
  return launch_q_centric(a, static_cast<cudaStream_t>(stream));
}

int64_t sparse_b200_q_centric_workspace_bytes(void) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  // at most one piece per CTA in the balanced round: two streams of 128 rows, bf16 O + fp32 LSE
  return static_cast<int64_t>(ctx->sm_count) * 2 * 128 * (128 * 2 + 4) + 512;
}

int sparse_b200_q_centric_ws(const void* q, const void* k, const void* v, const int32_t* block_idx,
                             const int32_t* block_count, void* out, float* lse, void* workspace,
                             int64_t workspace_bytes, int batch, int hq, int hkv, int sq, int skv, int topk,
                             void* stream) {
  int rc = check_attention(q, k, v, block_idx, out, batch, hq, hkv, sq, skv, topk, 1);
  if (rc) return rc;
  REQUIRE(workspace == nullptr || aligned16(workspace), "misaligned workspace");
  QCentricArgs a{q, k, v, block_idx, block_count, out, lse, batch, hq, hkv, sq, skv, topk, 1, 0};
  a.tail_ws = workspace;
  a.tail_bytes = workspace ? workspace_bytes : 0;
  return launch_q_centric(a, static_cast<cudaStream_t>(stream));
}

int sparse_b200_q_centric_scatter(const void* q, const void* k, const void* v, const int32_t* block_idx,
                                  const int32_t* block_count, void* const* outs, float* const* lses, int owners,
                                  int batch, int hq, int hkv, int sq, int skv, int topk, void* stream) {
  REQUIRE(outs && lses && owners >= 1 && owners <= 4, "1 to 4 destinations, as host arrays of device pointers");
  REQUIRE(outs[0] && lses[0], "null destination");
  int rc = check_attention(q, k, v, block_idx, outs[0], batch, hq, hkv, sq, skv, topk, 1);
  if (rc) return rc;
  QCentricArgs a{q, k, v, block_idx, block_count, outs[0], lses[0], batch, hq, hkv, sq, skv, topk, 1, 0};
  a.owners = owners;
  a.owner_out = outs;
  a.owner_lse = lses;
  return launch_q_centric(a, static_cast<cudaStream_t>(stream));
}

int sparse_b200_q_centric_partial(const void* q, const void* k, const void* v, const int32_t* seg_block_idx,
                                  const int32_t* seg_block_count, void* partial_out, float* partial_lse,
                                  int nseg, int partial_is_f32, int batch, int hq, int hkv, int sq, int skv,
                                  int topk, void* stream) {
  int rc = check_attention(q, k, v, seg_block_idx, partial_out, batch, hq, hkv, sq, skv, topk, nseg);
  if (rc) return rc;
  REQUIRE(seg_block_count && partial_lse, "segment counts and partial LSE are required");
  QCentricArgs a{q, k, v, seg_block_idx, seg_block_count, partial_out, partial_lse,
                 batch, hq, hkv, sq, skv, topk, nseg, partial_is_f32 ? 1 : 0};
  return launch_q_centric(a, static_cast<cudaStream_t>(stream));
}

int sparse_b200_combine(const void* partial, int partial_is_f32, const float* partial_lse, void* out, float* out_lse,
                        int64_t rows, int ranks, int rank_major, void* stream) {
  REQUIRE(partial && partial_lse && out, "partial, partial_lse and out must be non-null device pointers");
  REQUIRE(rows > 0 && ranks > 0, "rows and ranks must be positive");
  REQUIRE(aligned16(partial) && aligned16(out), "partial and out must be 16-byte aligned");
  const long long psr = rank_major ? rows * 128 : 128, psw = rank_major ? 128 : static_cast<long long>(ranks) * 128;
  const long long lsr = rank_major ? rows : 1, lsw = rank_major ? 1 : ranks;
  return launch_combine(partial, partial_is_f32, partial_lse, out, out_lse, rows, ranks, psr, psw, lsr, lsw,
                        static_cast<cudaStream_t>(stream));
}

int sparse_b200_split_kv_segments(const int32_t* block_idx, const int32_t* block_count, int32_t* seg_block_idx,
                                  int32_t* seg_block_count, int32_t* error_word, int batch, int hkv, int q_blocks,
                                  int topk, int kv_blocks, int nseg, void* stream) {
  REQUIRE(block_idx && seg_block_idx && seg_block_count && error_word, "null pointer");
  REQUIRE(batch > 0 && hkv > 0 && q_blocks > 0 && topk > 0 && kv_blocks > 0, "sizes must be positive");
  REQUIRE(nseg >= 1 && nseg <= kv_blocks, "segment count must be in [1, kv_blocks]");
  return launch_split_segments(block_idx, block_count, seg_block_idx, seg_block_count, error_word,
                               static_cast<long long>(batch) * hkv * q_blocks, topk, kv_blocks, nseg,
                               static_cast<cudaStream_t>(stream));
}

static size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

int64_t sparse_b200_kv_centric_workspace_bytes(int batch, int hq, int hkv, int sq, int topk, int nseg,
                                               int partial_is_f32) {
  if (batch <= 0 || hq <= 0 || hkv <= 0 || sq < 128 || topk <= 0 || nseg <= 0) return SB_ERR_INVALID;
  const size_t lists = static_cast<size_t>(batch) * hkv * (sq / 128);
  const size_t rows = static_cast<size_t>(batch) * hq * sq;
  size_t total = 256;                                                   // error word
  total += align256(lists * nseg * topk * 4) + align256(lists * nseg * 4);   // segment lists and counts
  total += align256(rows * nseg * 128 * (partial_is_f32 ? 4 : 2));      // partial O
  total += align256(rows * nseg * 4);                                   // partial LSE
  return static_cast<int64_t>(total);
}

int sparse_b200_kv_centric(const void* q, const void* k, const void* v, const int32_t* block_idx,
                           const int32_t* block_count, void* out, float* lse, void* workspace,
                           int64_t workspace_bytes, int nseg, int partial_is_f32, int batch, int hq, int hkv, int sq,
                           int skv, int topk, void* stream) {
  int rc = check_attention(q, k, v, block_idx, out, batch, hq, hkv, sq, skv, topk, nseg);
  if (rc) return rc;
  REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, "workspace must be 256-byte aligned");
  REQUIRE(nseg <= skv / 128, "more segments than KV blocks");
  REQUIRE(workspace_bytes >= sparse_b200_kv_centric_workspace_bytes(batch, hq, hkv, sq, topk, nseg, partial_is_f32),
          "workspace too small (see sparse_b200_kv_centric_workspace_bytes)");
  const size_t lists = static_cast<size_t>(batch) * hkv * (sq / 128);
  const size_t rows = static_cast<size_t>(batch) * hq * sq;
  unsigned char* w = static_cast<unsigned char*>(workspace);
  int32_t* err = reinterpret_cast<int32_t*>(w);
  w += 256;
  int32_t* seg_ids = reinterpret_cast<int32_t*>(w);
  w += align256(lists * nseg * topk * 4);
  int32_t* seg_counts = reinterpret_cast<int32_t*>(w);
  w += align256(lists * nseg * 4);
  void* partial = w;
  w += align256(rows * nseg * 128 * (partial_is_f32 ? 4 : 2));
  float* plse = reinterpret_cast<float*>(w);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(err, 0, 4, st) != cudaSuccess) return set_error(SB_ERR_CUDA, "memset failed");
  rc = launch_split_segments(block_idx, block_count, seg_ids, seg_counts, err, static_cast<long long>(lists), topk,
                             skv / 128, nseg, st);
  if (rc) return rc;
  QCentricArgs a{q, k, v, seg_ids, seg_counts, partial, plse, batch, hq, hkv, sq, skv, topk, nseg,
                 partial_is_f32 ? 1 : 0};
  rc = launch_q_centric(a, st);
  if (rc) return rc;
  return launch_combine(partial, partial_is_f32, plse, out, lse, static_cast<long long>(rows), nseg,
                        static_cast<long long>(rows) * 128, 128, static_cast<long long>(rows), 1, st);
}

int sparse_b200_pool_blocks(const void* x, void* desc, int batch, int heads, int seq, int representatives,
                            void* stream) {
  REQUIRE(x && desc, "null pointer");
  REQUIRE(batch > 0 && heads > 0 && seq >= 128 && seq % 128 == 0, "sequence must be a positive multiple of 128");
  REQUIRE(representatives == 1 || representatives == 2 || representatives == 4, "representatives must be 1, 2 or 4");
  REQUIRE(aligned16(x) && aligned16(desc), "x and desc must be 16-byte aligned");
  const long long num = static_cast<long long>(batch) * heads * (seq / 128) * representatives;
  if (pool_small_eligible(num))
    return launch_pool_small(x, desc, num, 128 / representatives, static_cast<cudaStream_t>(stream));
  return launch_pool(x, desc, num, 128 / representatives, static_cast<cudaStream_t>(stream));
}

// Query and key descriptors: one launch when both tensors are small, else one launch each.
static int pool_both(const void* q, void* q_desc, const void* k, void* k_desc, int batch, int hq, int hkv, int sq,
                     int skv, int r, void* stream) {
  const long long nq = static_cast<long long>(batch) * hq * (sq / 128) * r;
  const long long nk = static_cast<long long>(batch) * hkv * (skv / 128) * r;
  if (pool_small_eligible(nq + nk)) {
    if (!(aligned16(q) && aligned16(k) && aligned16(q_desc) && aligned16(k_desc)))
      return set_error(SB_ERR_INVALID, "x and desc must be 16-byte aligned");
    return launch_pool_small_pair(q, q_desc, nq, k, k_desc, nk, 128 / r, static_cast<cudaStream_t>(stream));
  }
  int rc = sparse_b200_pool_blocks(q, q_desc, batch, hq, sq, r, stream);
  if (rc) return rc;
  return sparse_b200_pool_blocks(k, k_desc, batch, hkv, skv, r, stream);
}

static int check_summary(int batch, int hq, int hkv, int qt, int nt, int r, int topk) {
  REQUIRE(batch > 0 && hkv > 0 && hq >= hkv && hq % hkv == 0, "Hq must be a positive multiple of Hkv");
  REQUIRE(qt > 0 && nt > 0, "block counts must be positive");
  REQUIRE(r == 1 || r == 2 || r == 4, "representatives must be 1, 2 or 4");
  REQUIRE((hq / hkv) * r <= 64, "group size x representatives must not exceed 64");
  REQUIRE(topk > 0 && topk <= nt, "top-k must be in [1, number of KV blocks]");
  return SB_OK;
}

int sparse_b200_summary_select(const void* q_desc, const void* k_desc, float* scores, int32_t* block_idx, int batch,
                               int hq, int hkv, int q_blocks, int kv_blocks, int representatives, int topk,
                               void* stream) {
  REQUIRE(q_desc && k_desc && block_idx, "null pointer");
  int rc = check_summary(batch, hq, hkv, q_blocks, kv_blocks, representatives, topk);
  if (rc) return rc;
  return launch_summary_score_topk(q_desc, k_desc, scores, block_idx, batch, hq, hkv, q_blocks, kv_blocks,
                                   representatives, topk, static_cast<cudaStream_t>(stream));
}

int sparse_b200_indexer_summary(const void* q, const void* k, void* q_desc, void* k_desc, float* scores,
                                int32_t* block_idx, int batch, int hq, int hkv, int sq, int skv, int representatives,
                                int topk, void* stream) {
  REQUIRE(q && k && q_desc && k_desc && block_idx, "null pointer");
  REQUIRE(sq >= 128 && sq % 128 == 0 && skv >= 128 && skv % 128 == 0, "Sq and Skv must be positive multiples of 128");
  int rc = check_summary(batch, hq, hkv, sq / 128, skv / 128, representatives, topk);
  if (rc) return rc;
  rc = pool_both(q, q_desc, k, k_desc, batch, hq, hkv, sq, skv, representatives, stream);
  if (rc) return rc;
  rc = launch_summary_small(q_desc, k_desc, scores, block_idx, nullptr, batch, hq, hkv, sq / 128, skv / 128,
                            representatives, topk, static_cast<cudaStream_t>(stream));
  if (rc != 1) return rc;            // small problem: cluster kernel, same ids and scores
  return launch_summary_score_topk(q_desc, k_desc, scores, block_idx, batch, hq, hkv, sq / 128, skv / 128,
                                   representatives, topk, static_cast<cudaStream_t>(stream));
}

int64_t sparse_b200_indexer_summary_aux_bytes(int batch, int hkv) {
  if (batch <= 0 || hkv <= 0) return SB_ERR_INVALID;
  return (2 * static_cast<int64_t>(batch) * hkv + 3) * 4;
}

int sparse_b200_indexer_summary_fast(const void* q, const void* k, void* q_desc, void* k_desc, void* aux,
                                     int32_t* block_idx, int batch, int hq, int hkv, int sq, int skv,
                                     int representatives, int topk, void* stream) {
  REQUIRE(q && k && q_desc && k_desc && aux && block_idx, "null pointer");
  REQUIRE(sq >= 128 && sq % 128 == 0 && skv >= 128 && skv % 128 == 0, "Sq and Skv must be positive multiples of 128");
  int rc = check_summary(batch, hq, hkv, sq / 128, skv / 128, representatives, topk);
  if (rc) return rc;
  REQUIRE((reinterpret_cast<uintptr_t>(aux) & 3u) == 0 && aligned16(q_desc) && aligned16(k_desc), "misaligned workspace");
  rc = pool_both(q, q_desc, k, k_desc, batch, hq, hkv, sq, skv, representatives, stream);
  if (rc) return rc;
  // small problems: the exact cluster kernel fills the GPU better than the tensor-core pre-filter
  rc = launch_summary_small(q_desc, k_desc, nullptr, block_idx,
                            static_cast<int32_t*>(aux) + 2 * static_cast<long long>(batch) * hkv, batch, hq, hkv,
                            sq / 128, skv / 128, representatives, topk, static_cast<cudaStream_t>(stream));
  if (rc != 1) return rc;
  rc = launch_summary_select_tc(q_desc, k_desc, aux, block_idx, batch, hq, hkv, sq / 128, skv / 128, representatives,
                                topk, static_cast<cudaStream_t>(stream));
  if (rc == 1)      // not eligible for the tensor-core path: exact kernel, same ids
    rc = launch_summary_score_topk(q_desc, k_desc, nullptr, block_idx, batch, hq, hkv, sq / 128, skv / 128,
                                   representatives, topk, static_cast<cudaStream_t>(stream));
  return rc;
}

int sparse_b200_indexed_attention_summary(const void* q, const void* k, const void* v, void* q_desc, void* k_desc,
                                          void* aux, int32_t* block_idx, void* out, float* lse, int batch, int hq,
                                          int hkv, int sq, int skv, int representatives, int topk, void* stream) {
  int rc = sparse_b200_indexer_summary_fast(q, k, q_desc, k_desc, aux, block_idx, batch, hq, hkv, sq, skv,
                                            representatives, topk, stream);
  if (rc) return rc;
  // same stream: the ids written by the indexer are ready for the attention kernel
  return sparse_b200_q_centric(q, k, v, block_idx, nullptr, out, lse, batch, hq, hkv, sq, skv, topk, stream);
}

int sparse_b200_nvfp4_quantize(const void* x, void* packed, void* scales, int batch, int heads_out, int group,
                               int seq, int paged, void* stream) {
  REQUIRE(x && packed && scales, "null pointer");
  REQUIRE(batch > 0 && heads_out > 0 && group > 0 && seq > 0, "sizes must be positive");
  REQUIRE(!paged || seq % 128 == 0, "paged output needs a sequence that is a multiple of 128");
  REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(packed) & 7u) == 0, "x must be 16-byte, packed 8-byte aligned");
  return launch_quantize(x, packed, scales, batch, heads_out, group, seq, paged, static_cast<cudaStream_t>(stream));
}

static int check_fp4(const void* qp, const void* qs, const void* kp, const void* ks, int batch, int hidx, int hk,
                     int len_q, int len_kv) {
  REQUIRE(qp && qs && kp && ks, "null pointer");
  REQUIRE(batch > 0 && len_q > 0 && len_q % 128 == 0, "B must be positive and Sq a positive multiple of 128");
  REQUIRE(len_kv >= 128 && len_kv % 128 == 0, "Skv must be a positive multiple of 128");
  REQUIRE(hidx > 0 && (hk == 1 || hk == hidx), "key index heads must be 1 or equal to the query index heads");
  REQUIRE((reinterpret_cast<uintptr_t>(qp) & 3u) == 0 && (reinterpret_cast<uintptr_t>(kp) & 3u) == 0,
          "packed codes must be 4-byte aligned");
  return SB_OK;
}

int sparse_b200_fp4_scores(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                           float* query_scores, float* tile_scores, int batch, int hidx, int hk, int len_q, int len_kv,
                           void* stream) {
  int rc = check_fp4(q_codes, q_scales, k_codes, k_scales, batch, hidx, hk, len_q, len_kv);
  if (rc) return rc;
  REQUIRE(query_scores || tile_scores, "at least one score output is required");
  return launch_fp4_scores(q_codes, q_scales, k_codes, k_scales, query_scores, tile_scores, batch, hidx, hk, len_q,
                           len_kv, static_cast<cudaStream_t>(stream));
}

int sparse_b200_fp4_scores_varlen(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                  const int32_t* cu_page_offsets, const int32_t* kv_indices, const int32_t* qo_offset,
                                  float* query_scores, int batch, int hq, int hk, int total_q, int total_pages,
                                  int max_seqlen_q, int max_seqlen_k, int causal, void* stream) {
  REQUIRE(q_codes && q_scales && k_codes && k_scales && cu_seqlens_q && cu_seqlens_k && cu_page_offsets && kv_indices &&
              query_scores,
          "null pointer");
  REQUIRE(batch > 0 && total_q > 0 && total_pages > 0 && max_seqlen_q > 0 && max_seqlen_k > 0,
          "sizes must be positive");
  REQUIRE(hq > 0 && hk > 0 && hq % hk == 0, "query heads must be a positive multiple of key heads");
  REQUIRE(causal || !qo_offset, "qo_offset is only valid with causal masking");
  REQUIRE((reinterpret_cast<uintptr_t>(q_codes) & 3u) == 0 && (reinterpret_cast<uintptr_t>(k_codes) & 3u) == 0,
          "packed codes must be 4-byte aligned");
  return launch_fp4_scores_varlen(q_codes, q_scales, k_codes, k_scales, cu_seqlens_q, cu_seqlens_k, cu_page_offsets,
                                  kv_indices, qo_offset, query_scores, batch, hq, hk, total_q, total_pages,
                                  max_seqlen_q, max_seqlen_k, causal, static_cast<cudaStream_t>(stream));
}

int sparse_b200_fp4_scores_varlen_fast(const void* q_codes, const void* q_scales, const void* k_codes,
                                       const void* k_scales, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                       const int32_t* cu_page_offsets, const int32_t* kv_indices,
                                       const int32_t* qo_offset, float* query_scores, int batch, int hq, int hk,
                                       int total_q, int total_pages, int max_seqlen_q, int max_seqlen_k, int causal,
                                       void* stream) {
  REQUIRE(q_codes && q_scales && k_codes && k_scales && cu_seqlens_q && cu_seqlens_k && cu_page_offsets && kv_indices &&
              query_scores,
          "null pointer");
  REQUIRE(batch > 0 && total_q > 0 && total_pages > 0 && max_seqlen_q > 0 && max_seqlen_k > 0,
          "sizes must be positive");
  REQUIRE(hq > 0 && hk > 0 && hq % hk == 0, "query heads must be a positive multiple of key heads");
  REQUIRE(causal || !qo_offset, "qo_offset is only valid with causal masking");
  REQUIRE((reinterpret_cast<uintptr_t>(q_codes) & 3u) == 0 && (reinterpret_cast<uintptr_t>(k_codes) & 3u) == 0,
          "packed codes must be 4-byte aligned");
  int rc = launch_fp4_scores_varlen_nv(q_codes, q_scales, k_codes, k_scales, cu_seqlens_q, cu_seqlens_k, cu_page_offsets,
                                       kv_indices, qo_offset, query_scores, batch, hq, hk, total_q, total_pages,
                                       max_seqlen_q, max_seqlen_k, causal, static_cast<cudaStream_t>(stream));
  if (rc == 1)   // operands not aligned for the TMA path: exact scorer, same contract
    rc = launch_fp4_scores_varlen(q_codes, q_scales, k_codes, k_scales, cu_seqlens_q, cu_seqlens_k, cu_page_offsets,
                                  kv_indices, qo_offset, query_scores, batch, hq, hk, total_q, total_pages, max_seqlen_q,
                                  max_seqlen_k, causal, static_cast<cudaStream_t>(stream));
  return rc;
}

int sparse_b200_tile_topk(const float* query_scores, int32_t* block_idx, int batch, int heads, int len_q, int kv_tiles,
                          int topk, void* stream) {
  REQUIRE(query_scores && block_idx, "null pointer");
  REQUIRE(batch > 0 && heads > 0 && len_q > 0 && len_q % 128 == 0, "len_q must be a positive multiple of 128");
  REQUIRE(kv_tiles > 0 && topk > 0 && topk <= kv_tiles, "top-k must be in [1, kv_tiles]");
  REQUIRE(aligned16(query_scores), "scores must be 16-byte aligned");
  return launch_tile_max_topk(query_scores, block_idx, batch, heads, len_q, kv_tiles, topk,
                              static_cast<cudaStream_t>(stream));
}

int sparse_b200_row_topk(const float* tile_scores, int32_t* block_idx, int64_t rows, int kv_tiles, int topk,
                         void* stream) {
  REQUIRE(tile_scores && block_idx, "null pointer");
  REQUIRE(rows > 0 && kv_tiles > 0 && topk > 0 && topk <= kv_tiles, "top-k must be in [1, kv_tiles]");
  return launch_row_topk(tile_scores, block_idx, rows, kv_tiles, topk, static_cast<cudaStream_t>(stream));
}

int sparse_b200_indexer_fp4(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                            float* tile_scores, int32_t* block_idx, int batch, int hidx, int hk, int len_q, int len_kv,
                            int topk, void* stream) {
  int rc = check_fp4(q_codes, q_scales, k_codes, k_scales, batch, hidx, hk, len_q, len_kv);
  if (rc) return rc;
  REQUIRE(tile_scores && block_idx, "tile score workspace and block_idx are required");
  REQUIRE(topk > 0 && topk <= len_kv / 128, "top-k must be in [1, kv_tiles]");
  rc = launch_fp4_scores(q_codes, q_scales, k_codes, k_scales, nullptr, tile_scores, batch, hidx, hk, len_q, len_kv,
                         static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return launch_row_topk(tile_scores, block_idx, static_cast<long long>(batch) * hidx * (len_q / 128), len_kv / 128,
                         topk, static_cast<cudaStream_t>(stream));
}

int64_t sparse_b200_kv_token_max_tasks(int batch, int hkv, int sq, int topk, int kv_blocks, int group_size) {
  if (batch <= 0 || hkv <= 0 || sq <= 0 || topk <= 0 || kv_blocks <= 0 || group_size <= 0 || group_size > 128)
    return SB_ERR_INVALID;
  const int64_t edges = static_cast<int64_t>(batch) * hkv * sq * topk;
  const int64_t rows = static_cast<int64_t>(batch) * hkv * kv_blocks;
  const int64_t cap = 128 / group_size;
  const int64_t bound = (edges + cap - 1) / cap + rows;
  return bound < edges ? bound : edges;
}

int sparse_b200_kv_token_metadata(const int32_t* selected, int32_t* counts, int32_t* cursors, int32_t* row_ptr,
                                  int32_t* query_ids, int32_t* ranks, int32_t* task_ptr, int32_t* tasks,
                                  int32_t* error_word, int batch, int hkv, int sq, int topk, int kv_blocks,
                                  int group_size, void* stream) {
  REQUIRE(selected && counts && cursors && row_ptr && query_ids && ranks && task_ptr && tasks && error_word,
          "null pointer");
  REQUIRE(batch > 0 && hkv > 0 && sq > 0 && topk > 0 && kv_blocks > 0, "sizes must be positive");
  REQUIRE(group_size == 1 || group_size == 2 || group_size == 4 || group_size == 8 || group_size == 16,
          "supported ratios Hq/Hkv are 1, 2, 4, 8, and 16");
  REQUIRE(static_cast<long long>(batch) * hkv * sq * topk < (1LL << 31) &&
              static_cast<long long>(batch) * hkv * kv_blocks < (1LL << 31) - 1,
          "metadata is limited to signed int32 offsets");
  REQUIRE((reinterpret_cast<uintptr_t>(tasks) & 15u) == 0, "tasks must be 16-byte aligned");
  return launch_token_metadata(selected, counts, cursors, row_ptr, query_ids, ranks, task_ptr, tasks, error_word,
                               batch * hkv, sq, topk, kv_blocks, group_size, static_cast<cudaStream_t>(stream));
}

int sparse_b200_kv_token_main(const void* q, const void* k, const void* v, const int32_t* tasks,
                              const int32_t* task_ptr, const int32_t* query_ids, const int32_t* ranks, void* partial,
                              float* partial_lse, int batch, int hq, int hkv, int sq, int skv, int topk,
                              void* stream) {
  REQUIRE(q && k && v && tasks && task_ptr && query_ids && ranks && partial && partial_lse, "null pointer");
  REQUIRE(batch > 0 && hkv > 0 && hq >= hkv && hq % hkv == 0, "Hq must be a positive multiple of Hkv");
  const int g = hq / hkv;
  REQUIRE(g == 1 || g == 2 || g == 4 || g == 8 || g == 16, "supported ratios Hq/Hkv are 1, 2, 4, 8, and 16");
  REQUIRE(sq > 0 && skv >= 128 && skv % 128 == 0 && topk > 0 && topk <= skv / 128,
          "Skv must be a positive multiple of 128 and TopK at most the number of KV blocks");
  REQUIRE(static_cast<long long>(batch) * hkv * skv < (1LL << 31), "flattened KV rows must fit int32");
  REQUIRE(static_cast<long long>(batch) * hkv * sq * topk < (1LL << 31), "B*Hkv*Sq*TopK must fit int32 (edge offsets)");
  REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(partial) && aligned16(tasks), "misaligned pointer");
  const long long rows = static_cast<long long>(batch) * hkv * (skv / 128);
  return launch_kv_token_main(q, k, v, tasks, task_ptr + rows, query_ids, ranks, partial, partial_lse, batch, hq, hkv,
                              sq, skv, topk, 0, static_cast<cudaStream_t>(stream));
}

static int kv_token_main_token_major(const void* q_token_major, const void* k, const void* v, const int32_t* tasks,
                                     const int32_t* task_ptr, const int32_t* query_ids, const int32_t* ranks,
                                     void* partial, float* partial_lse, int batch, int hq, int hkv, int sq, int skv,
                                     int topk, int layout, void* stream) {
  REQUIRE(q_token_major && k && v && tasks && task_ptr && query_ids && ranks && partial && partial_lse, "null pointer");
  REQUIRE(batch > 0 && hkv > 0 && hq >= hkv && hq % hkv == 0, "Hq must be a positive multiple of Hkv");
  const int g = hq / hkv;
  REQUIRE(g == 8 || g == 16, "the token-major layout is supported for Hq/Hkv of 8 and 16");
  REQUIRE(sq > 0 && skv >= 128 && skv % 128 == 0 && topk > 0 && topk <= skv / 128,
          "Skv must be a positive multiple of 128 and TopK at most the number of KV blocks");
  REQUIRE(static_cast<long long>(batch) * hkv * skv < (1LL << 31) && static_cast<long long>(batch) * sq < (1LL << 31),
          "flattened KV rows and tokens must fit int32");
  REQUIRE(static_cast<long long>(batch) * hkv * sq * topk < (1LL << 31), "B*Hkv*Sq*TopK must fit int32 (edge offsets)");
  REQUIRE(aligned16(q_token_major) && aligned16(k) && aligned16(v) && aligned16(partial) && aligned16(tasks),
          "misaligned pointer");
  const long long rows = static_cast<long long>(batch) * hkv * (skv / 128);
  return launch_kv_token_pipe(q_token_major, k, v, tasks, task_ptr + rows, query_ids, ranks, partial, partial_lse, batch,
                              hq, hkv, sq, skv, topk, layout, static_cast<cudaStream_t>(stream));
}

int sparse_b200_kv_token_main_tm(const void* q_token_major, const void* k, const void* v, const int32_t* tasks,
                                 const int32_t* task_ptr, const int32_t* query_ids, const int32_t* ranks,
                                 void* partial, float* partial_lse, int batch, int hq, int hkv, int sq, int skv,
                                 int topk, void* stream) {
  return kv_token_main_token_major(q_token_major, k, v, tasks, task_ptr, query_ids, ranks, partial, partial_lse, batch,
                                   hq, hkv, sq, skv, topk, 1, stream);
}

int sparse_b200_kv_token_main_tm_partial_tm(const void* q_token_major, const void* k, const void* v,
                                            const int32_t* tasks, const int32_t* task_ptr, const int32_t* query_ids,
                                            const int32_t* ranks, void* partial_token_major, float* partial_lse,
                                            int batch, int hq, int hkv, int sq, int skv, int topk, void* stream) {
  return kv_token_main_token_major(q_token_major, k, v, tasks, task_ptr, query_ids, ranks, partial_token_major,
                                   partial_lse, batch, hq, hkv, sq, skv, topk, 3, stream);
}

int sparse_b200_kv_token_main_layout(const void* q, const void* k, const void* v, const int32_t* tasks,
                                     const int32_t* task_ptr, const int32_t* query_ids, const int32_t* ranks,
                                     void* partial, float* partial_lse, int batch, int hq, int hkv, int sq, int skv,
                                     int topk, int layout, void* stream) {
  REQUIRE(layout >= 0 && layout < 8, "layout is a mask of bits 0 (q token-major), 1 (partials token-major), 2 (fp32)");
  REQUIRE((layout & 3) != 2, "token-major partials go with token-major q");
  if (layout & 3)
    return kv_token_main_token_major(q, k, v, tasks, task_ptr, query_ids, ranks, partial, partial_lse, batch, hq, hkv,
                                     sq, skv, topk, layout, stream);
  if (layout == 0)
    return sparse_b200_kv_token_main(q, k, v, tasks, task_ptr, query_ids, ranks, partial, partial_lse, batch, hq, hkv,
                                     sq, skv, topk, stream);
  // head-major fp32 partials: the checks of sparse_b200_kv_token_main, then the fp32 form of the same kernels
  REQUIRE(q && k && v && tasks && task_ptr && query_ids && ranks && partial && partial_lse, "null pointer");
  REQUIRE(batch > 0 && hkv > 0 && hq >= hkv && hq % hkv == 0, "Hq must be a positive multiple of Hkv");
  const int g = hq / hkv;
  REQUIRE(g == 1 || g == 2 || g == 4 || g == 8 || g == 16, "supported ratios Hq/Hkv are 1, 2, 4, 8, and 16");
  REQUIRE(sq > 0 && skv >= 128 && skv % 128 == 0 && topk > 0 && topk <= skv / 128,
          "Skv must be a positive multiple of 128 and TopK at most the number of KV blocks");
  REQUIRE(static_cast<long long>(batch) * hkv * skv < (1LL << 31), "flattened KV rows must fit int32");
  REQUIRE(static_cast<long long>(batch) * hkv * sq * topk < (1LL << 31), "B*Hkv*Sq*TopK must fit int32 (edge offsets)");
  REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(partial) && aligned16(tasks), "misaligned pointer");
  const long long rows = static_cast<long long>(batch) * hkv * (skv / 128);
  return launch_kv_token_main(q, k, v, tasks, task_ptr + rows, query_ids, ranks, partial, partial_lse, batch, hq, hkv,
                              sq, skv, topk, 1, static_cast<cudaStream_t>(stream));
}

int sparse_b200_combine_tm(const void* partial_token_major, int partial_is_f32, const float* partial_lse, void* out,
                           float* out_lse, int batch, int hq, int sq, int ranks, void* stream) {
  REQUIRE(partial_token_major && partial_lse && out, "null pointer");
  REQUIRE(batch > 0 && hq > 0 && sq > 0 && ranks > 0, "sizes must be positive");
  REQUIRE(aligned16(partial_token_major) && aligned16(out), "misaligned pointer");
  const long long rows = static_cast<long long>(batch) * hq * sq;
  // rows run (batch, head, token) as in the output; the kernel finds a row's partials at
  // ((b * Sq + s) * ranks * Hq + h) * 128, one rank Hq * 128 elements further
  return launch_combine(partial_token_major, partial_is_f32, partial_lse, out, out_lse, rows, ranks,
                        static_cast<long long>(hq) * 128, 128, 1, ranks, static_cast<cudaStream_t>(stream), hq, sq);
}

int sparse_b200_peer_alloc(int64_t bytes, void** ptr, void* handle64) {
  REQUIRE(ptr && handle64 && bytes > 0, "peer_alloc needs a size, a pointer slot and 64 bytes for the handle");
  if (!device_ctx()) return SB_ERR_CUDA;
  return peer_alloc(bytes, ptr, handle64);
}

int sparse_b200_peer_open(const void* handle64, void** ptr) {
  REQUIRE(ptr && handle64, "null pointer");
  if (!device_ctx()) return SB_ERR_CUDA;
  return peer_open(handle64, ptr);
}

int sparse_b200_peer_close(void* ptr) {
  REQUIRE(ptr, "null pointer");
  return peer_close(ptr);
}

int sparse_b200_peer_free(void* ptr) {
  REQUIRE(ptr, "null pointer");
  return peer_free(ptr);
}

int sparse_b200_peer_signal(int32_t* const* flags, int count, int value, void* stream) {
  REQUIRE(flags, "null pointer");
  return launch_peer_signal(flags, count, value, static_cast<cudaStream_t>(stream));
}

int sparse_b200_peer_wait(const int32_t* flags, int count, int value, int wait_ms, void* stream) {
  REQUIRE(flags && count > 0, "null pointer");
  return launch_peer_wait(flags, count, value, wait_ms, static_cast<cudaStream_t>(stream));
}

int sparse_b200_combine_peer(const void* const* partials, const float* const* partial_lses, const int32_t* ready_flags,
                             int value, int wait_ms, void* out, float* out_lse, int64_t rows, int ranks,
                             void* stream) {
  REQUIRE(partials && partial_lses && out, "null pointer");
  REQUIRE(rows > 0, "rows must be positive");
  REQUIRE(aligned16(out), "misaligned pointer");
  return launch_combine_peer(partials, partial_lses, ready_flags, value, wait_ms, out, out_lse, rows, ranks,
                             static_cast<cudaStream_t>(stream));
}

int64_t sparse_b200_indexer_fp4_workspace_bytes(int batch, int hidx, int hk, int len_q, int len_kv) {
  if (batch <= 0 || hidx <= 0 || hk <= 0 || len_q <= 0 || len_kv <= 0) return SB_ERR_INVALID;
  const int64_t tile = align256(static_cast<size_t>(batch) * hidx * (len_q / 128) * (len_kv / 128) * 4);
  return 256 + tile;
}

int sparse_b200_indexer_fp4_fast(const void* q_codes, const void* q_scales, const void* k_codes, const void* k_scales,
                                 void* workspace, int64_t workspace_bytes, int32_t* block_idx, int batch, int hidx,
                                 int hk, int len_q, int len_kv, int topk, void* stream) {
  int rc = check_fp4(q_codes, q_scales, k_codes, k_scales, batch, hidx, hk, len_q, len_kv);
  if (rc) return rc;
  REQUIRE(workspace && block_idx && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
          "workspace must be a 256-byte aligned device pointer");
  REQUIRE(topk > 0 && topk <= len_kv / 128, "top-k must be in [1, kv_tiles]");
  REQUIRE(workspace_bytes >= sparse_b200_indexer_fp4_workspace_bytes(batch, hidx, hk, len_q, len_kv),
          "workspace too small (see sparse_b200_indexer_fp4_workspace_bytes)");
  unsigned char* w = static_cast<unsigned char*>(workspace);
  void* aux = w;
  float* tile_scores = reinterpret_cast<float*>(w + 256);
  rc = launch_fp4_indexer_tc(q_codes, q_scales, k_codes, k_scales, aux, block_idx, batch, hidx, hk, len_q, len_kv, topk,
                             static_cast<cudaStream_t>(stream));
  if (rc == 1) {   // few pages per list: exact tile scores + top-k, same ids
    // tensor-core values prune each (query tile, page) pair to the few elements that can hold its maximum
    rc = launch_fp4_scores_prune(q_codes, q_scales, k_codes, k_scales, aux, tile_scores, batch, hidx, hk, len_q, len_kv,
                                 static_cast<cudaStream_t>(stream));
    const bool pruned = rc == SB_OK;
    if (rc == 1)   // exact scorer that evaluates every element
      rc = launch_fp4_scores(q_codes, q_scales, k_codes, k_scales, nullptr, tile_scores, batch, hidx, hk, len_q, len_kv,
                             static_cast<cudaStream_t>(stream));
    if (rc) return rc;
    rc = launch_row_topk(tile_scores, block_idx, static_cast<long long>(batch) * hidx * (len_q / 128), len_kv / 128,
                         topk, static_cast<cudaStream_t>(stream), pruned);
  }
  return rc;
}

int sparse_b200_indexed_attention_fp4(const void* q, const void* k, const void* v, void* q_codes, void* q_scales,
                                      void* k_codes, void* k_scales, void* workspace, int64_t workspace_bytes,
                                      int32_t* block_idx, void* out, float* lse, int batch, int hq, int hkv, int sq,
                                      int skv, int topk, int quantize, void* stream) {
  REQUIRE(q && k && v && q_codes && q_scales && k_codes && k_scales && block_idx && out, "null pointer");
  REQUIRE(batch > 0 && hkv > 0 && hq >= hkv && hq % hkv == 0, "Hq must be a positive multiple of Hkv");
  REQUIRE(sq >= 128 && sq % 128 == 0 && skv >= 128 && skv % 128 == 0, "Sq and Skv must be positive multiples of 128");
  int rc = SB_OK;
  if (quantize) {
    // index vector of a (token, KV head) = NVFP4 of the mean of the group's query heads; keys as they are
    rc = sparse_b200_nvfp4_quantize(q, q_codes, q_scales, batch, hkv, hq / hkv, sq, 0, stream);
    if (rc) return rc;
    rc = sparse_b200_nvfp4_quantize(k, k_codes, k_scales, batch, hkv, 1, skv, 1, stream);
    if (rc) return rc;
  }
  rc = sparse_b200_indexer_fp4_fast(q_codes, q_scales, k_codes, k_scales, workspace, workspace_bytes, block_idx, batch,
                                    hkv, hkv, sq, skv, topk, stream);
  if (rc) return rc;
  // same stream: the ids written by the indexer are ready for the attention kernel
  return sparse_b200_q_centric(q, k, v, block_idx, nullptr, out, lse, batch, hq, hkv, sq, skv, topk, stream);
}

}  // extern "C"
