// NVFP4 scorer for ragged batches over a paged key cache, optionally causal: per query and
// 128-key page the maximum score over the keys the query may see.
//
//   q codes  [total_q, Hq, 64] u8 (two e2m1 codes per byte), scales [total_q, Hq, 8] e4m3
//   k codes  [total_pages, Hk, 128, 64], scales [total_pages, Hk, 128, 8]
//   cu_seqlens_q / cu_seqlens_k / cu_page_offsets [B + 1] int32, kv_indices [sum of pages] int32
//   out      [Hq, ceil(max_seqlen_k / 128), total_q] fp32, -inf where a query sees no key of a page
//
// Request b owns queries cu_seqlens_q[b] .. cu_seqlens_q[b+1], keys 0 .. k_len of the logical
// pages kv_indices[cu_page_offsets[b] + t]; query head h reads key head h / (Hq / Hk). Causal:
// key j is visible to query i when j <= i + offset, offset = k_len - q_len unless qo_offset[b]
// is given. The contract of fp4_indexer_block_scores
// (indexers/fp4/vendor_minimax_msa/fp4_indexer_interface.py:745-811; offset rule
// src/sm100/fp4_indexer.py:525-529). Arithmetic: the exact one of indexer_fp4.cu (integer group
// sums on the tensor cores, scaled and added in group order), so scores are bit-identical with
// the dense scorer wherever both apply.
//
// Decode batches (every request has at most 8 new queries) take the PACKED form of the kernel: the
// 128 rows of a CTA are (head of one KV-head group, query) pairs, 8 query slots for each of up to 16
// heads, so that one pass over a key page serves the whole group instead of one head with 8 of 128
// rows alive; the role of Fp4IndexerDecodePackedQSm100
// (indexers/fp4/vendor_minimax_msa/src/sm100/fp4_indexer.py:1110-1229, taken there when
// max_seqlen_q <= 8 and Hq / Hk = 16; here for any group size). Same arithmetic, same scores.
#include <algorithm>
#include "fp4_exact.cuh"
#include "internal.h"
#include <math_constants.h>

namespace sb {
namespace {

constexpr int RW = FP4_ROW_WORDS;

__global__ void __launch_bounds__(256) fill_neg_inf_kernel(float* out, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = -CUDART_INF_F;
}

struct VarlenParams {
  const uint8_t* qp; const uint8_t* qs; const uint8_t* kp; const uint8_t* ks;
  const int32_t* cu_q; const int32_t* cu_k; const int32_t* cu_pages; const int32_t* kv_indices;
  const int32_t* qo_offset;     // may be null
  float* out;
  int batch, hq, hk, total_q, total_pages, qt_max, tiles_out, pages_per_cta, causal;
  int head_blocks;              // packed form: blocks of 16 heads per KV-head group
};

constexpr int PACK_Q = 8;       // query slots per head in the packed (decode) form
constexpr int PACK_HEADS = 16;  // heads per CTA in the packed form

// blockIdx.x = (request, query tile, query head), or (request, KV head, block of 16 group heads) in the
// packed form; blockIdx.y = chunk of logical pages. Warp w owns rows 16 w .. 16 w + 15 of the CTA
// against the 128 keys of a page. Row r is query qtile * 128 + r of head h, or, packed, query r % 8 of
// the (r / 8)-th head of the block.
template <bool PACKED>
__global__ void __launch_bounds__(256, 3) fp4_score_varlen_kernel(const VarlenParams p) {
  __shared__ uint32_t q_i8[128 * RW];
  __shared__ uint32_t k_i8[128 * RW];
  __shared__ float q_sc[128 * 8];
  __shared__ __align__(8) float k_sc[8 * 128];     // [group][key]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3, m0 = warp * 16;
  const int group = p.hq / p.hk;
  int h, qtile, b, head_block = 0, hk_packed = 0;
  if (PACKED) {
    head_block = blockIdx.x % p.head_blocks;
    const int rest = blockIdx.x / p.head_blocks;
    hk_packed = rest % p.hk;
    b = rest / p.hk;
    qtile = 0;
    h = hk_packed * group + head_block * PACK_HEADS;       // first head of the block
  } else {
    h = blockIdx.x % p.hq;
    const int rest = blockIdx.x / p.hq;
    qtile = rest % p.qt_max;
    b = rest / p.qt_max;
  }
  const int heads_here = PACKED ? min(PACK_HEADS, group - head_block * PACK_HEADS) : 1;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int k_len = p.cu_k[b + 1] - p.cu_k[b];
  if (qtile * 128 >= q_len || k_len <= 0) return;          // block-uniform
  // Inconsistent arguments must not become out-of-range accesses: the page loop stays inside the
  // output's page axis (sized from max_seqlen_k on the host) and inside this request's slice of
  // kv_indices, and the live rows stay inside total_q.
  const int page_begin = p.cu_pages[b];
  const int pages = min(min((k_len + 127) >> 7, p.tiles_out), p.cu_pages[b + 1] - page_begin);
  if (q_begin < 0 || page_begin < 0) return;               // block-uniform
  const int offset = p.causal ? (p.qo_offset ? p.qo_offset[b] : k_len - q_len) : 0;
  const int hk_idx = PACKED ? hk_packed : h / group;
  // queries of the request that this CTA serves (the packed form holds at most PACK_Q of them)
  const int rows_live = min(min(PACKED ? PACK_Q : 128, q_len - qtile * 128), p.total_q - q_begin - qtile * 128);
  if (rows_live <= 0) return;                              // block-uniform
  // row r of the CTA -> query position inside the request, head, alive?
  auto row_query = [&](int r) { return PACKED ? (r & (PACK_Q - 1)) : qtile * 128 + r; };
  auto row_head = [&](int r) { return PACKED ? h + (r >> 3) : h; };
  auto row_alive = [&](int r) {
    return PACKED ? ((r >> 3) < heads_here && (r & (PACK_Q - 1)) < rows_live) : r < rows_live;
  };

  // stage the query tile (rows past the request's end as zeros)
  for (int e = tid; e < 128 * 16; e += 256) {
    const int r = e >> 4, w = e & 15;
    uint32_t a = 0, c = 0;
    if (row_alive(r)) {
      const uint32_t word = *reinterpret_cast<const uint32_t*>(
          p.qp + ((static_cast<long long>(q_begin) + row_query(r)) * p.hq + row_head(r)) * 64 + w * 4);
      codes_to_int8(word, a, c);
    }
    q_i8[r * RW + 2 * w] = a;
    q_i8[r * RW + 2 * w + 1] = c;
  }
  for (int e = tid; e < 128 * 8; e += 256) {
    const int r = e >> 3;
    q_sc[e] = row_alive(r)
                  ? 0.25f * e4m3_to_float(p.qs[((static_cast<long long>(q_begin) + row_query(r)) * p.hq + row_head(r)) * 8 + (e & 7)])
                  : 0.f;
  }

  const unsigned long long magic2 = f32x2_pack(12582912.0f, 12582912.0f);
  const int page0 = blockIdx.y * p.pages_per_cta;
  for (int pg = page0; pg < min(page0 + p.pages_per_cta, pages); ++pg) {
    // nothing of this page is visible to the last live query of the tile: it stays -inf
    if (p.causal && pg * 128 > (PACKED ? 0 : qtile * 128) + rows_live - 1 + offset) break;
    const int phys = p.kv_indices[page_begin + pg];
    if (phys < 0 || phys >= p.total_pages) continue;       // block-uniform; the page stays -inf
    __syncthreads();
    const long long page = static_cast<long long>(phys) * p.hk + hk_idx;
    for (int e = tid; e < 128 * 16; e += 256) {
      const int r = e >> 4, w = e & 15;
      const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(p.kp + (page * 128 + r) * 64 + w * 4));
      uint32_t a, c;
      codes_to_int8(word, a, c);
      k_i8[r * RW + 2 * w] = a;
      k_i8[r * RW + 2 * w + 1] = c;
    }
    for (int e = tid; e < 128 * 8; e += 256)
      k_sc[(e & 7) * 128 + (e >> 3)] = e4m3_to_float(p.ks[(page * 128 + (e >> 3)) * 8 + (e & 7)]);
    __syncthreads();

    const int row0 = m0 + gid, row1 = row0 + 8;               // this thread's two rows
    const int qi0 = row_query(row0), qi1 = row_query(row1);   // and their query positions
    float r0 = -CUDART_INF_F, r1 = -CUDART_INF_F;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      unsigned long long acc[8][2];
#pragma unroll
      for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = 0ull;
#pragma unroll 1
      for (int g = 0; g < 8; ++g) {
        const uint32_t a0 = q_i8[(m0 + gid) * RW + g * 4 + tig];
        const uint32_t a1 = q_i8[(m0 + 8 + gid) * RW + g * 4 + tig];
        const float qs0 = q_sc[(m0 + gid) * 8 + g], qs1 = q_sc[(m0 + 8 + gid) * 8 + g];
        const unsigned long long q0 = f32x2_pack(qs0, qs0), q1 = f32x2_pack(qs1, qs1);
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int key0 = half * 64 + n * 8;
          const uint32_t b0 = k_i8[(key0 + gid) * RW + g * 4 + tig];
          const unsigned long long kk = *reinterpret_cast<const unsigned long long*>(&k_sc[g * 128 + key0 + tig * 2]);
          int d0, d1, d2, d3;
          asm volatile(
              "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};"
              : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
              : "r"(a0), "r"(a1), "r"(b0), "r"(0x4B400000));
          acc[n][0] = f32x2_fma(f32x2_sub(f32x2_pack_bits(d0, d1), magic2), f32x2_mul(q0, kk), acc[n][0]);
          acc[n][1] = f32x2_fma(f32x2_sub(f32x2_pack_bits(d2, d3), magic2), f32x2_mul(q1, kk), acc[n][1]);
        }
      }
      // maximum over the keys each of the two queries may see
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        float x0, x1, x2, x3;
        f32x2_unpack(acc[n][0], x0, x1);
        f32x2_unpack(acc[n][1], x2, x3);
        const int kj = pg * 128 + half * 64 + n * 8 + tig * 2;
        const bool in0 = kj < k_len, in1 = kj + 1 < k_len;
        const int lim0 = p.causal ? qi0 + offset : 0x7fffffff, lim1 = p.causal ? qi1 + offset : 0x7fffffff;
        if (in0 && kj <= lim0) r0 = fmaxf(r0, x0);
        if (in1 && kj + 1 <= lim0) r0 = fmaxf(r0, x1);
        if (in0 && kj <= lim1) r1 = fmaxf(r1, x2);
        if (in1 && kj + 1 <= lim1) r1 = fmaxf(r1, x3);
      }
    }
#pragma unroll
    for (int dlt = 1; dlt < 4; dlt <<= 1) {
      r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, dlt));
      r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, dlt));
    }
    if (tig == 0) {
      if (row_alive(row0))
        p.out[(static_cast<long long>(row_head(row0)) * p.tiles_out + pg) * p.total_q + q_begin + qi0] = r0;
      if (row_alive(row1))
        p.out[(static_cast<long long>(row_head(row1)) * p.tiles_out + pg) * p.total_q + q_begin + qi1] = r1;
    }
  }
}

}  // namespace

int launch_fp4_scores_varlen(const void* qp, const void* qs, const void* kp, const void* ks, const int32_t* cu_q,
                             const int32_t* cu_k, const int32_t* cu_pages, const int32_t* kv_indices,
                             const int32_t* qo_offset, float* out, int batch, int hq, int hk, int total_q,
                             int total_pages, int max_seqlen_q, int max_seqlen_k, int causal, cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  VarlenParams p{};
  p.qp = static_cast<const uint8_t*>(qp); p.qs = static_cast<const uint8_t*>(qs);
  p.kp = static_cast<const uint8_t*>(kp); p.ks = static_cast<const uint8_t*>(ks);
  p.cu_q = cu_q; p.cu_k = cu_k; p.cu_pages = cu_pages; p.kv_indices = kv_indices; p.qo_offset = qo_offset;
  p.out = out;
  p.batch = batch; p.hq = hq; p.hk = hk; p.total_q = total_q; p.total_pages = total_pages;
  p.qt_max = (max_seqlen_q + 127) / 128;
  p.tiles_out = (max_seqlen_k + 127) / 128;
  p.causal = causal;
  const long long n = static_cast<long long>(hq) * p.tiles_out * total_q;
  const long long fill_blocks = std::min<long long>((n + 255) / 256, 4LL * ctx->sm_count * 8);
  fill_neg_inf_kernel<<<static_cast<unsigned>(fill_blocks > 0 ? fill_blocks : 1), 256, 0, stream>>>(out, n);
  // decode batches: every request at most PACK_Q queries -> rows of a CTA = (group head, query) pairs
  const bool packed = max_seqlen_q <= PACK_Q && hq / hk > 1;
  p.head_blocks = (hq / hk + PACK_HEADS - 1) / PACK_HEADS;
  const long long items = packed ? static_cast<long long>(batch) * hk * p.head_blocks
                                 : static_cast<long long>(batch) * p.qt_max * hq;
  if (items > 0x7fffffffLL) return set_error(SB_ERR_INVALID, "too many (request, query tile, head) items");
  int ppc = 8;
  while (ppc > 1 && ((p.tiles_out + ppc - 1) / ppc) * items < 4LL * ctx->sm_count) ppc >>= 1;
  p.pages_per_cta = ppc;
  const dim3 grid(static_cast<unsigned>(items), static_cast<unsigned>((p.tiles_out + ppc - 1) / ppc));
  if (grid.y > 65535) return set_error(SB_ERR_INVALID, "too many KV pages per request");
  if (items > 0 && p.tiles_out > 0) {
    if (packed)
      fp4_score_varlen_kernel<true><<<grid, 256, 0, stream>>>(p);
    else
      fp4_score_varlen_kernel<false><<<grid, 256, 0, stream>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
