// NVFP4 block indexer: quantiser, exact scorer and tile top-k.
//
// Data contract (that of indexers/fp4/fp4.py:37-60): a 128-feature index vector
// is 64 bytes of e2m1 codes (low nibble = even feature) plus eight e4m3 scales,
// one per 16 features. Queries [B*Sq, Hidx, 64]; keys paged
// [B*Skv/128, Hk, 128, 64] with Hk = 1 (shared) or Hk = Hidx.
//
// Score arithmetic, exact until the last step, so the ids are reproducible bit
// for bit: with integer codes c = 2 * e2m1 value,
//   t_g = (sum_{i in group g} cq_i * ck_i) * (0.25 * qs_g * ks_g)   exact in fp32
//   dot = ((t_0 + t_1) + t_2) + ... + t_7                             fp32, in order
//   score(query, page) = max over the 128 keys of the page            (scorer)
//   tile score         = max over the 128 queries of a tile           (top-k input)
// Same quantities as Fp4IndexerStagedMmaSm100
// (indexers/fp4/vendor_minimax_msa/src/sm100/fp4_indexer.py:483-1086) followed by
// tile_max_topk16_kernel (indexers/fp4/tile_topk.cu:38-126), any top-k and any
// number of KV tiles; integer dot products run on dp4a.
#include "internal.h"
#include <cstdlib>
#include "topk.cuh"
#include "fp4_exact.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace sb {
namespace {

// ---------------------------------------------------------------- quantiser
// Rule (no counterpart in the reference, which feeds random bytes):
//   scale_g = e4m3_rne(min(amax_g / 6, 448)); code = nearest e2m1 to x / scale_g,
//   ties to the even code, saturating at 6; scale 0 -> codes 0.
// With group > 1 the input row is the fp32 mean, in head order, of `group`
// consecutive heads (index vector of a GQA group).
__device__ __forceinline__ uint32_t e2m1_code(float ratio) {
  const float a = fabsf(ratio);
  uint32_t c = 0;
  c = (a > 0.25f) ? 1u : c;                  // tie 0.25 -> 0
  c = (a >= 0.75f) ? 2u : c;                 // tie 0.75 -> 1.0 (code 2)
  c = (a > 1.25f) ? 3u : c;                  // tie 1.25 -> 1.0
  c = (a >= 1.75f) ? 4u : c;                 // tie 1.75 -> 2.0
  c = (a > 2.5f) ? 5u : c;                   // tie 2.5 -> 2.0
  c = (a >= 3.5f) ? 6u : c;                  // tie 3.5 -> 4.0
  c = (a > 5.0f) ? 7u : c;                   // tie 5.0 -> 4.0
  return (c != 0 && ratio < 0.f) ? (c | 8u) : c;
}

// x: [B, H_in, S, 128] bf16. Output row (b, h, s) quantises the fp32 mean, in
// head order, of heads h*group .. h*group+group-1 (group = 1: the head itself).
// Row placement: token-major [(b*S + s), h] (query index vectors) or paged
// [(b*S/128 + s/128), h, s%128] (key index pages). One thread per 16-feature group.
__global__ void __launch_bounds__(256) quantize_kernel(const __nv_bfloat16* __restrict__ x,
                                                       uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                                                       int batch, int heads_out, int group, int seq, int paged) {
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = gid >> 3;
  const int g16 = static_cast<int>(gid & 7);
  const long long rows = static_cast<long long>(batch) * heads_out * seq;
  if (row >= rows) return;
  const int s_pos = static_cast<int>(row % seq);
  const long long bh = row / seq;
  const int h = static_cast<int>(bh % heads_out);
  const long long b = bh / heads_out;
  const long long head_stride = static_cast<long long>(seq) * 128;
  const __nv_bfloat16* src =
      x + ((b * heads_out + h) * group) * head_stride + static_cast<long long>(s_pos) * 128 + g16 * 16;
  float v[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) v[e] = 0.f;
  for (int gh = 0; gh < group; ++gh) {
    const uint4* p = reinterpret_cast<const uint4*>(src + gh * head_stride);
    const uint4 a = __ldg(p), c = __ldg(p + 1);
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* hc = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fa = __bfloat1622float2(ha[e]), fc = __bfloat1622float2(hc[e]);
      v[2 * e] += fa.x; v[2 * e + 1] += fa.y;
      v[8 + 2 * e] += fc.x; v[8 + 2 * e + 1] += fc.y;
    }
  }
  if (group > 1) {
    const float gf = static_cast<float>(group);
#pragma unroll
    for (int e = 0; e < 16; ++e) v[e] = __fdiv_rn(v[e], gf);
  }
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(v[e]));
  const float want = fminf(__fdiv_rn(amax, 6.0f), 448.0f);
  const __nv_fp8_storage_t sbits = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
  const float sc = __half2float(__half(__nv_cvt_fp8_to_halfraw(sbits, __NV_E4M3)));
  uint32_t lo = 0, hi = 0;
  if (sc > 0.f) {
#pragma unroll
    for (int e = 0; e < 8; ++e) lo |= e2m1_code(__fdiv_rn(v[e], sc)) << (4 * e);
#pragma unroll
    for (int e = 0; e < 8; ++e) hi |= e2m1_code(__fdiv_rn(v[8 + e], sc)) << (4 * e);
  }
  long long dst;
  if (paged)
    dst = ((b * (seq >> 7) + (s_pos >> 7)) * heads_out + h) * 128 + (s_pos & 127);
  else
    dst = (b * seq + s_pos) * heads_out + h;
  *reinterpret_cast<uint2*>(packed + dst * 64 + g16 * 8) = make_uint2(lo, hi);
  scales[dst * 8 + g16] = sbits;
}

// ---------------------------------------------------------------- scorer
constexpr int ROW_WORDS = FP4_ROW_WORDS;

// One CTA: one query tile (128 queries of one index head) against `pages_per_cta`
// key pages. Thread (ty, tx) = (tid / 16, tid % 16) owns queries ty*8..ty*8+7 and
// keys tx, tx+16, ..., tx+112.
__global__ void __launch_bounds__(256) fp4_score_kernel(const uint8_t* __restrict__ qp, const uint8_t* __restrict__ qs,
                                                        const uint8_t* __restrict__ kp, const uint8_t* __restrict__ ks,
                                                        float* __restrict__ query_scores,  // [Hidx, tiles, B*Sq] or null
                                                        float* __restrict__ tile_scores,   // [B, Hidx, Qt, tiles] or null
                                                        int batch, int hidx, int hk, int len_q, int tiles,
                                                        int pages_per_cta) {
  __shared__ uint32_t q_i8[128 * ROW_WORDS];
  __shared__ uint32_t k_i8[128 * ROW_WORDS];
  __shared__ float q_sc[128 * 8];
  __shared__ float k_sc[128 * 8];
  __shared__ float red[8];

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int qt = len_q >> 7;
  const int qtile = blockIdx.y % qt;
  const int bh = blockIdx.y / qt;
  const int h = bh % hidx, b = bh / hidx;
  const long long q_row0 = static_cast<long long>(b) * len_q + static_cast<long long>(qtile) * 128;

  // stage the query tile: 128 rows x 16 words of codes, 8 scales (0.25 folded in)
  for (int e = tid; e < 128 * 16; e += 256) {
    const int r = e >> 4, w = e & 15;
    const uint32_t word = *reinterpret_cast<const uint32_t*>(qp + ((q_row0 + r) * hidx + h) * 64 + w * 4);
    uint32_t a, c;
    codes_to_int8(word, a, c);
    q_i8[r * ROW_WORDS + 2 * w] = a;
    q_i8[r * ROW_WORDS + 2 * w + 1] = c;
  }
  for (int e = tid; e < 128 * 8; e += 256)
    q_sc[e] = 0.25f * e4m3_to_float(qs[((q_row0 + (e >> 3)) * hidx + h) * 8 + (e & 7)]);

  const int page0 = blockIdx.x * pages_per_cta;
  for (int pg = page0; pg < min(page0 + pages_per_cta, tiles); ++pg) {
    __syncthreads();
    const long long page = (static_cast<long long>(b) * tiles + pg) * hk + (hk > 1 ? h : 0);
    for (int e = tid; e < 128 * 16; e += 256) {
      const int r = e >> 4, w = e & 15;
      const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(kp + (page * 128 + r) * 64 + w * 4));
      uint32_t a, c;
      codes_to_int8(word, a, c);
      k_i8[r * ROW_WORDS + 2 * w] = a;
      k_i8[r * ROW_WORDS + 2 * w + 1] = c;
    }
    for (int e = tid; e < 128 * 8; e += 256) k_sc[e] = e4m3_to_float(ks[(page * 128 + (e >> 3)) * 8 + (e & 7)]);
    __syncthreads();

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
#pragma unroll 1
    for (int g = 0; g < 8; ++g) {
      uint4 qv[8], kv[8];
      float qsc[8], ksc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        qv[i] = *reinterpret_cast<const uint4*>(&q_i8[(ty * 8 + i) * ROW_WORDS + g * 4]);
        qsc[i] = q_sc[(ty * 8 + i) * 8 + g];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        kv[j] = *reinterpret_cast<const uint4*>(&k_i8[(tx + 16 * j) * ROW_WORDS + g * 4]);
        ksc[j] = k_sc[(tx + 16 * j) * 8 + g];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // The integer sum is accumulated on top of the bit pattern of 1.5 * 2^23: the result
          // IS the float 12582912 + sum (|sum| <= 2304), and one exact subtraction gives
          // float(sum) without an int-to-float conversion (a quarter-rate instruction).
          int isum = __dp4a(static_cast<int>(qv[i].x), static_cast<int>(kv[j].x), 0x4B400000);
          isum = __dp4a(static_cast<int>(qv[i].y), static_cast<int>(kv[j].y), isum);
          isum = __dp4a(static_cast<int>(qv[i].z), static_cast<int>(kv[j].z), isum);
          isum = __dp4a(static_cast<int>(qv[i].w), static_cast<int>(kv[j].w), isum);
          // exact product (<= 12 + 8 significant bits), one rounding in the add
          acc[i][j] = fmaf(__int_as_float(isum) - 12582912.0f, qsc[i] * ksc[j], acc[i][j]);
        }
    }
    // per query: max over this thread's 8 keys, then over the 16 threads of the row
    float tile_best = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float m = acc[i][0];
#pragma unroll
      for (int j = 1; j < 8; ++j) m = fmaxf(m, acc[i][j]);
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
      if (query_scores && tx == 0)
        query_scores[(static_cast<long long>(h) * tiles + pg) * (static_cast<long long>(batch) * len_q) + q_row0 +
                     ty * 8 + i] = m;
      tile_best = fmaxf(tile_best, m);
    }
    if (tile_scores) {
      tile_best = fmaxf(tile_best, __shfl_xor_sync(0xffffffffu, tile_best, 16));
      if ((tid & 31) == 0) red[tid >> 5] = tile_best;
      __syncthreads();
      if (tid == 0) {
        float m = red[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
        tile_scores[((static_cast<long long>(b) * hidx + h) * qt + qtile) * tiles + pg] = m;
      }
    }
  }
}

// The same scores with the integer group sums on the tensor cores: one
// mma.sync.m16n8k16 (s8 x s8 -> s32) is exactly one 16-element scale group of a 16 x 8 patch
// of (query, key) pairs, and integer accumulation is exact, so every score is bit-identical
// with fp4_score_kernel: acc = fma(float(group sum), qs * ks, acc) in group order. The
// accumulator starts at the bit pattern of 1.5 * 2^23, which makes the result the float
// 12582912 + sum; one exact subtraction replaces the int-to-float conversion.
// Warp w owns queries 16 w .. 16 w + 15 against the 128 keys of the page (16 n-tiles).
__device__ __forceinline__ void mma_s8_16816(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, int c) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %8, %9, %10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(c), "r"(c), "r"(c), "r"(c));
}

__global__ void __launch_bounds__(256, 3) fp4_score_mma_kernel(const uint8_t* __restrict__ qp, const uint8_t* __restrict__ qs,
                                                            const uint8_t* __restrict__ kp, const uint8_t* __restrict__ ks,
                                                            float* __restrict__ query_scores,  // [Hidx, tiles, B*Sq] or null
                                                            float* __restrict__ tile_scores,   // [B, Hidx, Qt, tiles] or null
                                                            int batch, int hidx, int hk, int len_q, int tiles,
                                                            int pages_per_cta) {
  __shared__ uint32_t q_i8[128 * ROW_WORDS];
  __shared__ uint32_t k_i8[128 * ROW_WORDS];
  __shared__ float q_sc[128 * 8];
  __shared__ __align__(8) float k_sc[8 * 128];     // [group][key]
  __shared__ float red[8];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int m0 = warp * 16;
  const int qt = len_q >> 7;
  const int qtile = blockIdx.y % qt;
  const int bh = blockIdx.y / qt;
  const int h = bh % hidx, b = bh / hidx;
  const long long q_row0 = static_cast<long long>(b) * len_q + static_cast<long long>(qtile) * 128;

  for (int e = tid; e < 128 * 16; e += 256) {
    const int r = e >> 4, w = e & 15;
    const uint32_t word = *reinterpret_cast<const uint32_t*>(qp + ((q_row0 + r) * hidx + h) * 64 + w * 4);
    uint32_t a, c;
    codes_to_int8(word, a, c);
    q_i8[r * ROW_WORDS + 2 * w] = a;
    q_i8[r * ROW_WORDS + 2 * w + 1] = c;
  }
  for (int e = tid; e < 128 * 8; e += 256)
    q_sc[e] = 0.25f * e4m3_to_float(qs[((q_row0 + (e >> 3)) * hidx + h) * 8 + (e & 7)]);

  const int page0 = blockIdx.x * pages_per_cta;
  for (int pg = page0; pg < min(page0 + pages_per_cta, tiles); ++pg) {
    __syncthreads();
    const long long page = (static_cast<long long>(b) * tiles + pg) * hk + (hk > 1 ? h : 0);
    for (int e = tid; e < 128 * 16; e += 256) {
      const int r = e >> 4, w = e & 15;
      const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(kp + (page * 128 + r) * 64 + w * 4));
      uint32_t a, c;
      codes_to_int8(word, a, c);
      k_i8[r * ROW_WORDS + 2 * w] = a;
      k_i8[r * ROW_WORDS + 2 * w + 1] = c;
    }
    for (int e = tid; e < 128 * 8; e += 256)
      k_sc[(e & 7) * 128 + (e >> 3)] = e4m3_to_float(ks[(page * 128 + (e >> 3)) * 8 + (e & 7)]);
    __syncthreads();

    // two passes of 64 keys: 32 accumulators per thread instead of 64 keep three CTAs on an SM
    float r0 = -CUDART_INF_F, r1 = -CUDART_INF_F;
    const unsigned long long magic2 = f32x2_pack(12582912.0f, 12582912.0f);
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      unsigned long long acc[8][2];               // (row gid: two keys), (row gid + 8: two keys) per n-tile
#pragma unroll
      for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = 0ull;
#pragma unroll 1
      for (int g = 0; g < 8; ++g) {
        const uint32_t a0 = q_i8[(m0 + gid) * ROW_WORDS + g * 4 + tig];
        const uint32_t a1 = q_i8[(m0 + 8 + gid) * ROW_WORDS + g * 4 + tig];
        const float qs0 = q_sc[(m0 + gid) * 8 + g], qs1 = q_sc[(m0 + 8 + gid) * 8 + g];
        const unsigned long long q0 = f32x2_pack(qs0, qs0), q1 = f32x2_pack(qs1, qs1);
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int key0 = half * 64 + n * 8;
          const uint32_t b0 = k_i8[(key0 + gid) * ROW_WORDS + g * 4 + tig];
          const unsigned long long kk = *reinterpret_cast<const unsigned long long*>(&k_sc[g * 128 + key0 + tig * 2]);
          int d[4];
          mma_s8_16816(d, a0, a1, b0, 0x4B400000);
          // exact products (<= 12 + 8 significant bits), one rounding in each add; two lanes per instruction
          acc[n][0] = f32x2_fma(f32x2_sub(f32x2_pack_bits(d[0], d[1]), magic2), f32x2_mul(q0, kk), acc[n][0]);
          acc[n][1] = f32x2_fma(f32x2_sub(f32x2_pack_bits(d[2], d[3]), magic2), f32x2_mul(q1, kk), acc[n][1]);
        }
      }
      // per query: max over the thread's keys of each of its two rows
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        float x0, x1, x2, x3;
        f32x2_unpack(acc[n][0], x0, x1);
        f32x2_unpack(acc[n][1], x2, x3);
        r0 = fmaxf(r0, fmaxf(x0, x1));
        r1 = fmaxf(r1, fmaxf(x2, x3));
      }
    }
    // ... then over the quad
#pragma unroll
    for (int dlt = 1; dlt < 4; dlt <<= 1) {
      r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, dlt));
      r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, dlt));
    }
    if (query_scores && tig == 0) {
      float* dst = query_scores + (static_cast<long long>(h) * tiles + pg) * (static_cast<long long>(batch) * len_q) +
                   q_row0 + m0 + gid;
      dst[0] = r0;
      dst[8] = r1;
    }
    if (tile_scores) {
      float tile_best = fmaxf(r0, r1);
#pragma unroll
      for (int dlt = 4; dlt < 32; dlt <<= 1) tile_best = fmaxf(tile_best, __shfl_xor_sync(0xffffffffu, tile_best, dlt));
      if (lane == 0) red[warp] = tile_best;
      __syncthreads();
      if (tid == 0) {
        float m = red[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
        tile_scores[((static_cast<long long>(b) * hidx + h) * qt + qtile) * tiles + pg] = m;
      }
    }
  }
}

// ---------------------------------------------------------------- top-k stages
// query_scores [H, tiles, B*Sq] -> max over the 128 queries of a tile -> top-k
// (tile_max_topk16_kernel, indexers/fp4/tile_topk.cu:38-126, any k and tile count).
__global__ void __launch_bounds__(256) tile_max_topk_kernel(const float* __restrict__ query_scores,
                                                            int32_t* __restrict__ ids, int batch, int heads,
                                                            int len_q, int tiles, int topk) {
  extern __shared__ float smem[];
  float* scores = smem;
  float* scratch_f = scores + tiles;
  int* scratch_i = reinterpret_cast<int*>(scratch_f + 10);
  const int qt = len_q >> 7;
  const int row = blockIdx.x;                 // (b * heads + h) * qt + qtile
  const int qtile = row % qt, bh = row / qt, h = bh % heads, b = bh / heads;
  const long long total_q = static_cast<long long>(batch) * len_q;
  const long long q0 = static_cast<long long>(b) * len_q + static_cast<long long>(qtile) * 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = warp; t < tiles; t += 8) {
    const float4 v = *reinterpret_cast<const float4*>(query_scores + (static_cast<long long>(h) * tiles + t) * total_q +
                                                      q0 + lane * 4);
    float m = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if (lane == 0) scores[t] = m;
  }
  __syncthreads();
  block_topk(scores, tiles, topk, ids + static_cast<long long>(row) * topk, scratch_f, scratch_i);
}

// tile_scores [rows, tiles] -> top-k per row
__global__ void __launch_bounds__(256) row_topk_kernel(const float* __restrict__ tile_scores, int32_t* __restrict__ ids,
                                                       int tiles, int topk) {
  extern __shared__ float smem[];
  float* scores = smem;
  float* scratch_f = scores + tiles;
  int* scratch_i = reinterpret_cast<int*>(scratch_f + 10);
  const long long row = blockIdx.x;
  bool has_nan = false;
  // when launched as a programmatic dependent of the scoring kernel: wait for that grid's results
  // (returns at once in an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const float v = tile_scores[row * tiles + t];
    scores[t] = v;
    has_nan |= v != v;
  }
  // Short rows without NaN: the rank of a tile is the number of tiles that beat it (score
  // descending, index ascending), one tile per thread and step; k rounds of block-wide
  // arg-max cost more than that up to about a thousand tiles.
  if (!__syncthreads_or(has_nan) && tiles <= 1024) {
    for (int i = threadIdx.x; i < tiles; i += blockDim.x) {
      const float si = scores[i];
      int rank = 0;
#pragma unroll 4
      for (int j = 0; j < tiles; ++j) {
        const float sj = scores[j];
        rank += static_cast<int>(sj > si) | (static_cast<int>(sj == si) & static_cast<int>(j < i));
      }
      if (rank < topk) ids[row * topk + rank] = i;
    }
    return;
  }
  block_topk(scores, tiles, topk, ids + row * topk, scratch_f, scratch_i);
}

}  // namespace

static int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

int launch_quantize(const void* x, void* packed, void* scales, int batch, int heads_out, int group, int seq,
                    int paged, cudaStream_t stream) {
  const long long threads = static_cast<long long>(batch) * heads_out * seq * 8;
  quantize_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scales), batch,
      heads_out, group, seq, paged);
  return check_launch();
}

int launch_fp4_scores(const void* qp, const void* qs, const void* kp, const void* ks, float* query_scores,
                      float* tile_scores, int batch, int hidx, int hk, int len_q, int len_kv, cudaStream_t stream) {
  const int tiles = len_kv / 128, qt = len_q / 128;
  int pages_per_cta = 8;
  while (pages_per_cta > 1 && static_cast<long long>((tiles + pages_per_cta - 1) / pages_per_cta) * batch * hidx * qt < 592)
    pages_per_cta >>= 1;
  dim3 grid((tiles + pages_per_cta - 1) / pages_per_cta, batch * hidx * qt);
  // integer group sums on the tensor cores (bit-identical scores); SB_FP4_DP4A=1 keeps the dp4a kernel
  static const bool use_dp4a = [] { const char* e = getenv("SB_FP4_DP4A"); return e && e[0] == '1'; }();
  if (use_dp4a)
    fp4_score_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(qp), static_cast<const uint8_t*>(qs),
                                               static_cast<const uint8_t*>(kp), static_cast<const uint8_t*>(ks),
                                               query_scores, tile_scores, batch, hidx, hk, len_q, tiles, pages_per_cta);
  else
    fp4_score_mma_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(qp), static_cast<const uint8_t*>(qs),
                                                   static_cast<const uint8_t*>(kp), static_cast<const uint8_t*>(ks),
                                                   query_scores, tile_scores, batch, hidx, hk, len_q, tiles,
                                                   pages_per_cta);
  return check_launch();
}

static int topk_smem(int tiles) { return (tiles + 10) * sizeof(float) + 16 * sizeof(int); }

int launch_tile_max_topk(const float* query_scores, int32_t* ids, int batch, int heads, int len_q, int tiles, int topk,
                         cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  if (topk_smem(tiles) > 200 * 1024) return set_error(SB_ERR_INVALID, "too many KV tiles for the top-k stage");
  if (!ctx->misc_attr[5]) {
    cudaFuncSetAttribute(tile_max_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(row_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    ctx->misc_attr[5] = 1;
  }
  tile_max_topk_kernel<<<batch * heads * (len_q / 128), 256, topk_smem(tiles), stream>>>(query_scores, ids, batch, heads,
                                                                                         len_q, tiles, topk);
  return check_launch();
}

// after_scorer: launch as a programmatic dependent of the kernel launched just before on the stream
// (which must execute griddepcontrol.launch_dependents), so that launch latency and prologue overlap its tail.
int launch_row_topk(const float* tile_scores, int32_t* ids, long long rows, int tiles, int topk, cudaStream_t stream,
                    bool after_scorer) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  if (topk_smem(tiles) > 200 * 1024) return set_error(SB_ERR_INVALID, "too many KV tiles for the top-k stage");
  if (!ctx->misc_attr[5]) {
    cudaFuncSetAttribute(tile_max_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(row_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    ctx->misc_attr[5] = 1;
  }
  if (after_scorer) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(rows));
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = topk_smem(tiles);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, row_topk_kernel, tile_scores, ids, tiles, topk);
    return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  }
  row_topk_kernel<<<static_cast<unsigned>(rows), 256, topk_smem(tiles), stream>>>(tile_scores, ids, tiles, topk);
  return check_launch();
}

}  // namespace sb
