// Tensor-core path of the NVFP4 indexer: the same block ids as the exact dp4a scorer
// followed by tile top-k, bit for bit.
//
// A dequantised NVFP4 value (e2m1 code x e4m3 scale) has at most 7 significant bits
// and is exactly representable in bf16, so bf16 tensor-core MMAs on dequantised
// copies compute every product exactly; only their fp32 accumulation differs from
// the fixed group-by-group order that defines a score. As in the summary indexer
// the MMA result is therefore a PRE-FILTER: per query tile the C best pages by
// approximate tile score are the candidates. Approximate and exact score of a page differ
// by at most delta = 2^-14 * min(max_q ||q||_1 * max|k|, max_q ||q||_2 * max_k ||k||_2),
// so candidates more than 2 delta apart are ordered by their approximate scores for
// certain; the others are re-scored exactly. The top-k of the candidates is the answer
// when a lower bound of the k-th exact score > C-th approximate score + delta, and the
// tile falls back to exact scores of every page otherwise.
// Same role as Fp4IndexerStagedMmaSm100 + tile_max_topk16_kernel
// (indexers/fp4/vendor_minimax_msa/src/sm100/fp4_indexer.py:483-1086,
// indexers/fp4/tile_topk.cu:38-126).
#include "ptx.cuh"
#include "internal.h"
#include "topk.cuh"
#include "fp4_exact.cuh"
#include <cuda_bf16.h>

namespace sb {
namespace ftc {

constexpr int TILE_BYTES = 128 * 256;
constexpr int PANEL_BYTES = 128 * 128;
constexpr int A_STAGES = 2;
constexpr int C_MAX = 192;
constexpr int NUM_THREADS = 320;
constexpr int TMA_WARP = 8, MMA_WARP = 9;
constexpr float EPS = 6.103515625e-05f;   // 2^-14
constexpr int MAX_TILES = 16384;           // 64 KiB of scores

constexpr int OFF_A = 0;
constexpr int OFF_B = A_STAGES * TILE_BYTES;
constexpr int OFF_SCORES = OFF_B + TILE_BYTES;

struct Params {
  const uint8_t *qp, *qs, *kp, *ks;   // public NVFP4 layout (codes, e4m3 scales)
  const float* k_absmax;              // [0] max |dequantised key element|, [2] largest squared L2 norm of a key
  int32_t* ids;                       // [B, Hidx, Qt, topk]
  int* status;
  int* fallbacks;
  int batch, hidx, hk, len_q, tiles, topk, cand;
};

__device__ __forceinline__ int f2ord(float f) {
  const int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// codes + scales -> bf16 (exact). One thread per 8 features.
// Rows 0 .. q_rows - 1 are query vectors, the rest key vectors (both row counts are multiples
// of 16, so a block of 16 rows never holds both). Sixteen adjacent threads hold one row. For
// the key rows the largest |element| and the largest squared L2 norm go to stats[0] and
// stats[2] (stats[1] belongs to the caller), one pair of atomics per block.
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ q_codes, const uint8_t* __restrict__ q_scales,
                                                      __nv_bfloat16* __restrict__ q_out, long long q_rows,
                                                      const uint8_t* __restrict__ k_codes, const uint8_t* __restrict__ k_scales,
                                                      __nv_bfloat16* __restrict__ k_out, long long k_rows,
                                                      float* __restrict__ stats) {
  __shared__ float red_m[8], red_n[8];
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  long long row = gid >> 4;
  const int w = static_cast<int>(gid & 15);
  const bool is_key = row >= q_rows;
  const uint8_t* codes = is_key ? k_codes : q_codes;
  const uint8_t* scales = is_key ? k_scales : q_scales;
  __nv_bfloat16* out = is_key ? k_out : q_out;
  if (is_key) row -= q_rows;
  const bool live = row < (is_key ? k_rows : q_rows);
  float amax = 0.f, squares = 0.f;
  if (live) {
    const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(codes + row * 64 + w * 4));
    const float sc = 0.5f * e4m3_to_float(scales[row * 8 + (w >> 1)]);
    const unsigned long long lut = 0x0C08060403020100ULL;
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float f[2];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t c = (word >> (4 * (2 * e + t))) & 15u;
        float m = static_cast<float>((lut >> (8 * (c & 7u))) & 0xFFu);
        f[t] = ((c & 8u) ? -m : m) * sc;
        amax = fmaxf(amax, fabsf(f[t]));
        squares = fmaf(f[t], f[t], squares);
      }
      __nv_bfloat162 h = __floats2bfloat162_rn(f[0], f[1]);
      ow[e] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + row * 128 + w * 8) = o;
  }
  if (!is_key) return;                       // uniform within the block
#pragma unroll
  for (int d = 8; d > 0; d >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, d);   // the row's 16 threads
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    squares = fmaxf(squares, __shfl_xor_sync(0xffffffffu, squares, d));
  }
  if ((threadIdx.x & 31) == 0) {
    red_m[threadIdx.x >> 5] = amax;
    red_n[threadIdx.x >> 5] = squares;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) {
      amax = fmaxf(amax, red_m[i]);
      squares = fmaxf(squares, red_n[i]);
    }
    atomicMax(reinterpret_cast<int*>(stats), __float_as_int(amax));
    atomicMax(reinterpret_cast<int*>(stats + 2), __float_as_int(squares));
  }
}

// One CTA per (batch, index head, query tile), two CTAs per SM (the exact re-scoring of one
// overlaps the tensor-core scoring of the other): approximate tile scores of every key
// page on the tensor cores, then candidate selection and exact re-scoring.
// Warps 0-7 epilogue (lane quarter = warp & 3, column half = warp >> 2), warp 8 TMA,
// warp 9 MMA issue.
__global__ void __launch_bounds__(NUM_THREADS, 2)
fp4_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw);
  int* scores = reinterpret_cast<int*>(gbase + OFF_SCORES);
  const int score_bytes = (p.tiles * 4 + 15) & ~15;
  unsigned char* aux = gbase + OFF_SCORES + score_bytes;
  const uint32_t bar0 = base + OFF_SCORES + score_bytes;
  volatile int* misc = reinterpret_cast<volatile int*>(aux + 128);   // tmem base, abort, unsafe, l1q bits
  float* scratch_f = reinterpret_cast<float*>(aux + 192);            // [16]
  int* scratch_i = reinterpret_cast<int*>(aux + 256);                // [16]
  auto bar = [&](int i) { return bar0 + 8u * i; };
  enum { A_FULL = 0, A_EMPTY = A_STAGES, B_FULL = 2 * A_STAGES, ACC_FULL = 2 * A_STAGES + 1, ACC_EMPTY = 2 * A_STAGES + 3 };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = p.len_q >> 7;
  const int qtile = blockIdx.x % qt;
  const int bh = blockIdx.x / qt;
  const int h = bh % p.hidx, b = bh / p.hidx;
  const int hk_idx = p.hk > 1 ? h : 0;
  const long long q_row0 = static_cast<long long>(b) * p.len_q + static_cast<long long>(qtile) * 128;
  const int num_tiles = p.tiles;
  const int rot = static_cast<int>((static_cast<unsigned>(qtile) * 37u) % static_cast<unsigned>(num_tiles));
  Guard guard{misc + 1, p.status};

  if (threadIdx.x == 0) {
    misc[1] = 0;
    for (int i = 0; i < A_STAGES; ++i) {
      mbar_init(bar(A_FULL + i), 1);
      mbar_init(bar(A_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(ACC_FULL + i), 1);
      mbar_init(bar(ACC_EMPTY + i), 8);
    }
    mbar_init(bar(B_FULL), 1);
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), 256);
    tmem_relinquish();
  }
  for (int j = threadIdx.x; j < p.tiles; j += NUM_THREADS) scores[j] = static_cast<int>(0x80000000u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = static_cast<uint32_t>(misc[0]);

  if (warp == TMA_WARP) {
    if (lane == 0) {
      mbar_expect_tx(bar(B_FULL), TILE_BYTES);
      tma_load_3d(base + OFF_B, &q_map, 0, h, static_cast<int>(q_row0), bar(B_FULL));
      tma_load_3d(base + OFF_B + PANEL_BYTES, &q_map, 64, h, static_cast<int>(q_row0), bar(B_FULL));
    }
    bool ok = true;
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int s = t % A_STAGES, use = t / A_STAGES;
      if (use > 0) {
        bool w = mbar_wait(bar(A_EMPTY + s), (use - 1) & 1, guard, 0x500 + s);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
      }
      if (lane == 0) {
        const uint32_t dst = base + OFF_A + s * TILE_BYTES;
        const int pg = (t + rot) % num_tiles;
        const int row = ((b * p.tiles + pg) * p.hk + hk_idx) * 128;
        mbar_expect_tx(bar(A_FULL + s), TILE_BYTES);
        tma_load_2d(dst, &k_map, 0, row, bar(A_FULL + s));
        tma_load_2d(dst + PANEL_BYTES, &k_map, 64, row, bar(A_FULL + s));
      }
    }
    if (!ok)
      for (int t = max(0, num_tiles - A_STAGES); t < num_tiles; ++t)
        mbar_wait_drain(bar(A_FULL + t % A_STAGES), (t / A_STAGES) & 1);
  } else if (warp == MMA_WARP) {
    const uint32_t idesc = idesc_bf16(128, 128, false);
    bool ok = true;
    {
      bool w = mbar_wait(bar(B_FULL), 0, guard, 0x510);
      ok = __all_sync(0xffffffffu, w);
      tc_fence_after();
    }
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int s = t % A_STAGES, acc = t & 1;
      bool w = mbar_wait(bar(A_FULL + s), (t / A_STAGES) & 1, guard, 0x520 + s);
      if (w && t >= 2) w = mbar_wait(bar(ACC_EMPTY + acc), ((t >> 1) - 1) & 1, guard, 0x530 + acc);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint64_t a0 = desc_sw128_kmajor(base + OFF_A + s * TILE_BYTES);
        const uint64_t b0 = desc_sw128_kmajor(base + OFF_B);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t step = static_cast<uint64_t>((kk >> 2) * (PANEL_BYTES >> 4) + (kk & 3) * 2);
          mma_ss(tmem + acc * 128, a0 + step, b0 + step, idesc, kk > 0);
        }
        tc_commit(bar(A_EMPTY + s));
        tc_commit(bar(ACC_FULL + acc));
      }
    }
  } else {
    // epilogue: thread = key row of the page, this warp's 64-column half of the query tile
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int half = warp >> 2;
    bool ok = true;
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int acc = t & 1;
      bool w = mbar_wait(bar(ACC_FULL + acc), (t >> 1) & 1, guard, 0x540 + acc);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem + lane_base + acc * 128 + half * 64;
      uint32_t v[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(t_acc + c * 16, v[c]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(ACC_EMPTY + acc));
      float m4[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float m5[5];
#pragma unroll
        for (int j = 0; j < 5; ++j)
          m5[j] = max3(__uint_as_float(v[c][3 * j]), __uint_as_float(v[c][3 * j + 1]), __uint_as_float(v[c][3 * j + 2]));
        m4[c] = fmaxf(max3(m5[0], m5[1], m5[2]), max3(m5[3], m5[4], __uint_as_float(v[c][15])));
      }
      float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
      if (lane == 0) atomicMax(&scores[(t + rot) % num_tiles], f2ord(m));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
  if (misc[1]) return;

  // ------------------------------------------------------------- selection
  uint32_t* q_i8 = reinterpret_cast<uint32_t*>(gbase + OFF_A);
  uint32_t* k_i8 = q_i8 + 128 * FP4_ROW_WORDS;
  float* q_sc = reinterpret_cast<float*>(k_i8 + 128 * FP4_ROW_WORDS);
  float* k_sc = q_sc + 128 * 8;
  int32_t* cand_ids = reinterpret_cast<int32_t*>(gbase + OFF_B);
  int* cand_ex = reinterpret_cast<int*>(cand_ids + C_MAX);
  float* cand_apx = reinterpret_cast<float*>(cand_ex + C_MAX);     // approximate tile scores of the candidates
  int* near_s = reinterpret_cast<int*>(cand_apx + C_MAX);          // candidate needs its exact score
  const int C = p.cand;

  int32_t* out = p.ids + (static_cast<long long>(bh) * qt + qtile) * p.topk;

  fp4_stage_rows(q_i8, q_sc, p.qp + (q_row0 * p.hidx + h) * 64, static_cast<long long>(p.hidx) * 64,
                 p.qs + (q_row0 * p.hidx + h) * 8, static_cast<long long>(p.hidx) * 8, 0.25f);
  if (threadIdx.x == 0) { misc[2] = 0; misc[3] = 0; misc[4] = 0; misc[5] = __float_as_int(-INFINITY); }
  for (int c = threadIdx.x; c < C_MAX; c += NUM_THREADS) cand_ex[c] = static_cast<int>(0x80000000u);
  __syncthreads();
  if (threadIdx.x < 128) {                 // L1 norm and squared L2 norm of one dequantised query row
    float l1 = 0.f, l2 = 0.f;
    for (int g = 0; g < 8; ++g) {
      int sum = 0, squares = 0;
      for (int w = 0; w < 4; ++w) {
        const uint32_t word = q_i8[threadIdx.x * FP4_ROW_WORDS + g * 4 + w];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int v = static_cast<int>(static_cast<int8_t>((word >> (8 * e)) & 0xFFu));
          sum += abs(v);
          squares += v * v;
        }
      }
      const float unit = 2.0f * q_sc[threadIdx.x * 8 + g];      // value of one integer step in this group
      l1 += static_cast<float>(sum) * unit;
      l2 += static_cast<float>(squares) * unit * unit;
    }
    atomicMax(const_cast<int*>(misc + 3), __float_as_int(l1 * 1.0001f));
    atomicMax(const_cast<int*>(misc + 4), __float_as_int(l2 * 1.0001f));
  }
  float thr = 0.f;
  if (warp == 0) {
    // C-th largest approximate score and the candidate set (ties at the threshold in index order)
    const unsigned* keys = reinterpret_cast<const unsigned*>(scores);
    const unsigned lt_mask = (1u << lane) - 1u;
    unsigned T = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned trial = T | (1u << bit);
      int cnt = 0;
      for (int j = lane; j < p.tiles; j += 32) cnt += ((keys[j] ^ 0x80000000u) >= trial) ? 1 : 0;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
      if (cnt >= C) T = trial;
    }
    int n_gt = 0;
    for (int j = lane; j < p.tiles; j += 32) n_gt += ((keys[j] ^ 0x80000000u) > T) ? 1 : 0;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) n_gt += __shfl_xor_sync(0xffffffffu, n_gt, d);
    const int need_eq = C - n_gt;
    int out_run = 0, eq_run = 0;
    for (int base_j = 0; base_j < p.tiles; base_j += 32) {
      const int j = base_j + lane;
      const unsigned u = j < p.tiles ? (keys[j] ^ 0x80000000u) : 0u;
      const bool is_gt = j < p.tiles && u > T;
      const bool is_eq = j < p.tiles && u == T;
      const unsigned eq_ballot = __ballot_sync(0xffffffffu, is_eq);
      const bool take = is_gt || (is_eq && eq_run + __popc(eq_ballot & lt_mask) < need_eq);
      const unsigned take_ballot = __ballot_sync(0xffffffffu, take);
      if (take) {
        const int pos = out_run + __popc(take_ballot & lt_mask);
        cand_ids[pos] = j;
        cand_apx[pos] = ord2f(static_cast<int>(u ^ 0x80000000u));
      }
      out_run += __popc(take_ballot);
      eq_run += __popc(eq_ballot);
    }
    thr = ord2f(static_cast<int>(T ^ 0x80000000u));
  }
  __syncthreads();
  // exact tile score of one page: max over the 128 x 128 dots, whole CTA
  auto exact_page = [&](int pg) -> float {
    const long long page = (static_cast<long long>(b) * p.tiles + pg) * p.hk + hk_idx;
    fp4_stage_rows(k_i8, k_sc, p.kp + page * 128 * 64, 64, p.ks + page * 128 * 8, 8, 1.0f);
    __syncthreads();
    float m = -INFINITY;
    if (threadIdx.x < 256) m = fp4_block_max_mma(q_i8, q_sc, k_i8, k_sc, warp, lane);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    return m;                              // per-warp maximum; lane 0 publishes it
  };
  // Approximate and exact tile score differ by at most delta (the sum of |q_d k_d| bounded by
  // Hoelder and by Cauchy-Schwarz), so candidates more than 2 delta apart are ordered by their
  // approximate scores for certain: only a candidate with another one within 2 delta is re-scored.
  const float delta = EPS * fminf(__int_as_float(misc[3]) * p.k_absmax[0],
                                  sqrtf(__int_as_float(misc[4])) * sqrtf(p.k_absmax[2] * 1.0001f));
  const float two = 2.f * delta;
  for (int c = threadIdx.x; c < C; c += NUM_THREADS) {
    const float a = cand_apx[c];
    int near = 0;
#pragma unroll 4
    for (int j = 0; j < C; ++j) near |= static_cast<int>(j != c) & static_cast<int>(!(fabsf(a - cand_apx[j]) > two));
    near_s[c] = near;
  }
  __syncthreads();
  for (int c = 0; c < C; ++c) {
    if (!near_s[c]) continue;
    const float m = exact_page(cand_ids[c]);
    if (lane == 0) atomicMax(&cand_ex[c], f2ord(m));
    __syncthreads();
  }
  // rank of a candidate = number of candidates that beat it in (exact score descending, page
  // ascending): by the approximate scores when more than 2 delta apart, else by the exact ones
  for (int c = threadIdx.x; c < C; c += NUM_THREADS) {
    const float a = cand_apx[c], e = ord2f(cand_ex[c]);
    const int id = cand_ids[c];
    int rank = 0;
#pragma unroll 4
    for (int j = 0; j < C; ++j) {
      const float d = cand_apx[j] - a, ej = ord2f(cand_ex[j]);
      const int gt = static_cast<int>(d > two), lt = static_cast<int>(d < -two);
      const int exact = static_cast<int>(ej > e) | (static_cast<int>(ej == e) & static_cast<int>(cand_ids[j] < id));
      rank += gt | (((gt | lt) ^ 1) & exact);
    }
    if (rank < p.topk) out[rank] = id;
    if (rank == p.topk - 1) misc[5] = __float_as_int(near_s[c] ? e : a - delta);   // lower bound of the k-th exact score
  }
  __syncthreads();
  if (threadIdx.x == 0) misc[2] = ((C >= p.tiles) || (__int_as_float(misc[5]) > thr + delta)) ? 0 : 1;
  __syncthreads();
  if (misc[2]) {
    float* row = reinterpret_cast<float*>(scores);
    for (int pg = 0; pg < p.tiles; ++pg) {
      const float m = exact_page(pg);
      if (lane == 0) scratch_f[warp] = m;
      __syncthreads();
      if (threadIdx.x == 0) {
        float mm = scratch_f[0];
        for (int w = 1; w < NUM_THREADS / 32; ++w) mm = fmaxf(mm, scratch_f[w]);
        row[pg] = mm;
      }
      __syncthreads();
    }
    block_topk(row, p.tiles, p.topk, out, scratch_f, scratch_i);
    if (threadIdx.x == 0 && p.fallbacks) atomicAdd(p.fallbacks, 1);
  }
}


// ---------------------------------------------------------------- exact tile scores by pruning
// The exact score of a (query tile, key page) pair is the maximum of 128 x 128 exact dots. The
// tensor cores give every dot within delta of its exact value, so only the elements whose
// approximate value reaches (largest approximate value - 2 delta) can hold the exact maximum:
// any other element is below the exact value of the approximate arg-max. Those few elements
// (usually one) are evaluated with the canonical arithmetic (integer group sums, scaled and
// added in group order) straight from the codes in global memory. Same scores, bit for bit,
// as fp4_score_mma_kernel, which evaluates all 16384 elements of a pair exactly.
struct PruneParams {
  const uint8_t *qp, *qs, *kp, *ks;   // public NVFP4 layout (codes, e4m3 scales)
  const float* k_stats;               // [0] max |dequantised key element|, [2] largest squared L2 norm of a key
  float* tile_scores;                 // [B, Hidx, Qt, tiles]
  int* status;
  int batch, hidx, hk, len_q, tiles, pages_per_cta, chunks;
};

// Integer dot of one 16-element scale group straight from the e2m1 codes (two words per row):
// magnitudes 2 |value| through a byte-permute table, the sign of each product from the xor of
// the code sign bits, products of either sign summed apart with dp4a.
__device__ __forceinline__ int fp4_group_sum(uint32_t q0, uint32_t q1, uint32_t k0, uint32_t k1) {
  constexpr uint32_t LUT_LO = 0x03020100u, LUT_HI = 0x0C080604u;      // 2 |value| of codes 0..7
  int pos = 0, neg = 0;
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const uint32_t wq = w ? q1 : q0, wk = w ? k1 : k0;
    const uint32_t sg = ((wq ^ wk) >> 3) & 0x11111111u;               // 1 where the product is negative
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const uint32_t mq = __byte_perm(LUT_LO, LUT_HI, (wq >> (16 * hh)) & 0x7777u);
      const uint32_t mk = __byte_perm(LUT_LO, LUT_HI, (wk >> (16 * hh)) & 0x7777u);
      const uint32_t ng = __byte_perm(0x0000FF00u, 0u, (sg >> (16 * hh)) & 0x1111u);
      pos = __dp4a(static_cast<int>(mq & ~ng), static_cast<int>(mk), pos);
      neg = __dp4a(static_cast<int>(mq & ng), static_cast<int>(mk), neg);
    }
  }
  return pos - neg;
}

// canonical dot of a query row and a key row (16 code words and 8 e4m3 scales each); everything
// is requested from memory before the first use
__device__ __forceinline__ float fp4_exact_dot(const uint8_t* __restrict__ q_codes, const uint8_t* __restrict__ q_scales,
                                               const uint8_t* __restrict__ k_codes, const uint8_t* __restrict__ k_scales) {
  uint4 qw[4], kw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    qw[i] = __ldg(reinterpret_cast<const uint4*>(q_codes) + i);
    kw[i] = __ldg(reinterpret_cast<const uint4*>(k_codes) + i);
  }
  const uint2 qs8 = __ldg(reinterpret_cast<const uint2*>(q_scales));
  const uint2 ks8 = __ldg(reinterpret_cast<const uint2*>(k_scales));
  const uint32_t* q32 = reinterpret_cast<const uint32_t*>(qw);
  const uint32_t* k32 = reinterpret_cast<const uint32_t*>(kw);
  float acc = 0.f;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const int sum = fp4_group_sum(q32[2 * g], q32[2 * g + 1], k32[2 * g], k32[2 * g + 1]);
    const uint8_t qb = static_cast<uint8_t>(((g < 4 ? qs8.x : qs8.y) >> (8 * (g & 3))) & 0xFFu);
    const uint8_t kb = static_cast<uint8_t>(((g < 4 ? ks8.x : ks8.y) >> (8 * (g & 3))) & 0xFFu);
    const float c = (0.25f * e4m3_to_float(qb)) * e4m3_to_float(kb);
    acc = fmaf(static_cast<float>(sum), c, acc);
  }
  return acc;
}

constexpr int PR_QCAP = 2048;                // queued elements per CTA
constexpr int PR_OFF_AUX = OFF_SCORES;       // barriers (128 bytes), misc (128 bytes)
constexpr int PR_OFF_QUEUE = PR_OFF_AUX + 256;            // [PR_QCAP] elements waiting for their exact value
constexpr int PR_OFF_RES = PR_OFF_QUEUE + PR_QCAP * 4;     // [pages per CTA] exact maxima as ordered ints

// One CTA per (batch, index head, query tile, chunk of key pages), two CTAs per SM. Warps 0-7 epilogue (lane
// quarter = warp & 3, column half = warp >> 2), warp 8 TMA, warp 9 MMA issue. The epilogue
// warps meet twice per page at a named barrier (largest approximate value of the page, then
// largest exact value of the surviving elements); a warp whose bounded wait gave up keeps
// taking part in those meetings, so nobody is left waiting for it.
__global__ void __launch_bounds__(NUM_THREADS, 2)
fp4_prune_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                 const PruneParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw);
  unsigned char* aux = gbase + PR_OFF_AUX;
  const uint32_t bar0 = base + PR_OFF_AUX;
  // tmem base, abort flag, L1 bits, squared L2 bits, largest approximate value of a page [3 slots], queue length
  volatile int* misc = reinterpret_cast<volatile int*>(aux + 128);
  int* queue = reinterpret_cast<int*>(gbase + PR_OFF_QUEUE);
  int* res = reinterpret_cast<int*>(gbase + PR_OFF_RES);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  enum { A_FULL = 0, A_EMPTY = A_STAGES, B_FULL = 2 * A_STAGES, ACC_FULL = 2 * A_STAGES + 1, ACC_EMPTY = 2 * A_STAGES + 3 };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = p.len_q >> 7;
  const int chunk = blockIdx.x % p.chunks;
  const int list = blockIdx.x / p.chunks;            // (batch * Hidx + head) * Qt + query tile
  const int qtile = list % qt;
  const int bh = list / qt;
  const int h = bh % p.hidx, b = bh / p.hidx;
  const int hk_idx = p.hk > 1 ? h : 0;
  const long long q_row0 = static_cast<long long>(b) * p.len_q + static_cast<long long>(qtile) * 128;
  const int page0 = chunk * p.pages_per_cta;
  const int num_tiles = min(p.pages_per_cta, p.tiles - page0);
  Guard guard{misc + 1, p.status};

  if (threadIdx.x == 0) {
    misc[1] = 0;
    misc[2] = 0;
    misc[3] = 0;
    for (int i = 4; i < 7; ++i) misc[i] = INT_MIN;
    misc[7] = 0;
    for (int i = 0; i < A_STAGES; ++i) {
      mbar_init(bar(A_FULL + i), 1);
      mbar_init(bar(A_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(ACC_FULL + i), 1);
      mbar_init(bar(ACC_EMPTY + i), 8);
    }
    mbar_init(bar(B_FULL), 1);
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), 256);
    tmem_relinquish();
  }
  for (int t = threadIdx.x; t < num_tiles; t += NUM_THREADS) res[t] = INT_MIN;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = static_cast<uint32_t>(misc[0]);

  if (warp == TMA_WARP) {
    if (lane == 0) {
      mbar_expect_tx(bar(B_FULL), TILE_BYTES);
      tma_load_3d(base + OFF_B, &q_map, 0, h, static_cast<int>(q_row0), bar(B_FULL));
      tma_load_3d(base + OFF_B + PANEL_BYTES, &q_map, 64, h, static_cast<int>(q_row0), bar(B_FULL));
    }
    bool ok = true;
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int s = t % A_STAGES, use = t / A_STAGES;
      if (use > 0) {
        bool w = mbar_wait(bar(A_EMPTY + s), (use - 1) & 1, guard, 0x580 + s);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
      }
      if (lane == 0) {
        const uint32_t dst = base + OFF_A + s * TILE_BYTES;
        const int row = ((b * p.tiles + page0 + t) * p.hk + hk_idx) * 128;
        mbar_expect_tx(bar(A_FULL + s), TILE_BYTES);
        tma_load_2d(dst, &k_map, 0, row, bar(A_FULL + s));
        tma_load_2d(dst + PANEL_BYTES, &k_map, 64, row, bar(A_FULL + s));
      }
    }
    if (!ok)
      for (int t = max(0, num_tiles - A_STAGES); t < num_tiles; ++t)
        mbar_wait_drain(bar(A_FULL + t % A_STAGES), (t / A_STAGES) & 1);
  } else if (warp == MMA_WARP) {
    const uint32_t idesc = idesc_bf16(128, 128, false);
    bool ok = true;
    {
      bool w = mbar_wait(bar(B_FULL), 0, guard, 0x590);
      ok = __all_sync(0xffffffffu, w);
      tc_fence_after();
    }
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int s = t % A_STAGES, acc = t & 1;
      bool w = mbar_wait(bar(A_FULL + s), (t / A_STAGES) & 1, guard, 0x5a0 + s);
      if (w && t >= 2) w = mbar_wait(bar(ACC_EMPTY + acc), ((t >> 1) - 1) & 1, guard, 0x5b0 + acc);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint64_t a0 = desc_sw128_kmajor(base + OFF_A + s * TILE_BYTES);
        const uint64_t b0 = desc_sw128_kmajor(base + OFF_B);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t step = static_cast<uint64_t>((kk >> 2) * (PANEL_BYTES >> 4) + (kk & 3) * 2);
          mma_ss(tmem + acc * 128, a0 + step, b0 + step, idesc, kk > 0);
        }
        tc_commit(bar(A_EMPTY + s));
        tc_commit(bar(ACC_FULL + acc));
      }
    }
  } else {
    // epilogue: thread = key row of the page, this warp's 64-column half of the query tile
    auto meet = [&]() { asm volatile("bar.sync 1, 256;" ::: "memory"); };
    if (threadIdx.x < 128) {
      // L1 norm and squared L2 norm of one dequantised query row, from the operand tile the TMA
      // warp fetched (a row = 128 bytes in each of the two panels; the swizzle only permutes
      // 16-byte pieces inside them, and the lanes start at different pieces to spare the banks)
      float l1 = 0.f, l2 = 0.f;
      if (mbar_wait(bar(B_FULL), 0, guard, 0x5d0)) {
#pragma unroll
        for (int panel = 0; panel < 2; ++panel) {
          const uint4* row = reinterpret_cast<const uint4*>(gbase + OFF_B + panel * PANEL_BYTES + threadIdx.x * 128);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 piece = row[(c + lane) & 7];
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&piece);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(hh[e]);
              l1 += fabsf(f.x) + fabsf(f.y);
              l2 = fmaf(f.x, f.x, l2);
              l2 = fmaf(f.y, f.y, l2);
            }
          }
        }
      }
      atomicMax(const_cast<int*>(misc + 2), __float_as_int(l1 * 1.0001f));
      atomicMax(const_cast<int*>(misc + 3), __float_as_int(l2 * 1.0001f));
    }
    meet();
    const float delta = EPS * fminf(__int_as_float(misc[2]) * p.k_stats[0],
                                    sqrtf(__int_as_float(misc[3])) * sqrtf(p.k_stats[2] * 1.0001f));
    const float two = 2.f * delta;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int half = warp >> 2;
    const int key_row = (warp & 3) * 32 + lane;
    // exact value of element (page t of this CTA, key row, query column) into the page's maximum
    auto evaluate = [&](int t, int krow, int col) {
      const long long page = (static_cast<long long>(b) * p.tiles + page0 + t) * p.hk + hk_idx;
      const long long qrow = (q_row0 + col) * p.hidx + h;
      const float e = fp4_exact_dot(p.qp + qrow * 64, p.qs + qrow * 8, p.kp + (page * 128 + krow) * 64,
                                    p.ks + (page * 128 + krow) * 8);
      if (e == e) atomicMax(res + t, f2ord(e));
    };
    bool ok = true;
    for (int t = 0; t < num_tiles; ++t) {
      const int acc = t & 1, slot = 4 + t % 3;
      if (ok) {
        bool w = mbar_wait(bar(ACC_FULL + acc), (t >> 1) & 1, guard, 0x5c0 + acc);
        ok = __all_sync(0xffffffffu, w);
      }
      uint32_t v[4][16];
      float mine = -INFINITY;
      if (ok) {
        tc_fence_after();
        const uint32_t t_acc = tmem + lane_base + acc * 128 + half * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld16(t_acc + c * 16, v[c]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(ACC_EMPTY + acc));
        float m4[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float m5[5];
#pragma unroll
          for (int j = 0; j < 5; ++j)
            m5[j] = max3(__uint_as_float(v[c][3 * j]), __uint_as_float(v[c][3 * j + 1]), __uint_as_float(v[c][3 * j + 2]));
          m4[c] = fmaxf(max3(m5[0], m5[1], m5[2]), max3(m5[3], m5[4], __uint_as_float(v[c][15])));
        }
        mine = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        float m = mine;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        if (lane == 0) atomicMax(const_cast<int*>(misc + slot), f2ord(m));
      }
      meet();
      // the slot of the page before is free now (everyone read it before this meeting); it is
      // next written for page t + 2, after the meeting of page t + 1
      if (threadIdx.x == 0 && t > 0) misc[4 + (t - 1) % 3] = INT_MIN;
      if (ok) {
        const float thr = ord2f(misc[slot]) - two;
        if (!(mine < thr)) {                 // this key row holds at least one element that may be the maximum
          unsigned long long mask = 0ull;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (!(__uint_as_float(v[c][j]) < thr)) mask |= 1ull << (c * 16 + j);
          while (mask) {
            const int col = half * 64 + __ffsll(static_cast<long long>(mask)) - 1;
            mask &= mask - 1;
            const int at = atomicAdd(const_cast<int*>(misc + 7), 1);
            if (at < PR_QCAP) queue[at] = (t << 14) | (key_row << 7) | col;
            else evaluate(t, key_row, col);  // queue full (masses of ties): pay for it here
          }
        }
      }
    }
    meet();
    // the queued elements, one per thread at a time, then the scores of this CTA's pages
    const int queued = min(misc[7], PR_QCAP);
    for (int i = threadIdx.x; i < queued; i += 256) {
      const int e = queue[i];
      evaluate(e >> 14, (e >> 7) & 127, e & 127);
    }
    meet();
    if (ok)
      for (int t = threadIdx.x; t < num_tiles; t += 256)
        p.tile_scores[static_cast<long long>(list) * p.tiles + page0 + t] = ord2f(res[t]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace ftc

// Returns SB_OK when the tensor-core path ran, 1 when the problem is not eligible.
// q_deq / k_deq: bf16 workspaces of B*Sq*Hidx*128 and (B*Skv/128)*Hk*128*128 elements;
// aux: one float (key abs-max) + one int (fallback counter) + one float (largest squared key norm).
int launch_fp4_indexer_tc(const void* qp, const void* qs, const void* kp, const void* ks, void* q_deq, void* k_deq,
                          void* aux, int32_t* ids, int batch, int hidx, int hk, int len_q, int len_kv, int topk,
                          cudaStream_t stream) {
  using namespace ftc;
  const int tiles = len_kv / 128, qt = len_q / 128;
  const int extra = topk / 4 > 16 ? topk / 4 : 16;
  int cand = topk + extra;
  if (cand > tiles) cand = tiles;
  if (cand > C_MAX || tiles > MAX_TILES) return 1;
  // Every candidate is re-scored exactly by one CTA per list, while the exact scorer (integer
  // group sums on the tensor cores) spreads pages over the whole GPU: the pre-filter pays off
  // only when candidates are a small share of the pages (measured with top-16: slower than
  // the exact scorer at 32, 64 and 128 pages; 8x faster at 1024 pages, top-32).
  if (8 * cand > tiles) return 1;
  const long long q_rows = static_cast<long long>(batch) * len_q * hidx;
  const long long k_rows = static_cast<long long>(batch) * tiles * hk * 128;
  if (q_rows >= (1LL << 31) || k_rows >= (1LL << 31)) return 1;
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  if (cudaMemsetAsync(aux, 0, 12, stream) != cudaSuccess) return set_error(SB_ERR_CUDA, "memset failed");
  dequant_kernel<<<static_cast<unsigned>(((q_rows + k_rows) * 16 + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(qp), static_cast<const uint8_t*>(qs), static_cast<__nv_bfloat16*>(q_deq), q_rows,
      static_cast<const uint8_t*>(kp), static_cast<const uint8_t*>(ks), static_cast<__nv_bfloat16*>(k_deq), k_rows,
      static_cast<float*>(aux));
  CUtensorMap qm, km;
  {
    const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(hidx), static_cast<cuuint64_t>(batch) * len_q};
    const cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(hidx) * 256};
    const cuuint32_t box[3] = {64, 1, 128};
    const cuuint32_t steps[3] = {1, 1, 1};
    if (encode_tiled(&qm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, q_deq, dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the dequantised queries");
  }
  {
    const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(k_rows)};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t steps[2] = {1, 1};
    if (encode_tiled(&km, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_deq, dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the dequantised keys");
  }
  Params p{};
  p.qp = static_cast<const uint8_t*>(qp); p.qs = static_cast<const uint8_t*>(qs);
  p.kp = static_cast<const uint8_t*>(kp); p.ks = static_cast<const uint8_t*>(ks);
  p.k_absmax = static_cast<const float*>(aux);
  p.fallbacks = reinterpret_cast<int*>(aux) + 1;
  p.ids = ids;
  p.status = ctx->status;
  p.batch = batch; p.hidx = hidx; p.hk = hk; p.len_q = len_q; p.tiles = tiles; p.topk = topk; p.cand = cand;
  const size_t smem = OFF_SCORES + ((static_cast<size_t>(tiles) * 4 + 15) & ~static_cast<size_t>(15)) + 320 + 1024;
  if (!(ctx->tc_attr & (1 << 8))) {
    cudaError_t e = cudaFuncSetAttribute(fp4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fp4_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->tc_attr |= (1 << 8);
  }
  fp4_tc_kernel<<<batch * hidx * qt, NUM_THREADS, smem, stream>>>(qm, km, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

// Exact tile scores [B, Hidx, Qt, tiles] through fp4_prune_kernel. Returns SB_OK, or 1 when the
// problem is not eligible (the caller then runs the exact mma.sync scorer). Workspaces as for
// launch_fp4_indexer_tc; aux: [0] key abs-max, [1] untouched counter, [2] largest squared key norm.
int launch_fp4_scores_prune(const void* qp, const void* qs, const void* kp, const void* ks, void* q_deq, void* k_deq,
                            void* aux, float* tile_scores, int batch, int hidx, int hk, int len_q, int len_kv,
                            cudaStream_t stream) {
  using namespace ftc;
  const int tiles = len_kv / 128, qt = len_q / 128;
  const long long q_rows = static_cast<long long>(batch) * len_q * hidx;
  const long long k_rows = static_cast<long long>(batch) * tiles * hk * 128;
  const long long lists = static_cast<long long>(batch) * hidx * qt;
  if (q_rows >= (1LL << 31) || k_rows >= (1LL << 31) || lists * tiles >= (1LL << 31)) return 1;
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  if (cudaMemsetAsync(aux, 0, 12, stream) != cudaSuccess) return set_error(SB_ERR_CUDA, "memset failed");
  dequant_kernel<<<static_cast<unsigned>(((q_rows + k_rows) * 16 + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(qp), static_cast<const uint8_t*>(qs), static_cast<__nv_bfloat16*>(q_deq), q_rows,
      static_cast<const uint8_t*>(kp), static_cast<const uint8_t*>(ks), static_cast<__nv_bfloat16*>(k_deq), k_rows,
      static_cast<float*>(aux));
  CUtensorMap qm, km;
  {
    const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(hidx), static_cast<cuuint64_t>(batch) * len_q};
    const cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(hidx) * 256};
    const cuuint32_t box[3] = {64, 1, 128};
    const cuuint32_t steps[3] = {1, 1, 1};
    if (encode_tiled(&qm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, q_deq, dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the dequantised queries");
  }
  {
    const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(k_rows)};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t steps[2] = {1, 1};
    if (encode_tiled(&km, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_deq, dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the dequantised keys");
  }
  PruneParams p{};
  p.qp = static_cast<const uint8_t*>(qp); p.qs = static_cast<const uint8_t*>(qs);
  p.kp = static_cast<const uint8_t*>(kp); p.ks = static_cast<const uint8_t*>(ks);
  p.k_stats = static_cast<const float*>(aux);
  p.tile_scores = tile_scores;
  p.status = ctx->status;
  p.batch = batch; p.hidx = hidx; p.hk = hk; p.len_q = len_q; p.tiles = tiles;
  // Two CTAs fit an SM (about 106 KiB of shared memory, 96 registers, 256 TMEM columns each):
  // while one waits for its accumulator the other uses the tensor pipe. As many CTAs as fit
  // at once when the lists are few; a CTA keeps its query tile and takes a run of pages.
  long long chunks = (2LL * ctx->sm_count) / lists;
  if (chunks > tiles) chunks = tiles;
  if (chunks < 1) chunks = 1;
  p.pages_per_cta = static_cast<int>((tiles + chunks - 1) / chunks);
  p.chunks = (tiles + p.pages_per_cta - 1) / p.pages_per_cta;
  if (lists * p.chunks >= (1LL << 31)) return 1;
  if (!(ctx->tc_attr & (1 << 11))) {
    cudaError_t e = cudaFuncSetAttribute(fp4_prune_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fp4_prune_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->tc_attr |= (1 << 11);
  }
  const size_t smem = PR_OFF_RES + static_cast<size_t>(p.pages_per_cta) * 4 + 1024;
  fp4_prune_kernel<<<static_cast<unsigned>(lists * p.chunks), NUM_THREADS, smem, stream>>>(qm, km, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
