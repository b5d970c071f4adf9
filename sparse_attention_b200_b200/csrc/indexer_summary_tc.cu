// Tensor-core path of the R1 / R4 summary indexer: same block ids as the exact
// kernel of indexer_summary.cu, bit for bit, at tensor-core speed.
//
// An fp32-accumulating MMA does not reproduce the fixed summation order that
// defines a score, so the tensor cores only PRE-FILTER:
//   1. approximate scores of every KV block (tcgen05 MMA, key descriptors as the
//      M operand streamed by TMA, the query descriptors of QB query blocks as the
//      N operand, max over the group's rows and the R key representatives in the
//      epilogue) stay in shared memory;
//   2. per query block the C = k + extra best approximate blocks become
//      candidates and are re-scored with the exact arithmetic (fp32 FMAs in
//      feature order);
//   3. the exact top-k of the candidates is the answer if it is provably safe:
//      exact k-th score > C-th approximate score + delta, where delta bounds
//      |approximate - exact| for every block of the list
//      (delta = 2^-14 * max_m ||q_m||_1 * max|k element| * 128^-0.5, an order of
//      magnitude above the worst case of two 128-term fp32 sums);
//   4. otherwise (near ties, e.g. constant inputs) the list falls back to exact
//      scores of all blocks.
// Replaces descriptor_dot + reduce_topk (indexers/r1_r4/gpu_ops.py:19-49).
#include "ptx.cuh"
#include "internal.h"
#include "topk.cuh"
#include <cuda_bf16.h>

namespace sb {
namespace stc {

constexpr int TILE_BYTES = 128 * 256;      // 128 descriptors x 128 bf16
constexpr int PANEL_BYTES = 128 * 128;
#ifndef SB_STC_STAGES
#define SB_STC_STAGES 2
#endif
constexpr int A_STAGES = SB_STC_STAGES;
constexpr int SCORE_LIMIT = 232448 - 2048 - (A_STAGES + 1) * TILE_BYTES;   // bytes of shared memory left for scores
constexpr int C_MAX = 192;                 // candidates per list
constexpr int NUM_THREADS = 256;
constexpr int TMA_WARP = 4, MMA_WARP = 5;
constexpr float EPS = 6.103515625e-05f;    // 2^-14
constexpr float SCALE = 0.08838834764831845f;

constexpr int OFF_A = 0;
constexpr int OFF_B = A_STAGES * TILE_BYTES;
constexpr int OFF_SCORES = OFF_B + TILE_BYTES;
// after the scores: barriers, candidate arrays, scratch (offsets computed at run time)

struct Params {
  const __nv_bfloat16* qd;     // [B, Hq, qt, R, 128]
  const __nv_bfloat16* kd;     // [B, Hkv, nt, R, 128]
  const float* k_absmax;       // [B * Hkv] max |element| of the key descriptors of a head
  int32_t* ids;                // [B, Hkv, qt, topk]
  int* status;
  int* fallbacks;              // optional counter of lists that took the exact fallback
  int hq, hkv, qt, nt, r, topk, qb, cand;
  int q_chunks;                // ceil(qt / qb)
};

// monotone float <-> int mapping so shared-memory atomicMax works on scores
__device__ __forceinline__ int f2ord(float f) {
  const int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
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

// Exact score contribution of one key descriptor: max over the MP query rows of
// the fp32 dot product accumulated in feature order (q_s is [128][MP] fp32).
template <int MP>
__device__ __forceinline__ float exact_key_best(const float* q_s, const __nv_bfloat16* krow_g) {
  float acc[MP];
#pragma unroll
  for (int m = 0; m < MP; ++m) acc[m] = 0.f;
  const uint4* krow = reinterpret_cast<const uint4*>(krow_g);
#pragma unroll 2
  for (int c = 0; c < 16; ++c) {
    const uint4 kv = __ldg(krow + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&kv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 kf = __bfloat1622float2(h[e]);
      const float* q0 = q_s + (c * 8 + 2 * e) * MP;
#pragma unroll
      for (int m = 0; m < MP; ++m) acc[m] = fmaf(q0[m], kf.x, acc[m]);
#pragma unroll
      for (int m = 0; m < MP; ++m) acc[m] = fmaf(q0[MP + m], kf.y, acc[m]);
    }
  }
  float best = acc[0];
#pragma unroll
  for (int m = 1; m < MP; ++m) best = fmaxf(best, acc[m]);
  return best;
}

// One CTA: QB query blocks of one (batch, KV head) against every KV block.
// Warps 0-3 epilogue (TMEM lane quarters), warp 4 TMA, warp 5 MMA issue; all
// eight warps take part in the selection phase.
template <int GR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
score_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map, const Params p) {
  constexpr int MP = GR < 4 ? 4 : GR;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw);
  int* scores = reinterpret_cast<int*>(gbase + OFF_SCORES);
  const int score_bytes = (p.qb * p.nt * 4 + 15) & ~15;
  unsigned char* aux = gbase + OFF_SCORES + score_bytes;
  const uint32_t bar0 = base + OFF_SCORES + score_bytes;        // 9 barriers, 128 bytes reserved
  volatile int* misc = reinterpret_cast<volatile int*>(aux + 128);   // tmem base, abort, unsafe, l1q
  volatile int* flags = reinterpret_cast<volatile int*>(aux + 144);   // [128] list needs the exact fallback
  float* scratch_f = reinterpret_cast<float*>(aux + 144 + 128 * 4);
  int* scratch_i = reinterpret_cast<int*>(scratch_f + 10);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  enum { A_FULL = 0, A_EMPTY = A_STAGES, B_FULL = 2 * A_STAGES, ACC_FULL = 2 * A_STAGES + 1, ACC_EMPTY = 2 * A_STAGES + 3 };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.hq / p.hkv;
  const int chunk = blockIdx.x % p.q_chunks;
  const int bk = blockIdx.x / p.q_chunks;              // batch * Hkv + kv head
  const int b = bk / p.hkv, kvh = bk - b * p.hkv;
  const int qtile0 = chunk * p.qb;
  const int n_keys = p.nt * p.r;
  const int num_tiles = (n_keys + 127) >> 7;
  const int n_cols = p.qb * GR;                         // MMA N
  // CTAs of one head walk the key tiles from different starting points, so they do
  // not all ask the L2 for the same tile at the same moment (a max is order-free).
  const int rot = static_cast<int>((static_cast<unsigned>(chunk) * 37u) % static_cast<unsigned>(num_tiles));
  Guard guard{misc + 1, p.status};

  if (threadIdx.x == 0) {
    misc[1] = 0;
    for (int i = 0; i < A_STAGES; ++i) {
      mbar_init(bar(A_FULL + i), 1);
      mbar_init(bar(A_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(ACC_FULL + i), 1);
      mbar_init(bar(ACC_EMPTY + i), 4);
    }
    mbar_init(bar(B_FULL), 1);
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), 256);
    tmem_relinquish();
  }
  for (int j = threadIdx.x; j < p.qb * p.nt; j += NUM_THREADS) scores[j] = static_cast<int>(0x80000000u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = static_cast<uint32_t>(misc[0]);

  if (warp == TMA_WARP) {
    if (lane == 0) {
      const int rows = p.qb * GR;
      mbar_expect_tx(bar(B_FULL), rows * 256);
      tma_load_4d(base + OFF_B, &q_map, 0, 0, b * p.hq + kvh * group, qtile0, bar(B_FULL));
      tma_load_4d(base + OFF_B + PANEL_BYTES, &q_map, 64, 0, b * p.hq + kvh * group, qtile0, bar(B_FULL));
    }
    bool ok = true;
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int s = t % A_STAGES, use = t / A_STAGES;
      if (use > 0) {
        bool w = mbar_wait(bar(A_EMPTY + s), (use - 1) & 1, guard, 0x400 + s);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
      }
      if (lane == 0) {
        const uint32_t dst = base + OFF_A + s * TILE_BYTES;
        const int row = bk * n_keys + ((t + rot) % num_tiles) * 128;
        mbar_expect_tx(bar(A_FULL + s), TILE_BYTES);
        tma_load_2d(dst, &k_map, 0, row, bar(A_FULL + s));
        tma_load_2d(dst + PANEL_BYTES, &k_map, 64, row, bar(A_FULL + s));
      }
    }
    if (!ok)
      for (int t = max(0, num_tiles - A_STAGES); t < num_tiles; ++t)
        mbar_wait_drain(bar(A_FULL + t % A_STAGES), (t / A_STAGES) & 1);
  } else if (warp == MMA_WARP) {
    const uint32_t idesc = idesc_bf16(128, n_cols, false);
    bool ok = true;
    {
      bool w = mbar_wait(bar(B_FULL), 0, guard, 0x410);
      ok = __all_sync(0xffffffffu, w);
      tc_fence_after();
    }
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int s = t % A_STAGES, acc = t & 1;
      bool w = mbar_wait(bar(A_FULL + s), (t / A_STAGES) & 1, guard, 0x420 + s);
      if (w && t >= 2) w = mbar_wait(bar(ACC_EMPTY + acc), ((t >> 1) - 1) & 1, guard, 0x430 + acc);
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
  } else if (warp < 4) {
    // epilogue: thread = key descriptor row of the tile
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int r_log2 = 31 - __clz(p.r);                  // R is 1, 2 or 4
    const int n_chunks = n_cols >> 4;
    bool ok = true;
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int acc = t & 1;
      bool w = mbar_wait(bar(ACC_FULL + acc), (t >> 1) & 1, guard, 0x440 + acc);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      const int n = ((t + rot) % num_tiles) * 128 + warp * 32 + lane;
      const bool row_ok = n < n_keys;
      const int blk = n >> r_log2;
      const uint32_t t_acc = tmem + lane_base + acc * 128;
      // all columns into registers with one wait, then hand the accumulator back at once
      uint32_t v[8][16];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < n_chunks) tmem_ld16(t_acc + c * 16, v[c]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(ACC_EMPTY + acc));
      // Every (query block, KV block) pair is produced by exactly one lane group of one
      // tile, so a plain store suffices.
      auto flush = [&](int tl, float val) {
        for (int d = 1; d < p.r; d <<= 1) val = fmaxf(val, __shfl_xor_sync(0xffffffffu, val, d));
        if (row_ok && (lane & (p.r - 1)) == 0 && qtile0 + tl < p.qt) scores[tl * p.nt + blk] = f2ord(val);
      };
      float cur = -INFINITY;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < n_chunks) {
          if (GR >= 16) {
            float m5[5];
#pragma unroll
            for (int j = 0; j < 5; ++j)
              m5[j] = max3(__uint_as_float(v[c][3 * j]), __uint_as_float(v[c][3 * j + 1]), __uint_as_float(v[c][3 * j + 2]));
            const float m = fmaxf(max3(m5[0], m5[1], m5[2]), max3(m5[3], m5[4], __uint_as_float(v[c][15])));
            cur = fmaxf(cur, m);
            if ((((c + 1) * 16) % GR) == 0) {
              flush((c * 16) / GR, cur);
              cur = -INFINITY;
            }
          } else {
            constexpr int PER = GR >= 16 ? 1 : 16 / GR;
            constexpr int W = GR >= 16 ? 16 : GR;
#pragma unroll
            for (int sg = 0; sg < PER; ++sg) {
              float m = __uint_as_float(v[c][sg * W]);
#pragma unroll
              for (int j = 1; j < W; ++j) m = fmaxf(m, __uint_as_float(v[c][sg * W + j]));
              flush(c * PER + sg, m);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
  if (misc[1]) return;                       // a bounded wait gave up: status word is set

  // ------------------------------------------------------------- selection: one warp per list
  // The operand buffers are free now: per-warp fp32 query descriptors go to the A
  // stages, per-warp candidate arrays to the B tile.
  const __nv_bfloat16* kbase = p.kd + static_cast<long long>(bk) * n_keys * 128;
  const float kabs = p.k_absmax[bk];
  const int lists = min(p.qb, p.qt - qtile0);
  const int C = p.cand;
  {
    float* q_s = reinterpret_cast<float*>(gbase + OFF_A) + warp * 128 * MP;
    int32_t* cand_ids = reinterpret_cast<int32_t*>(gbase + OFF_B) + warp * 2 * C_MAX;
    float* cand_ex = reinterpret_cast<float*>(cand_ids + C_MAX);
    const unsigned lt_mask = (1u << lane) - 1u;
    for (int tl = warp; tl < lists; tl += NUM_THREADS / 32) {
      const int qtile = qtile0 + tl;
      const unsigned* keys = reinterpret_cast<const unsigned*>(scores + tl * p.nt);   // ordered ints
      // query descriptors of the list as fp32 [128][MP], and the largest L1 norm among them
      for (int m = 0; m < MP; ++m) {        // one descriptor row per step: 256 contiguous bytes
        const int mm = m < GR ? m : 0;
        const int g = mm / p.r, rq = mm - g * p.r;
        const long long qrow = ((static_cast<long long>(b) * p.hq + kvh * group + g) * p.qt + qtile) * p.r + rq;
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.qd + qrow * 128) + lane);
        const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        q_s[(4 * lane + 0) * MP + m] = f0.x;
        q_s[(4 * lane + 1) * MP + m] = f0.y;
        q_s[(4 * lane + 2) * MP + m] = f1.x;
        q_s[(4 * lane + 3) * MP + m] = f1.y;
      }
      __syncwarp();
      float l1 = 0.f;
      for (int m = lane; m < MP; m += 32) {
        float sum = 0.f;
        for (int d = 0; d < 128; ++d) sum += fabsf(q_s[d * MP + m]);
        l1 = fmaxf(l1, sum);
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) l1 = fmaxf(l1, __shfl_xor_sync(0xffffffffu, l1, d));
      const float delta = EPS * (l1 * 1.0001f) * kabs * SCALE;
      // C-th largest approximate score: bitwise search on the order-preserving keys
      unsigned T = 0;
      for (int bit = 31; bit >= 0; --bit) {
        const unsigned trial = T | (1u << bit);
        int cnt = 0;
        for (int j = lane; j < p.nt; j += 32) cnt += ((keys[j] ^ 0x80000000u) >= trial) ? 1 : 0;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
        if (cnt >= C) T = trial;
      }
      // candidates: everything above T, then ties at T in index order, C in total
      int n_gt = 0;
      for (int j = lane; j < p.nt; j += 32) n_gt += ((keys[j] ^ 0x80000000u) > T) ? 1 : 0;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) n_gt += __shfl_xor_sync(0xffffffffu, n_gt, d);
      const int need_eq = C - n_gt;
      int out_run = 0, eq_run = 0;
      for (int base_j = 0; base_j < p.nt; base_j += 32) {
        const int j = base_j + lane;
        const unsigned u = j < p.nt ? (keys[j] ^ 0x80000000u) : 0u;
        const bool is_gt = j < p.nt && u > T;
        const bool is_eq = j < p.nt && u == T;
        const unsigned eq_ballot = __ballot_sync(0xffffffffu, is_eq);
        const bool take = is_gt || (is_eq && eq_run + __popc(eq_ballot & lt_mask) < need_eq);
        const unsigned take_ballot = __ballot_sync(0xffffffffu, take);
        if (take) cand_ids[out_run + __popc(take_ballot & lt_mask)] = j;
        out_run += __popc(take_ballot);
        eq_run += __popc(eq_ballot);
      }
      __syncwarp();
      const float thr = ord2f(static_cast<int>(T ^ 0x80000000u)) * SCALE;
      // exact scores of the candidates (R adjacent lanes = the R key representatives of one block)
      for (int base_i = 0; base_i < C * p.r; base_i += 32) {
        const int item = base_i + lane;
        const bool valid = item < C * p.r;
        const int c = item / p.r, rk = item - c * p.r;
        const int blk = valid ? cand_ids[c] : 0;
        float best = valid ? exact_key_best<MP>(q_s, kbase + (static_cast<long long>(blk) * p.r + rk) * 128) : -INFINITY;
        for (int d = 1; d < p.r; d <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, d));
        if (valid && rk == 0) cand_ex[c] = best * SCALE;
      }
      __syncwarp();
      // exact top-k of the candidates by (score descending, block id ascending)
      constexpr int SLOTS = C_MAX / 32;
      float es[SLOTS];
      int ei[SLOTS];
#pragma unroll
      for (int sidx = 0; sidx < SLOTS; ++sidx) {
        const int c = lane + 32 * sidx;
        es[sidx] = c < C ? cand_ex[c] : -INFINITY;
        ei[sidx] = c < C ? cand_ids[c] : INT_MAX;
      }
      int32_t* out = p.ids + (static_cast<long long>(bk) * p.qt + qtile) * p.topk;
      float kth = -INFINITY;
      for (int rank = 0; rank < p.topk; ++rank) {
        float bs = es[0];
        int bi = ei[0];
#pragma unroll
        for (int sidx = 1; sidx < SLOTS; ++sidx)
          if (better(es[sidx], ei[sidx], bs, bi)) { bs = es[sidx]; bi = ei[sidx]; }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
          const float os = __shfl_xor_sync(0xffffffffu, bs, d);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
          if (better(os, oi, bs, bi)) { bs = os; bi = oi; }
        }
#pragma unroll
        for (int sidx = 0; sidx < SLOTS; ++sidx)
          if (ei[sidx] == bi) { es[sidx] = -INFINITY; ei[sidx] = INT_MAX; }
        if (lane == 0) out[rank] = bi;
        kth = bs;
      }
      const bool safe = (C >= p.nt) || (kth > thr + delta);
      if (lane == 0) flags[tl] = safe ? 0 : 1;
    }
  }
  __syncthreads();
  // Lists whose pre-filter could not be proven safe: exact scores of every block, whole CTA.
  for (int tl = 0; tl < lists; ++tl) {
    if (!flags[tl]) continue;
    const int qtile = qtile0 + tl;
    float* q_s = reinterpret_cast<float*>(gbase + OFF_A);
    float* row = reinterpret_cast<float*>(scores + tl * p.nt);
    __syncthreads();
    for (int e = threadIdx.x; e < 128 * MP; e += NUM_THREADS) {
      const int m = e % MP, d = e / MP;
      const int mm = m < GR ? m : 0;
      const int g = mm / p.r, rq = mm - g * p.r;
      const long long qrow = ((static_cast<long long>(b) * p.hq + kvh * group + g) * p.qt + qtile) * p.r + rq;
      q_s[d * MP + m] = __bfloat162float(p.qd[qrow * 128 + d]);
    }
    __syncthreads();
    for (int base_i = 0; base_i < n_keys; base_i += NUM_THREADS) {
      const int n = base_i + threadIdx.x;
      const bool valid = n < n_keys;
      float best = valid ? exact_key_best<MP>(q_s, kbase + static_cast<long long>(n) * 128) : -INFINITY;
      for (int d = 1; d < p.r; d <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, d));
      if (valid && (n % p.r) == 0) row[n / p.r] = best * SCALE;
    }
    __syncthreads();
    block_topk(row, p.nt, p.topk, p.ids + (static_cast<long long>(bk) * p.qt + qtile) * p.topk, scratch_f, scratch_i);
    if (threadIdx.x == 0 && p.fallbacks) atomicAdd(p.fallbacks, 1);
  }
}

// max |element| of the key descriptors of each (batch, KV head)
__global__ void __launch_bounds__(256) absmax_kernel(const __nv_bfloat16* __restrict__ kd, float* __restrict__ out,
                                                     long long per_head) {
  const int head = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(kd + static_cast<long long>(head) * per_head);
  const long long n16 = per_head / 8;
  float m = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = __ldg(src + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out + head), __float_as_int(m));
}

template <int GR>
static int launch_gr(const CUtensorMap& qm, const CUtensorMap& km, const Params& p, int grid, size_t smem,
                     DeviceCtx* ctx, int slot, cudaStream_t stream) {
  if (!(ctx->tc_attr & (1 << slot))) {
    cudaError_t e = cudaFuncSetAttribute(score_tc_kernel<GR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->tc_attr |= (1 << slot);
  }
  score_tc_kernel<GR><<<grid, NUM_THREADS, smem, stream>>>(qm, km, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace stc

// Returns SB_OK when the tensor-core path ran, 1 when the problem is not eligible
// (the caller then runs the exact kernel), negative on error.
// aux: device floats [B*Hkv] (key abs-max, filled here) + 1 int (fallback counter).
int launch_summary_select_tc(const void* qd, const void* kd, void* aux, int32_t* ids, int batch, int hq, int hkv,
                             int qt, int nt, int r, int topk, cudaStream_t stream) {
  using namespace stc;
  const int group = hq / hkv, gr = group * r;
  if (gr > 64 || (gr & (gr - 1)) != 0) return 1;
  const int extra = topk / 4 > 16 ? topk / 4 : 16;
  int cand = topk + extra;
  if (cand > nt) cand = nt;
  if (cand > C_MAX) return 1;
  int qb = 128 / gr;
  while (qb > 1 && qb * gr > 16 && (qb / 2) >= qt) qb >>= 1;        // do not cover far more query blocks than exist
  while (static_cast<long long>(qb) * nt * 4 > SCORE_LIMIT && qb * gr > 16) qb >>= 1;
  if (static_cast<long long>(qb) * nt * 4 > SCORE_LIMIT || qb * gr < 16) return 1;
  if (static_cast<long long>(batch) * hkv * nt * r >= (1LL << 31) || qb > 256 || r > 256 || group > 256) return 1;
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;

  CUtensorMap qm, km;
  {
    const cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(r), static_cast<cuuint64_t>(batch) * hq,
                                static_cast<cuuint64_t>(qt)};
    const cuuint64_t strides[3] = {256, static_cast<cuuint64_t>(qt) * r * 256, static_cast<cuuint64_t>(r) * 256};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(r), static_cast<cuuint32_t>(group),
                               static_cast<cuuint32_t>(qb)};
    const cuuint32_t steps[4] = {1, 1, 1, 1};
    if (encode_tiled(&qm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(qd), dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
      return 1;                                  // layout not expressible: use the exact kernel
  }
  {
    const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(batch) * hkv * nt * r};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t steps[2] = {1, 1};
    if (encode_tiled(&km, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kd), dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
      return 1;
  }
  float* absmax = static_cast<float*>(aux);
  int* fallbacks = reinterpret_cast<int*>(absmax + static_cast<size_t>(batch) * hkv);
  if (cudaMemsetAsync(aux, 0, (static_cast<size_t>(batch) * hkv + 1) * 4, stream) != cudaSuccess)
    return set_error(SB_ERR_CUDA, "memset failed");
  const long long per_head = static_cast<long long>(nt) * r * 128;
  int chunks = static_cast<int>((per_head / 8 + 256 * 8 - 1) / (256 * 8));
  if (chunks > 64) chunks = 64;
  if (chunks < 1) chunks = 1;
  absmax_kernel<<<dim3(chunks, batch * hkv), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(kd), absmax, per_head);

  Params p{};
  p.qd = static_cast<const __nv_bfloat16*>(qd);
  p.kd = static_cast<const __nv_bfloat16*>(kd);
  p.k_absmax = absmax;
  p.ids = ids;
  p.status = ctx->status;
  p.fallbacks = fallbacks;
  p.hq = hq; p.hkv = hkv; p.qt = qt; p.nt = nt; p.r = r; p.topk = topk; p.qb = qb; p.cand = cand;
  p.q_chunks = (qt + qb - 1) / qb;
  const int grid = batch * hkv * p.q_chunks;
  const size_t smem = OFF_SCORES + ((static_cast<size_t>(qb) * nt * 4 + 15) & ~static_cast<size_t>(15)) + 144 +
                      128 * 4 + 10 * 4 + 16 * 4 + 1024;
  switch (gr) {
    case 1: return launch_gr<1>(qm, km, p, grid, smem, ctx, 0, stream);
    case 2: return launch_gr<2>(qm, km, p, grid, smem, ctx, 1, stream);
    case 4: return launch_gr<4>(qm, km, p, grid, smem, ctx, 2, stream);
    case 8: return launch_gr<8>(qm, km, p, grid, smem, ctx, 3, stream);
    case 16: return launch_gr<16>(qm, km, p, grid, smem, ctx, 4, stream);
    case 32: return launch_gr<32>(qm, km, p, grid, smem, ctx, 5, stream);
    case 64: return launch_gr<64>(qm, km, p, grid, smem, ctx, 6, stream);
  }
  return 1;
}

}  // namespace sb
