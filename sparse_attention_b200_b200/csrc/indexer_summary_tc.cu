// Tensor-core path of the R1 / R4 summary indexer: same block ids as the exact
// kernel of indexer_summary.cu, bit for bit, at tensor-core speed.
//
// An fp32-accumulating MMA does not reproduce the fixed summation order that
// defines a score, so the tensor cores only PRE-FILTER:
//   1. approximate scores of every KV block (tcgen05 MMA, key descriptors as the
//      M operand streamed by TMA, the query descriptors of QB query blocks as the
//      N operand, max over the group's rows and the R key representatives in the
//      epilogue) stay in shared memory;
//   2. per query block the C = k + extra best approximate blocks become candidates;
//      |approximate - exact| <= delta for every block of the list, with
//      delta = 2^-14 * min(max_m ||q_m||_1 * max|k element|, max_m ||q_m||_2 * max ||k row||_2) * 128^-0.5
//      (the sum of |q_d k_d| bounded by Hoelder and by Cauchy-Schwarz; 2^-14 is an order
//      of magnitude above the worst case of two 128-term fp32 sums);
//   3. two candidates whose approximate scores are more than 2 delta apart are ordered by
//      them for certain; a candidate with another one within 2 delta is re-scored with the
//      exact arithmetic (fp32 FMAs in feature order), and such pairs are ordered by
//      (exact score, block id). The top-k of the candidates is the answer if it is provably
//      safe: a lower bound of the k-th exact score > C-th approximate score + delta;
//   4. otherwise (ties that reach beyond the candidates, e.g. constant inputs) the list
//      falls back to exact scores of all blocks.
// The bound checks itself: every re-scored candidate has both of its scores in hand; a
// difference above delta sends the list to the exact fallback and is counted, and the largest
// observed |approximate - exact| / delta is kept for inspection.
// Replaces descriptor_dot + reduce_topk (indexers/r1_r4/gpu_ops.py:19-49).
#include "summary_tc_common.cuh"
#include "topk.cuh"

namespace sb {
namespace stc {

constexpr int TILE_BYTES = 128 * 256;      // 128 descriptors x 128 bf16
constexpr int PANEL_BYTES = 128 * 128;
#ifndef SB_STC_STAGES
#define SB_STC_STAGES 2
#endif
constexpr int A_STAGES = SB_STC_STAGES;
constexpr int SCORE_LIMIT = 232448 - 2048 - (A_STAGES + 1) * TILE_BYTES;   // bytes of shared memory left for scores
constexpr int LIST_WORDS = 3 * C_MAX;      // per list: block ids, approximate scores, exact scores (ordered ints)
constexpr int NUM_THREADS = 512;            // ten warps have a role in the scoring phase; all sixteen re-score
constexpr int EPI_WARPS = 8;               // two column halves x four TMEM lane quarters
constexpr int SEL_WARPS = 8;               // warps of the selection phase (one list each at a time)
constexpr int TMA_WARP = 8, MMA_WARP = 9;

constexpr int OFF_A = 0;
constexpr int OFF_B = A_STAGES * TILE_BYTES;
constexpr int OFF_SCORES = OFF_B + TILE_BYTES;
// after the scores: barriers, candidate arrays, scratch (offsets computed at run time)

// Exact score contribution of one key descriptor: max over the MP query rows of
// the fp32 dot product accumulated in feature order (q_s is [128][MP] fp32, 16-byte
// aligned). The key row is fetched a quarter (32 features) ahead of the arithmetic.
template <int MP>
__device__ __forceinline__ float exact_key_best(const float* q_s, const __nv_bfloat16* krow_g) {
  float acc[MP];
#pragma unroll
  for (int m = 0; m < MP; ++m) acc[m] = 0.f;
  const uint4* krow = reinterpret_cast<const uint4*>(krow_g);
  uint4 cur[4], nxt[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) cur[i] = __ldg(krow + i);
#pragma unroll 1
  for (int part = 0; part < 4; ++part) {
    if (part < 3) {
#pragma unroll
      for (int i = 0; i < 4; ++i) nxt[i] = __ldg(krow + 4 * (part + 1) + i);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&cur[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 kf = __bfloat1622float2(h[e]);
        const float4* q0 = reinterpret_cast<const float4*>(q_s + ((part * 4 + i) * 8 + 2 * e) * MP);
#pragma unroll
        for (int m = 0; m < MP / 4; ++m) {
          const float4 qa = q0[m];
          acc[4 * m + 0] = fmaf(qa.x, kf.x, acc[4 * m + 0]);
          acc[4 * m + 1] = fmaf(qa.y, kf.x, acc[4 * m + 1]);
          acc[4 * m + 2] = fmaf(qa.z, kf.x, acc[4 * m + 2]);
          acc[4 * m + 3] = fmaf(qa.w, kf.x, acc[4 * m + 3]);
        }
#pragma unroll
        for (int m = 0; m < MP / 4; ++m) {
          const float4 qa = q0[MP / 4 + m];
          acc[4 * m + 0] = fmaf(qa.x, kf.y, acc[4 * m + 0]);
          acc[4 * m + 1] = fmaf(qa.y, kf.y, acc[4 * m + 1]);
          acc[4 * m + 2] = fmaf(qa.z, kf.y, acc[4 * m + 2]);
          acc[4 * m + 3] = fmaf(qa.w, kf.y, acc[4 * m + 3]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
  }
  float best = acc[0];
#pragma unroll
  for (int m = 1; m < MP; ++m) best = fmaxf(best, acc[m]);
  return best;
}

// Exact dot products of FOUR key descriptors against MQ query rows (q_s points at the first
// of them inside the [128][stride] fp32 array): every fp32 sum runs in feature order, as in
// exact_key_best, but a query value fetched from shared memory feeds four FMAs per lane
// instead of one (the one-row form is bound by shared-memory loads). best[j] = max over the
// MQ rows for key j.
template <int MQ>
__device__ __forceinline__ void exact_quad_best(const float* q_s, int stride, const uint4* k0, const uint4* k1,
                                                const uint4* k2, const uint4* k3, float (&best)[4]) {
  // two query rows per 64-bit accumulator, packed FMAs (each half an ordinary fp32 FMA)
  unsigned long long acc[4][MQ / 2];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int m = 0; m < MQ / 2; ++m) acc[j][m] = 0ull;
  // A lane's 128 features are strictly sequential, so a wait for memory inside the loop is
  // paid in full: the 16-byte pieces of the four rows are requested two steps (16 features)
  // ahead, through three rotating buffers.
  const uint4* kr[4] = {k0, k1, k2, k3};
  auto fetch = [&](uint4 (&buf)[4], int c) {
    const int cc = c < 15 ? c : 15;
#pragma unroll
    for (int j = 0; j < 4; ++j) buf[j] = __ldg(kr[j] + cc);
  };
  auto step = [&](const uint4 (&buf)[4], int c) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      unsigned long long kx[4], ky[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 kf = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(&buf[j])[e]);
        kx[j] = f32x2_pack(kf.x, kf.x);
        ky[j] = f32x2_pack(kf.y, kf.y);
      }
      const ulonglong2* qa = reinterpret_cast<const ulonglong2*>(q_s + (c * 8 + 2 * e) * stride);
      const ulonglong2* qb = reinterpret_cast<const ulonglong2*>(q_s + (c * 8 + 2 * e + 1) * stride);
#pragma unroll
      for (int m = 0; m < MQ / 4; ++m) {
        const ulonglong2 q = qa[m];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[j][2 * m] = f32x2_fma(q.x, kx[j], acc[j][2 * m]);
          acc[j][2 * m + 1] = f32x2_fma(q.y, kx[j], acc[j][2 * m + 1]);
        }
      }
#pragma unroll
      for (int m = 0; m < MQ / 4; ++m) {
        const ulonglong2 q = qb[m];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[j][2 * m] = f32x2_fma(q.x, ky[j], acc[j][2 * m]);
          acc[j][2 * m + 1] = f32x2_fma(q.y, ky[j], acc[j][2 * m + 1]);
        }
      }
    }
  };
  uint4 b0[4], b1[4], b2[4];
  fetch(b0, 0);
  fetch(b1, 1);
#pragma unroll 1
  for (int c = 0; c < 15; c += 3) {              // on entry b0 = step c, b1 = step c + 1
    fetch(b2, c + 2);
    step(b0, c);
    fetch(b0, c + 3);
    step(b1, c + 1);
    fetch(b1, c + 4);
    step(b2, c + 2);
  }
  step(b0, 15);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float bst = -INFINITY;
#pragma unroll
    for (int m = 0; m < MQ / 2; ++m) {
      float lo, hi;
      f32x2_unpack(acc[j][m], lo, hi);
      bst = fmaxf(bst, fmaxf(lo, hi));
    }
    best[j] = bst;
  }
}

// One CTA: QB query blocks of one (batch, KV head) against every KV block.
// Warps 0-7 epilogue (warp & 3 = TMEM lane quarter, warp >> 2 = half of the accumulator
// columns when the columns split on a list boundary), warp 8 TMA, warp 9 MMA issue, the
// rest wait; the selection phase uses all sixteen.
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
  int* scratch_i = reinterpret_cast<int*>(scratch_f + 20);
  int* work_cnt = scratch_i + 20 + SEL_WARPS;            // [SEL_WARPS] candidates that need an exact score
  float* delta_s = reinterpret_cast<float*>(work_cnt + SEL_WARPS);   // [SEL_WARPS] error bound of a list
  float* kth_s = delta_s + SEL_WARPS;                    // [SEL_WARPS] lower bound of the k-th exact score
  int* l2_s = reinterpret_cast<int*>(kth_s + SEL_WARPS);  // [SEL_WARPS] largest squared L2 norm of a query descriptor
  volatile int* viol_s = l2_s + SEL_WARPS;                // [SEL_WARPS] a re-scored candidate of the list broke the bound
  int* l1_s = scratch_i + 20;                            // [SEL_WARPS] largest L1 norm of a list's query descriptors
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
  // The column halves must hold whole lists (GR >= 16: a list is GR / 16 chunks of 16
  // columns; GR < 16: a chunk holds 16 / GR lists), else warps 4-7 sit the tiles out.
  const bool split = p.qb >= 2 && n_cols >= 32;
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
      mbar_init(bar(ACC_EMPTY + i), split ? 8 : 4);
    }
    mbar_init(bar(B_FULL), 1);
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), 256);
    tmem_relinquish();
  }
  for (int j = threadIdx.x; j < p.qb * p.nt; j += NUM_THREADS) scores[j] = static_cast<int>(0x80000000u);
  if (threadIdx.x < SEL_WARPS) l1_s[threadIdx.x] = l2_s[threadIdx.x] = 0;
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
        bool w = mbar_wait(bar(A_EMPTY + s), (use - 1) & 1, guard, 0x900 + s);
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
      bool w = mbar_wait(bar(B_FULL), 0, guard, 0x910);
      ok = __all_sync(0xffffffffu, w);
      tc_fence_after();
    }
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int s = t % A_STAGES, acc = t & 1;
      bool w = mbar_wait(bar(A_FULL + s), (t / A_STAGES) & 1, guard, 0x920 + s);
      if (w && t >= 2) w = mbar_wait(bar(ACC_EMPTY + acc), ((t >> 1) - 1) & 1, guard, 0x930 + acc);
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
  } else if (warp < (split ? EPI_WARPS : 4)) {
    // epilogue: thread = key descriptor row of the tile, over this warp's share of the columns
    const int quarter = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int r_log2 = 31 - __clz(p.r);                  // R is 1, 2 or 4
    const int n_chunks = split ? (n_cols >> 5) : (n_cols >> 4);     // at most 4 either way
    const int c0 = (warp >> 2) * n_chunks;               // first chunk of this warp
    const int list0 = GR >= 16 ? (c0 * 16) / GR : c0 * (16 / (GR >= 16 ? 16 : GR));
    bool ok = true;
    for (int t = 0; ok && t < num_tiles; ++t) {
      const int acc = t & 1;
      bool w = mbar_wait(bar(ACC_FULL + acc), (t >> 1) & 1, guard, 0x940 + acc);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      const int n = ((t + rot) % num_tiles) * 128 + quarter * 32 + lane;
      const bool row_ok = n < n_keys;
      const int blk = n >> r_log2;
      const uint32_t t_acc = tmem + lane_base + acc * 128 + c0 * 16;
      // all columns into registers with one wait, then hand the accumulator back at once
      uint32_t v[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c < n_chunks) tmem_ld16(t_acc + c * 16, v[c]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(ACC_EMPTY + acc));
      // Every (query block, KV block) pair is produced by exactly one lane group of one
      // tile, so a plain store suffices.
      auto flush = [&](int tl, float val) {
        for (int d = 1; d < p.r; d <<= 1) val = fmaxf(val, __shfl_xor_sync(0xffffffffu, val, d));
        tl += list0;
        if (row_ok && (lane & (p.r - 1)) == 0 && qtile0 + tl < p.qt) scores[tl * p.nt + blk] = f2ord(val);
      };
      float cur = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
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

  // ------------------------------------------------------------- selection, SEL_WARPS lists per round
  // The operand buffers are free now: the fp32 query descriptors of the round's lists go to
  // the A stages, their candidate arrays to the B tile. Per round:
  //   1. all threads stage the query descriptors of the round's lists and their L1 norms;
  //   2. two to sixteen warps per list find the C-th largest approximate score and the candidates;
  //   3. all threads find the candidates whose order the approximate scores do not settle,
  //      and re-score those exactly, (four key rows, up to 8 query rows) per lane;
  //   4. all threads rank the candidates by counting; one thread per list proves safety.
  const __nv_bfloat16* kbase = p.kd + static_cast<long long>(bk) * n_keys * 128;
  const float kabs = p.k_absmax[bk], knorm = sqrtf(p.k_norm2[bk]);
  const int lists = min(p.qb, p.qt - qtile0);
  const int C = p.cand;
  constexpr int MQ = MP < 8 ? MP : 8;            // query rows of one re-scoring item
  float* q_all = reinterpret_cast<float*>(gbase + OFF_A);
  int32_t* cand_all = reinterpret_cast<int32_t*>(gbase + OFF_B);
  for (int tl0 = 0; tl0 < lists; tl0 += SEL_WARPS) {
    const int nl = min(SEL_WARPS, lists - tl0);
    // 1. one descriptor row per thread: the transposing stores of a warp then fall into 32
    //    different banks (a row per warp would put all of them into one)
    for (int idx = threadIdx.x; idx < nl * MP; idx += NUM_THREADS) {
      const int l = idx / MP, m = idx - l * MP;
      const int mm = m < GR ? m : 0;             // padding repeats descriptor 0: the maximum is unchanged
      const int g = mm / p.r, rq = mm - g * p.r;
      const long long qrow = ((static_cast<long long>(b) * p.hq + kvh * group + g) * p.qt + qtile0 + tl0 + l) * p.r + rq;
      const uint4* src = reinterpret_cast<const uint4*>(p.qd + qrow * 128);
      float* dst = q_all + l * 128 * MP + m;
      float sum = 0.f, squares = 0.f;
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        const uint4 raw = __ldg(src + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          dst[(c * 8 + 2 * e) * MP] = f.x;
          dst[(c * 8 + 2 * e + 1) * MP] = f.y;
          sum += fabsf(f.x);
          sum += fabsf(f.y);
          squares = fmaf(f.x, f.x, squares);
          squares = fmaf(f.y, f.y, squares);
        }
      }
      atomicMax(l1_s + l, __float_as_int(sum));  // non-negative floats order as ints
      atomicMax(l2_s + l, __float_as_int(squares));
    }
    __syncthreads();
    // 2. `wpl` warps per list (as many as there are, but no more than one per 1024 keys: with
    //    short lists the meetings cost more than the shared scan saves); each takes a contiguous
    //    slice of the list's keys and the warps of a list meet at a named barrier
    int wpl = nl <= 1 ? 16 : nl <= 2 ? 8 : nl <= 4 ? 4 : 2;
    while (wpl > 1 && wpl * 1024 > p.nt) wpl >>= 1;
    const int slot = warp / wpl, sub = warp - slot * wpl;
    const bool active = slot < nl;
    const bool mine = active && sub == 0;        // this warp speaks for list tl of the round
    const int tl = tl0 + slot;
    int32_t* cand_ids = cand_all + slot * LIST_WORDS;
    float* cand_apx = reinterpret_cast<float*>(cand_ids + C_MAX);
    const unsigned lt_mask = (1u << lane) - 1u;
    float delta = 0.f, thr = 0.f;
    if (active) {
      auto group_sync = [&]() {
        if (wpl > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(wpl * 32) : "memory");
        else __syncwarp();
      };
      const unsigned* keys = reinterpret_cast<const unsigned*>(scores + tl * p.nt);   // ordered ints
      int* hist = cand_all + SEL_WARPS * LIST_WORDS + slot * 256;
      // per list: smallest key, largest key, candidates written, -, ties seen by each warp
      unsigned* grp = reinterpret_cast<unsigned*>(cand_all + SEL_WARPS * LIST_WORDS + SEL_WARPS * 256 + slot * 24);
      const int span = (((p.nt + wpl - 1) / wpl) + 31) & ~31;
      const int lo = sub * span, hi = min(p.nt, lo + span);
      // sum of |q_d k_d| over the features, bounded by Hoelder (L1 x max) and by Cauchy-Schwarz
      delta = EPS * 1.0001f * fminf(__int_as_float(l1_s[slot]) * kabs, sqrtf(__int_as_float(l2_s[slot])) * knorm) * SCALE;
      // C-th largest approximate score T by radix selection, eight bits per pass: histogram
      // of the digit among the keys that match the digits found so far, then the largest
      // digit whose suffix count reaches what is still needed. The keys are first moved to
      // w = (key - smallest key) << (leading zeros of the range): scores of one list share
      // their exponent bits, and a digit taken from those would send every lane of a warp to
      // the same histogram bin. Afterwards `need` keys equal to T are wanted besides all above.
      if (sub == 0 && lane == 0) {
        grp[0] = 0xffffffffu;
        grp[1] = 0u;
        grp[2] = 0u;
      }
      group_sync();
      unsigned umin = 0xffffffffu, umax = 0u;
#pragma unroll 8
      for (int j = lo + lane; j < hi; j += 32) {
        const unsigned u = keys[j] ^ 0x80000000u;
        umin = min(umin, u);
        umax = max(umax, u);
      }
      umin = __reduce_min_sync(0xffffffffu, umin);
      umax = __reduce_max_sync(0xffffffffu, umax);
      if (lane == 0 && lo < hi) {
        atomicMin(grp, umin);
        atomicMax(grp + 1, umax);
      }
      group_sync();
      umin = grp[0];
      umax = grp[1];
      const int lz = min(__clz(umax - umin), 31);
      unsigned W = 0;
      int need = C;
      for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (shift + 8 <= lz) break;              // the remaining bits of every w are zero
        for (int i = sub * 32 + lane; i < 256; i += wpl * 32) hist[i] = 0;
        group_sync();
        // keys are fetched eight at a time: a load cannot be moved above an atomic by the
        // compiler, and one round trip to shared memory per key is what this loop costs otherwise
        const unsigned top = pass == 0 ? 0u : W >> (shift + 8);
        // the trip count must be the same for every lane (the vote below takes the whole warp): the loop
        // runs on the slice's first index, the lane offset is added inside
        for (int jb = lo; jb < hi; jb += 256) {
          const int j0 = jb + lane;
          unsigned x[8];
          bool any = false;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            x[i] = j0 + 32 * i < hi ? ((keys[j0 + 32 * i] ^ 0x80000000u) - umin) << lz : 0u;
            any |= j0 + 32 * i < hi && (pass == 0 || (x[i] >> (shift + 8)) == top);
          }
          if (!__any_sync(0xffffffffu, any)) continue;      // after the first pass few keys still match
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (j0 + 32 * i < hi && (pass == 0 || (x[i] >> (shift + 8)) == top))
              atomicAdd(hist + ((x[i] >> shift) & 255u), 1);
        }
        group_sync();
        int h[8], lsum = 0;                      // lane l holds digits 8 l .. 8 l + 7
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          h[i] = hist[8 * lane + i];
          lsum += h[i];
        }
        int above = lsum;                        // inclusive suffix sum over lanes >= this one
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_down_sync(0xffffffffu, above, d);
          if (lane + d < 32) above += o;
        }
        above -= lsum;                           // keys in digits of higher lanes
        const bool here = above < need && need <= above + lsum;   // exactly one lane
        int digit = 0, left = 0;
        if (here) {
          int run = above;
#pragma unroll
          for (int i = 7; i >= 0; --i) {
            if (run < need && need <= run + h[i]) {
              digit = 8 * lane + i;
              left = need - run;
            }
            run += h[i];
          }
        }
        const int src = __ffs(__ballot_sync(0xffffffffu, here)) - 1;
        digit = __shfl_sync(0xffffffffu, digit, src);
        need = __shfl_sync(0xffffffffu, left, src);
        W |= static_cast<unsigned>(digit) << shift;
        group_sync();                            // every warp has read the histogram
      }
      const unsigned T = (W >> lz) + umin;
      // candidates: everything above T, then ties at T in index order, C in total. First the
      // ties of each slice are counted, so that a warp knows how many lie before its slice.
      const int need_eq = need;
      int eq_mine = 0;
      for (int j0 = lo; j0 < hi; j0 += 256) {
        int c8 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = j0 + 32 * i + lane;
          c8 += static_cast<int>(j < hi && (keys[j] ^ 0x80000000u) == T);
        }
        eq_mine += c8;
      }
      eq_mine = __reduce_add_sync(0xffffffffu, eq_mine);
      if (lane == 0) grp[4 + sub] = static_cast<unsigned>(eq_mine);
      group_sync();
      int eq_run = 0;
      for (int w = 0; w < sub; ++w) eq_run += static_cast<int>(grp[4 + w]);
      for (int j0 = lo; j0 < hi; j0 += 256) {    // eight groups of 32 keys per step
        unsigned u[8];
        bool any_ge = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = j0 + 32 * i + lane;
          u[i] = j < hi ? (keys[j] ^ 0x80000000u) : 0u;
          any_ge |= j < hi && u[i] >= T;
        }
        if (!__any_sync(0xffffffffu, any_ge)) continue;     // most steps hold no candidate
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = j0 + 32 * i + lane;
          const bool is_ge = j < hi && u[i] >= T;
          const bool is_eq = is_ge && u[i] == T;
          const unsigned eq_ballot = __ballot_sync(0xffffffffu, is_eq);
          const bool take = is_ge && (!is_eq || eq_run + __popc(eq_ballot & lt_mask) < need_eq);
          const unsigned take_ballot = __ballot_sync(0xffffffffu, take);
          eq_run += __popc(eq_ballot);
          if (take_ballot == 0u) continue;
          int first = 0;                         // the order of the candidates in their arrays is free
          if (lane == 0) first = static_cast<int>(atomicAdd(grp + 2, static_cast<unsigned>(__popc(take_ballot))));
          first = __shfl_sync(0xffffffffu, first, 0);
          if (take) {
            const int pos = first + __popc(take_ballot & lt_mask);
            cand_ids[pos] = j;
            cand_apx[pos] = ord2f(static_cast<int>(u[i] ^ 0x80000000u)) * SCALE;
          }
        }
      }
      thr = ord2f(static_cast<int>(T ^ 0x80000000u)) * SCALE;
      if (mine && lane == 0) {
        delta_s[slot] = delta;
        work_cnt[slot] = 0;
        kth_s[slot] = -INFINITY;
        viol_s[slot] = 0;
      }
    }
    __syncthreads();
    // 3a. Approximate and exact score of a block differ by at most delta, so two candidates
    //     whose approximate scores are more than 2 delta apart are ordered by them for certain.
    //     Only a candidate with another one within 2 delta needs its exact score: those go to
    //     the work list of their list (the histograms are free by now).
    int* work = cand_all + SEL_WARPS * LIST_WORDS;            // [SEL_WARPS][C_MAX] candidate slots
    for (int idx = threadIdx.x; idx < nl * C; idx += NUM_THREADS) {
      const int l = idx / C, c = idx - l * C;
      const float* apx = reinterpret_cast<const float*>(cand_all + l * LIST_WORDS + C_MAX);
      const float a = apx[c], two = 2.f * delta_s[l];
      int near = 0;
#pragma unroll 4
      for (int j = 0; j < C; ++j) near |= static_cast<int>(j != c) & static_cast<int>(!(fabsf(a - apx[j]) > two));
      int* ord = cand_all + l * LIST_WORDS + 2 * C_MAX;
      if (near) {
        ord[c] = f2ord(-INFINITY);
        work[l * C_MAX + atomicAdd(work_cnt + l, 1)] = c;
      } else {
        ord[c] = INT_MIN;                        // "no exact score": below every ordered float
      }
    }
    __syncthreads();
    // 3b. exact scores of the work lists. Items of a list: (quad of key rows, chunk of MQ query
    //     rows), chunks fastest: the MP / MQ lanes of a quad ask for the same key bytes (one
    //     memory transaction), and their query values sit in different banks. Key row = work
    //     entry * R + representative; rows past the end repeat the last one (a maximum does
    //     not mind).
    {
      int pre[SEL_WARPS + 1];
      pre[0] = 0;
#pragma unroll
      for (int l = 0; l < SEL_WARPS; ++l) {
        const int rows = l < nl ? work_cnt[l] * p.r : 0;
        pre[l + 1] = pre[l] + ((rows + 3) >> 2) * (MP / MQ);
      }
      const int total = pre[SEL_WARPS];
      for (int base_i = warp * 32; base_i < total; base_i += NUM_THREADS) {
        const int item = base_i + lane;
        if (item < total) {
          int l = 0, first = 0;
#pragma unroll
          for (int x = 1; x < SEL_WARPS; ++x)
            if (item >= pre[x]) { l = x; first = pre[x]; }
          const int rem = item - first;
          const int quad = rem / (MP / MQ), chunk = rem - quad * (MP / MQ);
          const int rows = work_cnt[l] * p.r;
          const int32_t* ids_l = cand_all + l * LIST_WORDS;
          int* ord_l = cand_all + l * LIST_WORDS + 2 * C_MAX;
          int cidx[4];
          const uint4* krow[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = min(quad * 4 + j, rows - 1);
            const int n = row / p.r, rk = row - n * p.r;
            cidx[j] = work[l * C_MAX + n];
            krow[j] = reinterpret_cast<const uint4*>(kbase + (static_cast<long long>(ids_l[cidx[j]]) * p.r + rk) * 128);
          }
          float best[4];
          exact_quad_best<MQ>(q_all + l * 128 * MP + chunk * MQ, MP, krow[0], krow[1], krow[2], krow[3], best);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (best[j] == best[j]) atomicMax(ord_l + cidx[j], f2ord(best[j]));   // a NaN leaves the slot alone
        }
      }
    }
    __syncthreads();
    // 4. rank of a candidate = number of candidates that beat it in (exact score descending,
    //    block id ascending): decided by the approximate scores when they are more than
    //    2 delta apart, else by the exact scores (both candidates have one then).
    for (int idx = threadIdx.x; idx < nl * C; idx += NUM_THREADS) {
      const int l = idx / C, c = idx - l * C;
      const int32_t* ids_l = cand_all + l * LIST_WORDS;
      const float* apx = reinterpret_cast<const float*>(ids_l + C_MAX);
      const int* ord = ids_l + 2 * C_MAX;
      const float dl = delta_s[l], two = 2.f * dl;
      const float a = apx[c];
      const int o = ord[c], id = ids_l[c];
      const float e = ord2f(o) * SCALE;
      if (o != INT_MIN && e == e) {              // both scores in hand: the bound must hold
        const float diff = fabsf(a - e);
        if (dl > 0.f) atomicMax(p.max_ratio, __float_as_int(diff / dl));
        if (!(diff <= dl)) {
          viol_s[l] = 1;
          atomicAdd(p.violations, 1);
        }
      }
      int rank = 0;
#pragma unroll 4
      for (int j = 0; j < C; ++j) {
        const float d = apx[j] - a, ej = ord2f(ord[j]) * SCALE;
        const int gt = static_cast<int>(d > two), lt = static_cast<int>(d < -two);
        const int exact = static_cast<int>(ej > e) | (static_cast<int>(ej == e) & static_cast<int>(ids_l[j] < id));
        rank += gt | ((gt | lt) ^ 1) & exact;
      }
      if (rank < p.topk) p.ids[(static_cast<long long>(bk) * p.qt + qtile0 + tl0 + l) * p.topk + rank] = id;
      // a lower bound of the k-th exact score, for the safety test
      if (rank == p.topk - 1) kth_s[l] = o != INT_MIN ? e : a - dl;
    }
    __syncthreads();
    // safe: no block outside the candidates (exact score <= thr + delta) can reach the top k
    if (mine && lane == 0) flags[tl] = (!viol_s[slot] && ((C >= p.nt) || (kth_s[slot] > thr + delta))) ? 0 : 1;
    if (tl0 + SEL_WARPS < lists) {               // another round re-uses the buffers
      __syncthreads();
      if (threadIdx.x < SEL_WARPS) l1_s[threadIdx.x] = l2_s[threadIdx.x] = 0;
      __syncthreads();
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

// max |element| and max squared L2 norm of the key descriptors of each (batch, KV head);
// sixteen adjacent lanes hold one descriptor (per_head is a multiple of 128 elements)
__global__ void __launch_bounds__(256) absmax_kernel(const __nv_bfloat16* __restrict__ kd, float* __restrict__ out,
                                                     float* __restrict__ out_norm2, long long per_head) {
  const int head = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(kd + static_cast<long long>(head) * per_head);
  const long long n16 = per_head / 8;
  float m = 0.f, n2 = 0.f;
  const int lane = threadIdx.x & 31;
  for (long long base = static_cast<long long>(blockIdx.x) * blockDim.x + (threadIdx.x - lane); base < n16;
       base += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = base + lane;
    const uint4 v = i < n16 ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float sq = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
      sq = fmaf(f.x, f.x, sq);
      sq = fmaf(f.y, f.y, sq);
    }
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
    n2 = fmaxf(n2, sq);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    n2 = fmaxf(n2, __shfl_xor_sync(0xffffffffu, n2, d));
  }
  if (lane == 0) {
    atomicMax(reinterpret_cast<int*>(out + head), __float_as_int(m));
    atomicMax(reinterpret_cast<int*>(out_norm2 + head), __float_as_int(n2));
  }
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
// aux: device floats [B*Hkv] (key abs-max) + [B*Hkv] (largest squared key norm), both filled
// here, + 3 words: lists that took the exact fallback (int), re-scored candidates that broke the error
// bound (int), largest observed |approximate - exact| / delta (float).
int launch_summary_select_tc(const void* qd, const void* kd, void* aux, int32_t* ids, int batch, int hq, int hkv,
                             int qt, int nt, int r, int topk, cudaStream_t stream) {
  using namespace stc;
  const int group = hq / hkv, gr = group * r;
  if (gr > 64 || (gr & (gr - 1)) != 0) return 1;
  const int extra = topk / 4 > 16 ? topk / 4 : 16;
  int cand = topk + extra;
  if (cand > nt) cand = nt;
  if (cand > C_MAX) return 1;
  if (static_cast<long long>(batch) * hkv * nt * r >= (1LL << 31) || r > 256 || group > 256) return 1;
  // the one-CTA-per-unit kernel keeps all scores of its lists in shared memory
  int qb = 128 / gr;
  while (qb > 1 && qb * gr > 16 && (qb / 2) >= qt) qb >>= 1;        // do not cover far more query blocks than exist
  while (static_cast<long long>(qb) * nt * 4 > SCORE_LIMIT && qb * gr > 16) qb >>= 1;
  const bool unit_form_ok = !(static_cast<long long>(qb) * nt * 4 > SCORE_LIMIT || qb * gr < 16 || qb > 256);
  // The persistent kernel overlaps the selection of one unit with the scoring of the next; it pays
  // where scoring dominates (long lists). Short lists are selection-bound and stay with the kernel
  // whose whole CTA selects.
  const bool stream_form_ok = gr == 32 && qt >= 256 / gr && r <= 4 &&
                              (static_cast<long long>(nt) * r >= STREAM_MIN_KEY_ROWS || !unit_form_ok);
  if (!unit_form_ok && !stream_form_ok) return 1;
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;

  float* absmax = static_cast<float*>(aux);
  float* norm2 = absmax + static_cast<size_t>(batch) * hkv;
  int* fallbacks = reinterpret_cast<int*>(norm2 + static_cast<size_t>(batch) * hkv);
  if (cudaMemsetAsync(aux, 0, (2 * static_cast<size_t>(batch) * hkv + 3) * 4, stream) != cudaSuccess)
    return set_error(SB_ERR_CUDA, "memset failed");
  const long long per_head = static_cast<long long>(nt) * r * 128;
  int chunks = static_cast<int>((per_head / 8 + 256 * 8 - 1) / (256 * 8));
  if (chunks > 64) chunks = 64;
  if (chunks < 1) chunks = 1;
  absmax_kernel<<<dim3(chunks, batch * hkv), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(kd), absmax, norm2, per_head);

  Params p{};
  p.qd = static_cast<const __nv_bfloat16*>(qd);
  p.kd = static_cast<const __nv_bfloat16*>(kd);
  p.k_absmax = absmax;
  p.k_norm2 = norm2;
  p.ids = ids;
  p.status = ctx->status;
  p.fallbacks = fallbacks;
  p.violations = fallbacks + 1;
  p.max_ratio = fallbacks + 2;
  p.hq = hq; p.hkv = hkv; p.qt = qt; p.nt = nt; p.r = r; p.topk = topk; p.cand = cand;

  if (stream_form_ok) {
    // lists it could not prove carry -1 as their first id and are re-done exactly
    int rc = launch_summary_stream(qd, kd, p, batch, ctx, stream);
    if (rc == SB_OK)
      return launch_summary_score_topk(qd, kd, nullptr, ids, batch, hq, hkv, qt, nt, r, topk, stream, 1);
    if (rc != 1) return rc;
  }
  if (!unit_form_ok) return 1;

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
  p.qb = qb;
  p.q_chunks = (qt + qb - 1) / qb;
  const int grid = batch * hkv * p.q_chunks;
  const size_t smem = OFF_SCORES + ((static_cast<size_t>(qb) * nt * 4 + 15) & ~static_cast<size_t>(15)) + 144 +
                      128 * 4 + 20 * 4 + 20 * 4 + 6 * SEL_WARPS * 4 + 1024;
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
