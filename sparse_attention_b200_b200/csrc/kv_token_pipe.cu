// KV-centric attention for per-TOKEN selection lists, pipelined variant for GQA groups of
// 8 or 16 query heads per KV head (the reference's KV-centric contract is Hq16 / Hkv1).
//
// A task = (KV-head group, KV block, up to 128/G queries that selected the block); its
// 128-row Q tile is the G heads of each of those queries. One persistent CTA per SM walks
// a contiguous range of the task list (tasks are ordered by (group, block), so a CTA
// reloads K/V two or three times in all) and keeps TWO tasks in flight, one per stream:
//   warp 13      TMA producer: the K/V block when it changes (the pipeline drains there,
//                two or three times per CTA); per query one 3-D box {64 columns, 1 token,
//                G heads} of Q per 64-column panel, straight into the 128-byte-swizzled
//                operand tile of a four-slot ring (Q rows mostly come from HBM: four
//                tasks of loads in flight cover that latency)
//   warp 12      one thread issues QK(j), then PV(j-1) of the other stream (tcgen05, TMEM)
//   warps 0-3 / 4-7   softmax of stream 0 / 1 over the single block, P (bf16) back into S,
//                1/row-sum to shared memory, LSE to global memory
//   warps 8-11   epilogue: O out of tensor memory, normalise, stage, and one 4-D TMA store
//                {64 columns, 1 rank, 1 token, G heads} per query and panel into the partial
//                slot (query, rank) the selection list gave the block
// Same computation as kv_tma11_ops::main_kernel
// (attention/kv_centric/optimization_round11/tma11_kernel.cu:97-390) for any TopK, with q
// head-major [B,Hq,Sq,128], partials [B,Hq,Sq,TopK,128] bf16 and LSE [B,Hq,Sq,TopK].
// Rows of a tile beyond the task's query count keep whatever the buffer held: every row
// of S, P and O depends on its own Q row only, and those rows are never stored.
#include <algorithm>
#include "ptx.cuh"
#include "internal.h"

namespace sb {
namespace kvp {

constexpr int TILE_BYTES = 128 * 256;
constexpr int PANEL_BYTES = 128 * 128;
constexpr int NUM_THREADS = 512;
constexpr int EPI_WARP0 = 8;
constexpr int MMA_WARP = 12;
constexpr int LOAD_WARP = 13;
// register budgets per thread after the setup barrier: 128 * (2 * 176 + 64 + 96) = 65536
constexpr int SOFTMAX_REGS = 176;
constexpr int EPI_REGS = 64;
constexpr int CTRL_REGS = 96;

constexpr int QRING = 4;
constexpr int OFF_Q = 0;                               // [QRING] Q tiles
constexpr int OFF_KV = QRING * TILE_BYTES;             // K tile, V tile
constexpr int OFF_STAGE = OFF_KV + 2 * TILE_BYTES;     // 4 epilogue warps x 8 KiB
constexpr int STAGE_BYTES = 8192;
constexpr int OFF_STATS = OFF_STAGE + 4 * STAGE_BYTES; // [2 streams][128 rows] 1 / row sum
constexpr int OFF_BAR = OFF_STATS + 2 * 128 * 4;
enum {
  S_FULL = 0, P_FULL = 2, O_FULL = 4, O_EMPTY = 6, STATS_FULL = 8, STATS_EMPTY = 10, KV_FULL = 12, KV_EMPTY = 13,
  Q_FULL = 14, Q_EMPTY = 14 + QRING, NUM_BARS = 14 + 2 * QRING
};
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;       // tmem base, abort flag
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;       // + slack for manual 1024 alignment
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory map exceeds the per-CTA limit");

struct Params {
  const int32_t* tasks;         // [T, 4] (group, block, first edge, count)
  const int32_t* task_count;    // number of tasks (device memory)
  const int32_t* qids;
  const int32_t* ranks;
  float* lses;                  // [B, Hq, Sq, TopK]
  int* status;
  int batch, hq, hkv, sq, skv, topk, group, group_log2, edges;
  int phases;                   // upper bound on the number of passes over the task list (see Walk)
  int q_token_major;            // q is [B, Sq, Hq, 128]: the G heads of a token are one dense box
  int partial_token_major;      // partials are [B, Sq, TopK, Hq, 128] (the reference's token-major operators)
  float* partial_f32;           // non-null: fp32 partials (the reference's fp32 controls), written with plain stores
  float scale_log2;
};

// Order in which a CTA visits tasks. The task list (sorted by KV-head group, then block) is
// cut into `phases` equal segments; within a segment every CTA takes a contiguous share,
// and the CTAs go through the segments together. At any time the whole GPU then gathers Q
// rows of a few groups only, so they come from L2 instead of HBM (one contiguous share of
// the whole list per CTA spreads the gathers over all of Q), at the price of one more
// K/V reload per CTA and segment.
struct Walk {
  int total, seg, per, count;   // tasks, tasks per segment, tasks per CTA and segment, slots to visit
  __device__ __forceinline__ int task(int i) const {      // -1: nothing in this slot
    const int ph = i / per, j = static_cast<int>(blockIdx.x) * per + (i - ph * per);
    const long long t = static_cast<long long>(ph) * seg + j;
    return (j < seg && t < total) ? static_cast<int>(t) : -1;
  }
};

struct Task {
  int group, block, start, count;
  bool valid;
};

__device__ __forceinline__ Task read_task(const Params& p, const Walk& walk, int i) {
  const int t = i < walk.count ? walk.task(i) : -1;
  if (t < 0) return Task{0, 0, 0, 0, false};
  const int4 raw = *reinterpret_cast<const int4*>(p.tasks + static_cast<long long>(t) * 4);
  Task k;
  k.group = raw.x; k.block = raw.y; k.start = raw.z; k.count = raw.w;
  k.valid = k.group >= 0 && k.group < p.batch * p.hkv && k.block >= 0 && k.block < p.skv / 128 && k.start >= 0 &&
            k.count > 0 && k.count <= (128 >> p.group_log2) && static_cast<long long>(k.start) + k.count <= p.edges;
  return k;
}

// 3-D tile load {x, y, z}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// 4-D tile store {x, y, z, w}; no coordinate may be negative
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, int x, int y, int z, int w, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(map),
               "r"(x), "r"(y), "r"(z), "r"(w), "r"(src)
               : "memory");
}

template <bool F32>      // fp32 partials (plain stores) instead of bf16 (staged, TMA stores)
__global__ void __launch_bounds__(NUM_THREADS, 1)
kv_token_pipe_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                     const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap o_map,
                     const Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(gbase + OFF_MISC);
  float* stats = reinterpret_cast<float*>(gbase + OFF_STATS);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Guard guard{misc + 1, p.status};

  if (threadIdx.x == 0) {
    misc[1] = 0;
    for (int i = 0; i < QRING; ++i) {
      mbar_init(bar(Q_FULL + i), 1);
      mbar_init(bar(Q_EMPTY + i), 1);
    }
    mbar_init(bar(KV_FULL), 1);
    mbar_init(bar(KV_EMPTY), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(P_FULL + i), 4);
      mbar_init(bar(O_FULL + i), 1);
      mbar_init(bar(O_EMPTY + i), 4);
      mbar_init(bar(STATS_FULL + i), 4);
      mbar_init(bar(STATS_EMPTY + i), 4);
    }
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), 512);
    tmem_relinquish();
  }
  if (warp == LOAD_WARP && lane == 0) {
    prefetch_tmap(&q_map);
    prefetch_tmap(&k_map);
    prefetch_tmap(&v_map);
    prefetch_tmap(&o_map);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = static_cast<uint32_t>(misc[0]);
  // tensor memory columns: S0 0..127, S1 128..255, O0 256..383, O1 384..511; P over S.

  Walk walk;
  walk.total = *p.task_count;
  {
    const int grid = static_cast<int>(gridDim.x);
    const int phases = max(1, min(p.phases, walk.total / (grid * 16)));   // at least 16 tasks per CTA and segment
    walk.seg = (walk.total + phases - 1) / phases;
    walk.per = max(1, (walk.seg + grid - 1) / grid);
    walk.count = phases * walk.per;
  }
  const int t_begin = 0, t_end = walk.count;
  const int G = p.group;

  if (warp >= MMA_WARP) {
  setmaxnreg_dec<CTRL_REGS>();
  if (warp == LOAD_WARP) {
    // ------------------------------------------------------------- TMA producer
    uint32_t n = 0;                 // valid tasks so far
    int loads = 0;                  // K/V block loads so far
    int cur_group = -1, cur_block = -1;
    bool ok = true;
    // the query ids of a task are fetched one task ahead
    auto fetch_qi = [&](const Task& k) -> int {
      int qi = -1;
      if (k.valid && lane < k.count) {
        qi = p.qids[k.start + lane];
        if (qi < 0 || qi >= p.sq) qi = -1;
      }
      return qi;
    };
    Task k = read_task(p, walk, t_begin);
    int qi = fetch_qi(k);
    for (int t = t_begin; ok && t < t_end; ++t) {
      const Task cur = k;
      const int cur_qi = qi;
      k = read_task(p, walk, t + 1);
      qi = fetch_qi(k);
      if (!cur.valid) continue;
      const uint32_t slot = n % QRING, use = n / QRING;
      ++n;
      if (cur.group != cur_group || cur.block != cur_block) {
        cur_group = cur.group; cur_block = cur.block;
        if (loads > 0) {
          bool w = mbar_wait(bar(KV_EMPTY), (loads - 1) & 1, guard, 0x700);
          ok = __all_sync(0xffffffffu, w);
          if (!ok) break;
        }
        ++loads;
        if (lane == 0) {
          const int kv_row = cur.group * p.skv + cur.block * 128;
          const uint32_t dst = base + OFF_KV;
          mbar_expect_tx(bar(KV_FULL), 2 * TILE_BYTES);
          tma_load_2d(dst, &k_map, 0, kv_row, bar(KV_FULL));
          tma_load_2d(dst + PANEL_BYTES, &k_map, 64, kv_row, bar(KV_FULL));
          tma_load_2d(dst + TILE_BYTES, &v_map, 0, kv_row, bar(KV_FULL));
          tma_load_2d(dst + TILE_BYTES + PANEL_BYTES, &v_map, 64, kv_row, bar(KV_FULL));
        }
      }
      if (use > 0) {
        bool w = mbar_wait(bar(Q_EMPTY + slot), (use - 1) & 1, guard, 0x710 + slot);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
      }
      const unsigned live = __ballot_sync(0xffffffffu, cur_qi >= 0);
      if (lane == 0) mbar_expect_tx(bar(Q_FULL + slot), static_cast<uint32_t>(__popc(live)) * G * 256u);
      __syncwarp();
      if (cur_qi >= 0) {
        const int b = cur.group / p.hkv, kvh = cur.group - b * p.hkv;
        const uint32_t dst = base + OFF_Q + slot * TILE_BYTES + lane * G * 128;
        // head-major q: {column, token, batch * Hq + head}; token-major q: {column, head, batch * Sq + token}
        const int y = p.q_token_major ? kvh * G : cur_qi;
        const int z = p.q_token_major ? b * p.sq + cur_qi : b * p.hq + kvh * G;
        tma_load_3d(dst, &q_map, 0, y, z, bar(Q_FULL + slot));
        tma_load_3d(dst + PANEL_BYTES, &q_map, 64, y, z, bar(Q_FULL + slot));
      }
    }
    if (!ok) {
      // let copies in flight land before the CTA gives up its shared memory
      for (uint32_t i = 0; i < QRING; ++i)
        if (n > i) mbar_wait_drain(bar(Q_FULL + ((n - 1 - i) % QRING)), ((n - 1 - i) / QRING) & 1);
      if (loads > 0) mbar_wait_drain(bar(KV_FULL), (loads - 1) & 1);
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = idesc_bf16(128, 128, false);
      constexpr uint32_t IDESC_PV = idesc_bf16(128, 128, true);
      uint32_t n = 0;
      int loads = 0, cur_group = -1, cur_block = -1;
      bool ok = true;
      bool pv_pending = false;      // the PV of task n - 1 has not been issued yet
      // O_{s} = P_{s} V of the task numbered m (stream m & 1)
      auto issue_pv = [&](uint32_t m) -> bool {
        const uint32_t s = m & 1, u = m >> 1;
        if (!mbar_wait(bar(P_FULL + s), u & 1, guard, 0x720 + s)) return false;
        if (u > 0 && !mbar_wait(bar(O_EMPTY + s), (u - 1) & 1, guard, 0x730 + s)) return false;
        tc_fence_after();
        const uint64_t b0 = desc_sw128_mnmajor(base + OFF_KV + TILE_BYTES, PANEL_BYTES, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          mma_ts(tmem + 256 + s * 128, tmem + s * 128 + kk * 8, b0 + static_cast<uint64_t>(kk * (2048 >> 4)),
                 IDESC_PV, kk > 0 ? 1u : 0u);
        tc_commit(bar(O_FULL + s));
        return true;
      };
      Task k = read_task(p, walk, t_begin);
      for (int t = t_begin; ok && t < t_end; ++t) {
        const Task cur = k;
        k = read_task(p, walk, t + 1);                        // fetched one task ahead of its use
        if (!cur.valid) continue;
        const uint32_t s = n & 1, slot = n % QRING, use = n / QRING;
        if (cur.group != cur_group || cur.block != cur_block) {
          cur_group = cur.group; cur_block = cur.block;
          // the old block is done with once the last PV on it has completed
          if (pv_pending) {
            ok = issue_pv(n - 1);
            pv_pending = false;
            if (!ok) break;
          }
          if (loads > 0) tc_commit(bar(KV_EMPTY));
          ok = mbar_wait(bar(KV_FULL), loads & 1, guard, 0x740);
          ++loads;
          if (!ok) break;
        }
        ok = mbar_wait(bar(Q_FULL + slot), use & 1, guard, 0x750 + slot);
        if (!ok) break;
        tc_fence_after();
        {
          const uint64_t a0 = desc_sw128_kmajor(base + OFF_Q + slot * TILE_BYTES);
          const uint64_t b0 = desc_sw128_kmajor(base + OFF_KV);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t step = static_cast<uint64_t>((kk >> 2) * (PANEL_BYTES >> 4) + (kk & 3) * 2);
            mma_ss(tmem + s * 128, a0 + step, b0 + step, IDESC_QK, kk > 0);
          }
        }
        tc_commit(bar(S_FULL + s));
        tc_commit(bar(Q_EMPTY + slot));
        if (pv_pending) {
          ok = issue_pv(n - 1);
          if (!ok) break;
        }
        pv_pending = true;
        ++n;
      }
      if (ok && pv_pending) issue_pv(n - 1);
    }
    __syncwarp();
  }
  } else if (warp < EPI_WARP0) {
    // ------------------------------------------------------------- softmax
    setmaxnreg_inc<SOFTMAX_REGS>();
    const uint32_t s = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + s * 128;
    uint32_t n = 0;
    bool ok = true;
    for (int t = t_begin; ok && t < t_end; ++t) {
      const Task k = read_task(p, walk, t);
      if (!k.valid) continue;
      const uint32_t mine = (n & 1) == s, u = n >> 1;
      ++n;
      if (!mine) continue;
      // where this row's LSE goes (fetched before the scores are ready)
      long long lse_at = -1;
      {
        const int tl = row >> p.group_log2, g = row & (G - 1);
        if (tl < k.count) {
          const int qi = p.qids[k.start + tl], rank = p.ranks[k.start + tl];
          if (qi >= 0 && qi < p.sq && rank >= 0 && rank < p.topk) {
            const int b = k.group / p.hkv, kvh = k.group - b * p.hkv;
            lse_at = ((static_cast<long long>(b) * p.hq + kvh * G + g) * p.sq + qi) * p.topk + rank;
          }
        }
      }
      bool w = mbar_wait(bar(S_FULL + s), u & 1, guard, 0x760 + s);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, sv[c]);
      tc_wait_ld();
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          mx[(j >> 1) & 3] = max3(mx[(j >> 1) & 3], __uint_as_float(sv[c][j]), __uint_as_float(sv[c][j + 1]));
      const float row_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
      float2 part[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg2 = make_float2(-row_max, -row_max);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 x =
              fma2(make_float2(__uint_as_float(sv[c][2 * j]), __uint_as_float(sv[c][2 * j + 1])), scale2, neg2);
          const float2 e = make_float2(ex2_approx(x.x), ex2_approx(x.y));
          part[j & 1] = add2(part[j & 1], e);
          pk[j] = pack_bf16x2(e.x, e.y);
        }
        tmem_st16(t_s + c * 16, pk);
      }
      const float row_sum = (part[0].x + part[0].y) + (part[1].x + part[1].y);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL + s));
      // 1 / row sum to the epilogue warps (after they released the previous task's)
      if (u > 0) {
        bool w2 = mbar_wait(bar(STATS_EMPTY + s), (u - 1) & 1, guard, 0x770 + s);
        ok = __all_sync(0xffffffffu, w2);
        if (!ok) break;
      }
      stats[s * 128 + row] = 1.0f / row_sum;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(STATS_FULL + s));
      if (lse_at >= 0) p.lses[lse_at] = (row_max + log2f(row_sum)) * 0.6931471805599453f;
    }
  } else {
    // ------------------------------------------------------------- epilogue warps
    setmaxnreg_dec<EPI_REGS>();
    const int quarter = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t stage = base + OFF_STAGE + quarter * STAGE_BYTES;
    unsigned char* stage_g = gbase + OFF_STAGE + quarter * STAGE_BYTES;
    const int per_warp = 32 >> p.group_log2;       // queries whose heads this warp holds
    uint32_t n = 0;
    bool ok = true;
    for (int t = t_begin; ok && t < t_end; ++t) {
      const Task k = read_task(p, walk, t);
      if (!k.valid) continue;
      const uint32_t s = n & 1, u = n >> 1;
      ++n;
      // lane l < per_warp owns query quarter * per_warp + l of the task
      int qi = -1, rank = -1;
      {
        const int tl = quarter * per_warp + lane;
        if (lane < per_warp && tl < k.count) {
          qi = p.qids[k.start + tl];
          rank = p.ranks[k.start + tl];
          if (qi < 0 || qi >= p.sq || rank < 0 || rank >= p.topk) qi = rank = -1;
        }
      }
      bool w = mbar_wait(bar(STATS_FULL + s), u & 1, guard, 0x780 + s);
      w = mbar_wait(bar(O_FULL + s), u & 1, guard, 0x790 + s) && w;
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      const float inv = stats[s * 128 + quarter * 32 + lane];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(STATS_EMPTY + s));
      const uint32_t t_o = tmem + lane_base + 256 + s * 128;
      if constexpr (F32) {
        // fp32 partials: lane = row (query lane / G, head lane % G) writes its 512 bytes from tensor memory
        const int owner = lane >> p.group_log2, g = lane & (G - 1);
        const int row_q = __shfl_sync(0xffffffffu, qi, owner), row_rank = __shfl_sync(0xffffffffu, rank, owner);
        const int b = k.group / p.hkv, head = (k.group - b * p.hkv) * G + g;
        const long long row =
            p.partial_token_major
                ? ((static_cast<long long>(b) * p.sq + row_q) * p.topk + row_rank) * p.hq + head
                : ((static_cast<long long>(b) * p.hq + head) * p.sq + row_q) * p.topk + row_rank;
        float4* dst = reinterpret_cast<float4*>(p.partial_f32 + (row_q >= 0 ? row : 0) * 128);
#pragma unroll 1
        for (int cc = 0; cc < 8; ++cc) {
          uint32_t ov[16];
          tmem_ld16(t_o + cc * 16, ov);
          tc_wait_ld();
          if (row_q >= 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              dst[cc * 4 + j] = make_float4(__uint_as_float(ov[4 * j]) * inv, __uint_as_float(ov[4 * j + 1]) * inv,
                                            __uint_as_float(ov[4 * j + 2]) * inv, __uint_as_float(ov[4 * j + 3]) * inv);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(O_EMPTY + s));
        continue;
      }
      bulk_wait_read0();                             // this lane's earlier stores have left the staging tile
      __syncwarp();
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t ov[32];
        tmem_ld32(t_o + cc * 32, ov);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 val = make_uint4(
              pack_bf16x2(__uint_as_float(ov[8 * j]) * inv, __uint_as_float(ov[8 * j + 1]) * inv),
              pack_bf16x2(__uint_as_float(ov[8 * j + 2]) * inv, __uint_as_float(ov[8 * j + 3]) * inv),
              pack_bf16x2(__uint_as_float(ov[8 * j + 4]) * inv, __uint_as_float(ov[8 * j + 5]) * inv),
              pack_bf16x2(__uint_as_float(ov[8 * j + 6]) * inv, __uint_as_float(ov[8 * j + 7]) * inv));
          *reinterpret_cast<uint4*>(stage_g + (cc >> 1) * 4096 + lane * 128 +
                                    ((((cc & 1) * 4 + j) ^ (lane & 7)) << 4)) = val;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(O_EMPTY + s));
      fence_async_smem();
      __syncwarp();
      if (qi >= 0) {
        const int b = k.group / p.hkv, kvh = k.group - b * p.hkv;
        const uint32_t src = stage + lane * G * 128;
        if (p.partial_token_major) {              // box {64 columns, G heads, 1 rank, 1 token}
          tma_store_4d(&o_map, 0, kvh * G, rank, b * p.sq + qi, src);
          tma_store_4d(&o_map, 64, kvh * G, rank, b * p.sq + qi, src + 4096);
        } else {
          tma_store_4d(&o_map, 0, rank, qi, b * p.hq + kvh * G, src);
          tma_store_4d(&o_map, 64, rank, qi, b * p.hq + kvh * G, src + 4096);
        }
        bulk_commit();
      }
    }
    bulk_wait_all();                                 // output stores of this lane have completed
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace kvp

// Pipelined main stage for Hq / Hkv of 8 or 16 (arguments of launch_kv_token_main; q_token_major bit 0:
// q is [B, Sq, Hq, 128] instead of [B, Hq, Sq, 128]; bit 1: the partials are [B, Sq, TopK, Hq, 128]
// instead of [B, Hq, Sq, TopK, 128]; bit 2: the partials are fp32 instead of bf16).
int launch_kv_token_pipe(const void* q, const void* k, const void* v, const int32_t* tasks, const int32_t* task_count,
                         const int32_t* qids, const int32_t* ranks, void* partial, float* lses, int batch, int hq,
                         int hkv, int sq, int skv, int topk, int q_token_major, cudaStream_t stream) {
  using namespace kvp;
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  const int group = hq / hkv;
  Params p{};
  p.tasks = tasks; p.task_count = task_count; p.qids = qids; p.ranks = ranks;
  p.lses = lses;
  p.status = ctx->status;
  p.batch = batch; p.hq = hq; p.hkv = hkv; p.sq = sq; p.skv = skv; p.topk = topk; p.group = group;
  p.group_log2 = 0;
  while ((1 << p.group_log2) < group) ++p.group_log2;
  p.edges = static_cast<int>(static_cast<long long>(batch) * hkv * sq * topk);
  p.scale_log2 = 1.4426950408889634f / sqrtf(128.0f);
  p.q_token_major = q_token_major & 1;
  p.partial_token_major = (q_token_major >> 1) & 1;
  p.partial_f32 = (q_token_major & 4) ? static_cast<float*>(partial) : nullptr;
  q_token_major &= 1;
  // one segment per 24 MB of Q: the Q rows a segment gathers then stay within L2
  const long long q_bytes = static_cast<long long>(batch) * hq * sq * 256;
  p.phases = static_cast<int>(std::min<long long>(64, (q_bytes + (24LL << 20) - 1) / (24LL << 20)));

  CUtensorMap qm, km, vm, om;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  {
    const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(batch) * hkv * skv};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, 128};
    if (encode_tiled(&km, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(k), dims, strides, box, ones,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        encode_tiled(&vm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(v), dims, strides, box, ones,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for k/v");
  }
  {
    // one box = the G heads of a KV group at one token, 64 columns.
    // head-major q [B*Hq, Sq, 128]: rows Sq * 256 bytes apart; token-major q [B*Sq, Hq, 128]: one dense
    // block of G * 256 bytes (the layout of the reference's TMA variants, api11.py:1-7).
    cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(sq), static_cast<cuuint64_t>(batch) * hq};
    cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(sq) * 256};
    cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(group)};
    if (q_token_major) {
      dims[1] = static_cast<cuuint64_t>(hq); dims[2] = static_cast<cuuint64_t>(batch) * sq;
      strides[1] = static_cast<cuuint64_t>(hq) * 256;
      box[1] = static_cast<cuuint32_t>(group); box[2] = 1;
    }
    if (encode_tiled(&qm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, ones,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for q");
  }
  {
    // partial [B*Hq, Sq, TopK, 128]: one box = the G heads of a KV group at one (token, rank);
    // token-major [B*Sq, TopK, Hq, 128]: the same G rows of 64 columns, heads next to the columns
    cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(topk), static_cast<cuuint64_t>(sq),
                          static_cast<cuuint64_t>(batch) * hq};
    cuuint64_t strides[3] = {256, static_cast<cuuint64_t>(topk) * 256, static_cast<cuuint64_t>(sq) * topk * 256};
    cuuint32_t box[4] = {64, 1, 1, static_cast<cuuint32_t>(group)};
    if (p.partial_token_major) {
      dims[1] = static_cast<cuuint64_t>(hq); dims[2] = static_cast<cuuint64_t>(topk);
      dims[3] = static_cast<cuuint64_t>(batch) * sq;
      strides[0] = 256; strides[1] = static_cast<cuuint64_t>(hq) * 256;
      strides[2] = static_cast<cuuint64_t>(topk) * hq * 256;
      box[1] = static_cast<cuuint32_t>(group); box[3] = 1;
    }
    // (fp32 partials are written with plain stores: the map is encoded over the same base and never used)
    if (encode_tiled(&om, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, partial, dims, strides, box, ones,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the partial outputs");
  }
  const int slot = p.partial_f32 ? 18 : 10;
  if (!(ctx->tc_attr & (1 << slot))) {
    cudaError_t e = p.partial_f32 ? cudaFuncSetAttribute(kv_token_pipe_kernel<true>,
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES)
                                  : cudaFuncSetAttribute(kv_token_pipe_kernel<false>,
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->tc_attr |= (1 << slot);
  }
  if (p.partial_f32)
    kv_token_pipe_kernel<true><<<ctx->sm_count, NUM_THREADS, SMEM_BYTES, stream>>>(qm, km, vm, om, p);
  else
    kv_token_pipe_kernel<false><<<ctx->sm_count, NUM_THREADS, SMEM_BYTES, stream>>>(qm, km, vm, om, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
