// Q-centric block-sparse attention forward for sm_100a (B200).
//
// One persistent CTA per SM walks a static list of work items. An item is two
// query streams of 128 rows each:
//   * pair mode  (even GQA group size): two query heads of one KV-head group at
//     the same query block. They share one selection list, so every selected K
//     and V tile is fetched once and used by both streams.
//   * split mode (group size 1 or odd): two neighbouring query blocks of one
//     head, each with its own list and its own K/V tiles.
// Roles (four warpgroups, 512 threads): warps 0-3 softmax of stream 0, warps 4-7
// softmax of stream 1, warps 8-11 epilogue (read O out of tensor memory, normalise,
// TMA-store; the softmax warps go straight on to the next item), one thread of warp 12
// issues tcgen05 MMAs (waits, issue and commits in a single thread keep the
// P-ready -> MMA-issue latency short), warp 13 issues TMA loads. After the setup
// barrier setmaxnreg moves registers from the last two warpgroups to the softmax warps.
// K/V tiles selected by block index are gathered by TMA into a ring of 32 KiB
// shared-memory slots; S = QK^T and O += PV accumulate in tensor memory
// (S0,S1,O0,O1 = 512 columns); P is written back over S as packed bf16 and fed to the
// PV MMA straight from tensor memory. The ring, the Q buffers and all barriers stay
// live across items: the first QK of a stream's next item is issued right after its
// last PV, and loads of the next item overlap the tail of the current one.
//
// Replaces the reference kernels dense14_sparse_two_q_kernel
// (attention/q_centric/01_block_sparse.cu:181) and dense14_sparse_gqa_kernel
// (attention/q_centric/02_gqa_block_sparse.cu:178); adds LSE output, per-row
// block counts, 64-bit output addressing and an outer "segment" dimension used
// by the KV-centric operator and the cross-GPU KV split.
#include "ptx.cuh"
#include "internal.h"

namespace sb {
namespace qc {

constexpr int TILE = 128;            // rows per Q tile and per KV block
constexpr int HEAD_DIM = 128;
constexpr int TILE_BYTES = TILE * HEAD_DIM * 2;   // 32 KiB
constexpr int PANEL_BYTES = TILE * 128;            // 64-column half of a tile
#ifndef SB_QC_RING
#define SB_QC_RING 4
#endif
constexpr int RING = SB_QC_RING;     // K/V ring slots
constexpr int NUM_THREADS = 512;     // four warpgroups: softmax 0, softmax 1, epilogue, {MMA, TMA, 2 idle}
constexpr int EPI_WARP0 = 8;         // warps 8..11: warp w serves tensor-memory lanes 32 * (w % 4) ..
constexpr int MMA_WARP = 12;
constexpr int LOAD_WARP = 13;
// register budgets per thread after the setup barrier (setmaxnreg); 128 * (2 * 176 + 64 + 96) = 65536
constexpr int SOFTMAX_REGS = 176;
constexpr int EPI_REGS = 64;
constexpr int CTRL_REGS = 96;        // MMA issuer, TMA producer, idle warps
constexpr int TMEM_COLS = 512;
constexpr float RESCALE_LOG2 = 8.0f;   // keep a stale row max while it lags by < 2^8

// shared memory map (offsets from a 1024-aligned base)
constexpr int OFF_Q = 0;
constexpr int OFF_RING = 2 * TILE_BYTES;
constexpr int OFF_STAGE = OFF_RING + RING * TILE_BYTES;   // 4 epilogue warps x 8 KiB output staging
constexpr int STAGE_BYTES = 8192;
constexpr int OFF_STATS = OFF_STAGE + 4 * STAGE_BYTES;    // [2 streams][128 rows] 1 / row sum
constexpr int OFF_BAR = OFF_STATS + 2 * TILE * 4;
// barrier indices (8 bytes each)
constexpr int BAR_Q_FULL = 0;      // [2]
constexpr int BAR_Q_EMPTY = 2;     // [2]
constexpr int BAR_S_FULL = 4;      // [2]
constexpr int BAR_P_FULL = 6;      // [2]
constexpr int BAR_O_FULL = 8;      // [2]
constexpr int BAR_STATS_FULL = 10; // [2] softmax -> epilogue: 1 / row sum of the item is in shared memory
constexpr int BAR_O_EMPTY = 12;    // [2] epilogue -> MMA: O has been read out of tensor memory
constexpr int BAR_STATS_EMPTY = 14; // [2] epilogue -> softmax: the previous item's 1 / row sum has been read
constexpr int BAR_P_HALF = 16;     // [2] pair mode: the first three quarters of P are stored
constexpr int BAR_KV_FULL = 18;    // [RING]
constexpr int BAR_KV_EMPTY = 18 + RING;  // [RING]
constexpr int NUM_BARS = 18 + 2 * RING;
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;   // tmem base (4 B), abort flag (4 B), 8 B unused, then one
                                                   // hand-over counter per softmax warp (8 x 4 B)
constexpr int SMEM_BYTES = OFF_MISC + 48 + 1024;   // + slack for manual 1024 alignment
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory map exceeds the per-CTA limit");

struct Params {
  const int32_t* ids;      // [nseg, B, Hkv, Qt, topk]
  const int32_t* counts;   // [nseg, B, Hkv, Qt] or nullptr (= topk everywhere)
  void* out;               // [nseg, B, Hq, Sq, 128] bf16 or fp32
  float* lse;              // [nseg, B, Hq, Sq] or nullptr
  int* status;
  int batch, hq, hkv, sq, skv, topk, nseg;
  int group, qt, pair_mode;
  int items_per_seg, num_items;
  float scale_log2;
  // Tail balancing (single-segment bf16 launches with a workspace): the items of the last, partly
  // filled round (index >= tail_first) are cut into tail_parts pieces of their lists; piece v writes a
  // normalised partial (O, LSE) into the workspace and tail_merge_kernel combines the pieces.
  // num_virtual = items as the roles see them; without balancing tail_first = num_virtual = num_items.
  int tail_first, tail_parts, num_virtual;
  float* tail_lse;         // [pieces * 2 * 128]
};

struct Stream {
  bool valid;          // this stream exists (split mode, odd tile count)
  int count;           // live list entries
  const int32_t* list; // its selection list
  int q_row;           // first row in the 2-D view of Q
  int kv_row;          // first row of its KV head in the 2-D view of K/V
  long long out_row;   // first output row (64-bit: outputs may exceed 2^31 elements)
  bool tail;           // a piece of a tail item: out_row is a row of the workspace
};

__device__ __forceinline__ void decode_item(const Params& p, int virt, Stream (&s)[2]) {
  int item = virt, part = 0;
  const bool tail = virt >= p.tail_first;
  if (tail) {
    const int t = virt - p.tail_first;
    item = p.tail_first + t / p.tail_parts;
    part = t - (t / p.tail_parts) * p.tail_parts;
  }
  const int seg = item / p.items_per_seg;
  const int local = item - seg * p.items_per_seg;
  if (p.pair_mode) {
    const int pairs = p.group >> 1;
    const int pair = local % pairs;
    const int t = local / pairs;
    const int qtile = t % p.qt;
    const int bk = t / p.qt;            // batch * Hkv + kv head
    const int b = bk / p.hkv, kvh = bk - b * p.hkv;
    const long long row = (static_cast<long long>(seg) * p.batch * p.hkv + bk) * p.qt + qtile;
    const int cnt = p.counts ? p.counts[row] : p.topk;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int head = kvh * p.group + 2 * pair + q;
      const int bh = b * p.hq + head;
      s[q].valid = true;
      s[q].count = cnt;
      s[q].list = p.ids + row * p.topk;
      s[q].q_row = bh * p.sq + qtile * TILE;
      s[q].kv_row = bk * p.skv;
      s[q].out_row = (static_cast<long long>(seg) * p.batch * p.hq + bh) * p.sq + qtile * TILE;
    }
  } else {
    const int qpairs = (p.qt + 1) >> 1;
    const int qp = local % qpairs;
    const int bh = local / qpairs;      // batch * Hq + head
    const int b = bh / p.hq, head = bh - b * p.hq;
    const int kvh = head / p.group;
    const int bk = b * p.hkv + kvh;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int qtile = 2 * qp + q;
      const bool valid = qtile < p.qt;
      const long long row = (static_cast<long long>(seg) * p.batch * p.hkv + bk) * p.qt + (valid ? qtile : 0);
      s[q].valid = valid;
      s[q].count = valid ? (p.counts ? p.counts[row] : p.topk) : 0;
      s[q].list = p.ids + row * p.topk;
      s[q].q_row = bh * p.sq + qtile * TILE;
      s[q].kv_row = bk * p.skv;
      s[q].out_row = (static_cast<long long>(seg) * p.batch * p.hq + bh) * p.sq + qtile * TILE;
    }
  }
  // counts come from the caller: clamp to the list capacity
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    s[q].count = min(max(s[q].count, 0), p.topk);
    s[q].tail = tail;
    if (tail) {                                  // this piece's share of the list, its rows in the workspace
      const int lo = part * s[q].count / p.tail_parts, hi = (part + 1) * s[q].count / p.tail_parts;
      s[q].list += lo;
      s[q].count = hi - lo;
      s[q].out_row = (static_cast<long long>(virt - p.tail_first) * 2 + q) * TILE;
    }
  }
}

// Live list lengths of the two streams of an item: all the MMA issuer needs to know
// (it keeps few registers so that its wait -> issue path stays free of spills).
__device__ __forceinline__ void item_counts(const Params& p, int virt, int (&cnt)[2]) {
  int item = virt, part = 0;
  const bool tail = virt >= p.tail_first;
  if (tail) {
    const int t = virt - p.tail_first;
    item = p.tail_first + t / p.tail_parts;
    part = t - (t / p.tail_parts) * p.tail_parts;
  }
  const int seg = item / p.items_per_seg;
  const int local = item - seg * p.items_per_seg;
  if (p.pair_mode) {
    int c = p.topk;
    if (p.counts) {
      const int t = local / (p.group >> 1);          // (batch * Hkv + kv head) * Qt + query tile
      c = p.counts[static_cast<long long>(seg) * p.batch * p.hkv * p.qt + t];
    }
    cnt[0] = cnt[1] = min(max(c, 0), p.topk);
  } else {
    const int qpairs = (p.qt + 1) >> 1;
    const int bh = local / qpairs;
    const int qp = local - bh * qpairs;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int qtile = 2 * qp + q;
      int c = qtile < p.qt ? p.topk : 0;
      if (p.counts && qtile < p.qt) {
        const int b = bh / p.hq, head = bh - b * p.hq;
        const int bk = b * p.hkv + head / p.group;
        c = p.counts[(static_cast<long long>(seg) * p.batch * p.hkv + bk) * p.qt + qtile];
      }
      cnt[q] = min(max(c, 0), p.topk);
    }
  }
  if (tail) {
#pragma unroll
    for (int q = 0; q < 2; ++q) cnt[q] = (part + 1) * cnt[q] / p.tail_parts - part * cnt[q] / p.tail_parts;
  }
}

// One list cursor of the load warp: 32 ids cached across the lanes.
struct IdCursor {
  int cached;
  __device__ __forceinline__ int get(const int32_t* list, int count, int i, int lane) {
    if ((i & 31) == 0) cached = (i + lane < count) ? __ldg(list + i + lane) : 0;
    return __shfl_sync(0xffffffffu, cached, i & 31);
  }
};

// Scatter launches (one segment, bf16): the flattened [B*Hq*Sq] rows are cut into `slices` equal runs of
// slice_tiles 128-row tiles; slice 0 goes to (out, lse) through o_map, slice j > 0 to (out[j-1], lse[j-1]) through
// m[j-1] - memory that may belong to another GPU and be mapped into this process (the KV-range split across
// GPUs: every finished tile travels to the rank that merges it while the kernel computes the next ones).
// A kernel parameter of its own, and an instantiation of its own, so that the ordinary launch keeps its
// parameter block and register allocation.
constexpr int MAX_SLICES = 4;
struct ScatterOn {
  CUtensorMap m[MAX_SLICES - 1];
  void* out[MAX_SLICES - 1];
  float* lse[MAX_SLICES - 1];
  int slices, slice_tiles;
};
struct ScatterOff {};

// slice of the tile that starts at out_row; out_row becomes the row within the slice
__device__ __forceinline__ int slice_of(const ScatterOn& sc, long long& out_row) {
  const int tile = static_cast<int>(out_row >> 7);            // 32-bit arithmetic on tile numbers, no division
  const int d = (tile >= sc.slice_tiles ? 1 : 0) + (tile >= 2 * sc.slice_tiles ? 1 : 0) + (tile >= 3 * sc.slice_tiles ? 1 : 0);
  out_row = static_cast<long long>(tile - d * sc.slice_tiles) << 7;
  return d;
}
__device__ __forceinline__ int slice_of(const ScatterOff&, long long&) { return 0; }

template <bool OUT_F32, typename Scatter>
__global__ void __launch_bounds__(NUM_THREADS, 1)
q_centric_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                 const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap o_map,
                 const __grid_constant__ CUtensorMap o_tail_map, const Params p,
                 const __grid_constant__ Scatter sc) {
  constexpr bool SCATTER = sizeof(Scatter) > 1;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(gbase + OFF_MISC);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Guard guard{misc + 1, p.status};

  if (threadIdx.x == 0) {
    misc[1] = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_Q_FULL + i), 1);
      mbar_init(bar(BAR_Q_EMPTY + i), 1);
      mbar_init(bar(BAR_S_FULL + i), 1);
      mbar_init(bar(BAR_P_FULL + i), 4);   // one arrival per softmax warp
      mbar_init(bar(BAR_O_FULL + i), 1);
      mbar_init(bar(BAR_P_HALF + i), 4);
      mbar_init(bar(BAR_STATS_FULL + i), 4);
      mbar_init(bar(BAR_O_EMPTY + i), 4);
      mbar_init(bar(BAR_STATS_EMPTY + i), 4);
    }
    for (int i = 0; i < RING; ++i) {
      mbar_init(bar(BAR_KV_FULL + i), 1);
      mbar_init(bar(BAR_KV_EMPTY + i), 1);
    }
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), TMEM_COLS);
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
  float* stats = reinterpret_cast<float*>(gbase + OFF_STATS);
  // tensor memory columns: S0 0..127, S1 128..255, O0 256..383, O1 384..511.
  // P (bf16 pairs) overwrites columns 0..63 of its S.

  if (warp >= MMA_WARP) {
  // fourth warpgroup: MMA issuer, TMA producer and two idle warps share one register budget
  setmaxnreg_dec<CTRL_REGS>();
  if (warp == LOAD_WARP) {
    // ------------------------------------------------------------- TMA producer
    uint32_t fills = 0;            // tiles pushed into the ring so far
    uint32_t qloads[2] = {0, 0};
    bool ok = true;
    auto push = [&](const CUtensorMap* map, int row) -> bool {
      const uint32_t slot = fills % RING, use = fills / RING;
      if (use > 0) {
        bool w = mbar_wait(bar(BAR_KV_EMPTY + slot), (use - 1) & 1, guard, 0x100 + slot);
        if (!__all_sync(0xffffffffu, w)) return false;
      }
      if (lane == 0) {
        const uint32_t dst = base + OFF_RING + slot * TILE_BYTES;
        mbar_expect_tx(bar(BAR_KV_FULL + slot), TILE_BYTES);
        tma_load_2d(dst, map, 0, row, bar(BAR_KV_FULL + slot));
        tma_load_2d(dst + PANEL_BYTES, map, 64, row, bar(BAR_KV_FULL + slot));
      }
      ++fills;
      return true;
    };
    auto push_q = [&](int q, int row) -> bool {
      if (qloads[q] > 0) {
        bool w = mbar_wait(bar(BAR_Q_EMPTY + q), (qloads[q] - 1) & 1, guard, 0x110 + q);
        if (!__all_sync(0xffffffffu, w)) return false;
      }
      if (lane == 0) {
        const uint32_t dst = base + OFF_Q + q * TILE_BYTES;
        mbar_expect_tx(bar(BAR_Q_FULL + q), TILE_BYTES);
        tma_load_2d(dst, &q_map, 0, row, bar(BAR_Q_FULL + q));
        tma_load_2d(dst + PANEL_BYTES, &q_map, 64, row, bar(BAR_Q_FULL + q));
      }
      ++qloads[q];
      return true;
    };
    // Token order (must mirror the MMA warp): the first K tile of a stream's NEXT item
    // (and its Q tile) follows that stream's last V tile of the current item, so the
    // next item's first QK can be issued before the current item has drained.
    bool primed[2] = {false, false};
    for (int item = blockIdx.x; ok && item < p.num_virtual; item += gridDim.x) {
      Stream s[2], nx[2];
      decode_item(p, item, s);
      const bool has_next = item + static_cast<int>(gridDim.x) < p.num_virtual;
      if (has_next) decode_item(p, item + gridDim.x, nx);
      IdCursor kc[2], vc[2], nc[2];
      kc[0].cached = kc[1].cached = vc[0].cached = vc[1].cached = nc[0].cached = nc[1].cached = 0;
      if (p.pair_mode) {
        const int n = s[0].count;
        const bool was_primed = primed[0];
        primed[0] = primed[1] = false;
        if (n == 0) continue;
        if (!was_primed) {
          ok = push_q(0, s[0].q_row) && push_q(1, s[1].q_row) &&
               push(&k_map, s[0].kv_row + kc[0].get(s[0].list, n, 0, lane) * TILE);
        } else {
          kc[0].get(s[0].list, n, 0, lane);      // keep the cursor in step
        }
        for (int i = 0; ok && i < n; ++i) {
          ok = push(&v_map, s[0].kv_row + vc[0].get(s[0].list, n, i, lane) * TILE);
          if (!ok) break;
          if (i + 1 < n) {
            ok = push(&k_map, s[0].kv_row + kc[0].get(s[0].list, n, i + 1, lane) * TILE);
          } else if (has_next && nx[0].count > 0) {
            ok = push_q(0, nx[0].q_row) &&
                 push(&k_map, nx[0].kv_row + nc[0].get(nx[0].list, nx[0].count, 0, lane) * TILE) &&
                 push_q(1, nx[1].q_row);
            primed[0] = primed[1] = true;
          }
        }
      } else {
        bool was_primed[2] = {primed[0], primed[1]};
        primed[0] = primed[1] = false;
        for (int q = 0; ok && q < 2; ++q)
          if (s[q].count > 0) {
            if (!was_primed[q])
              ok = push_q(q, s[q].q_row) &&
                   push(&k_map, s[q].kv_row + kc[q].get(s[q].list, s[q].count, 0, lane) * TILE);
            else
              kc[q].get(s[q].list, s[q].count, 0, lane);
          }
        const int n = max(s[0].count, s[1].count);
        for (int i = 0; ok && i < n; ++i)
          for (int q = 0; ok && q < 2; ++q)
            if (i < s[q].count) {
              ok = push(&v_map, s[q].kv_row + vc[q].get(s[q].list, s[q].count, i, lane) * TILE);
              if (!ok) break;
              if (i + 1 < s[q].count) {
                ok = push(&k_map, s[q].kv_row + kc[q].get(s[q].list, s[q].count, i + 1, lane) * TILE);
              } else if (has_next && nx[q].count > 0) {
                ok = push_q(q, nx[q].q_row) &&
                     push(&k_map, nx[q].kv_row + nc[q].get(nx[q].list, nx[q].count, 0, lane) * TILE);
                primed[q] = true;
              }
            }
      }
    }
    if (!ok) {
      // Let copies already in flight land before the CTA gives up its shared memory.
      for (uint32_t f = (fills > RING ? fills - RING : 0); f < fills; ++f)
        mbar_wait_drain(bar(BAR_KV_FULL + f % RING), (f / RING) & 1);
      for (int q = 0; q < 2; ++q)
        if (qloads[q] > 0) mbar_wait_drain(bar(BAR_Q_FULL + q), (qloads[q] - 1) & 1);
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------- MMA issuer (one thread)
    if (lane == 0) {
    constexpr uint32_t IDESC_QK = idesc_bf16(TILE, TILE, false);
    constexpr uint32_t IDESC_PV = idesc_bf16(TILE, HEAD_DIM, true);
    uint32_t taken = 0;            // ring tiles consumed so far
    uint32_t qtaken[2] = {0, 0};
    uint32_t pphase[2] = {0, 0};
    bool ok = true;
    auto acquire = [&](uint32_t& slot) -> bool {
      slot = taken % RING;
      bool w = mbar_wait(bar(BAR_KV_FULL + slot), (taken / RING) & 1, guard, 0x200 + slot);
      ++taken;
      tc_fence_after();
      return w;
    };
    auto wait_q = [&](int q) -> bool {
      bool w = mbar_wait(bar(BAR_Q_FULL + q), qtaken[q] & 1, guard, 0x210 + q);
      ++qtaken[q];
      tc_fence_after();
      return w;
    };
    auto wait_p = [&](int q) -> bool {
      bool w = mbar_wait(bar(BAR_P_FULL + q), pphase[q], guard, 0x220 + q);
      pphase[q] ^= 1;
      tc_fence_after();
      return w;
    };
    // S_q = Q_q K^T : 8 MMAs of K = 16 over two 64-column panels.
    auto issue_qk = [&](int q, uint32_t slot) {
      {
        const uint64_t a0 = desc_sw128_kmajor(base + OFF_Q + q * TILE_BYTES);
        const uint64_t b0 = desc_sw128_kmajor(base + OFF_RING + slot * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t step = static_cast<uint64_t>((kk >> 2) * (PANEL_BYTES >> 4) + (kk & 3) * 2);
          mma_ss(tmem + q * TILE, a0 + step, b0 + step, IDESC_QK, kk > 0);
        }
      }
    };
    // O_q (+)= P_q V : A from tensor memory (8 columns per K = 16), B = V MN-major.
    auto issue_pv_part = [&](int q, uint32_t slot, bool accumulate, int k0, int k1) {
      {
        const uint64_t b0 = desc_sw128_mnmajor(base + OFF_RING + slot * TILE_BYTES, PANEL_BYTES, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          if (kk >= k0 && kk < k1)
            mma_ts(tmem + 256 + q * HEAD_DIM, tmem + q * TILE + kk * 8,
                   b0 + static_cast<uint64_t>(kk * (2048 >> 4)), IDESC_PV, (accumulate || kk > 0) ? 1u : 0u);
      }
    };
    uint32_t o_done[2] = {0, 0};   // items of each stream whose O went to the epilogue warps
    // Pair mode starts PV on the first three quarters of P while the softmax warps finish
    // the last one (measured: -5 % on GQA shapes; in split mode the extra wait of the
    // in-order issuer costs more than the early start gains, +3 %).
    uint32_t hphase[2] = {0, 0};
    auto pv = [&](int q, uint32_t slot, bool accumulate) -> bool {
      if (p.pair_mode) {
        if (!mbar_wait(bar(BAR_P_HALF + q), hphase[q], guard, 0x230 + q)) return false;
        hphase[q] ^= 1;
        tc_fence_after();
      } else if (!wait_p(q)) {
        return false;
      }
      if (!accumulate && o_done[q] > 0) {
        // the first PV of an item overwrites O: the previous item's O must have been read out
        if (!mbar_wait(bar(BAR_O_EMPTY + q), (o_done[q] - 1) & 1, guard, 0x240 + q)) return false;
        tc_fence_after();
      }
      if (p.pair_mode) {
        issue_pv_part(q, slot, accumulate, 0, 6);
        if (!wait_p(q)) return false;
        issue_pv_part(q, slot, accumulate, 6, 8);
      } else {
        issue_pv_part(q, slot, accumulate, 0, 8);
      }
      return true;
    };
    auto commit_o = [&](int q) { tc_commit(bar(BAR_O_FULL + q)); ++o_done[q]; };
    auto commit = [&](int b) { tc_commit(bar(b)); };

    bool primed[2] = {false, false};
    int cnt[2] = {0, 0}, ncnt[2] = {0, 0};
    if (static_cast<int>(blockIdx.x) < p.num_virtual) item_counts(p, blockIdx.x, ncnt);
    for (int item = blockIdx.x; ok && item < p.num_virtual; item += gridDim.x) {
      cnt[0] = ncnt[0]; cnt[1] = ncnt[1];
      const bool has_next = item + static_cast<int>(gridDim.x) < p.num_virtual;
      if (has_next) item_counts(p, item + gridDim.x, ncnt);
      uint32_t kslot = 0, vslot = 0;
      if (p.pair_mode) {
        const int n = cnt[0];
        const bool was_primed = primed[0];
        primed[0] = primed[1] = false;
        if (n == 0) continue;
        if (!was_primed) {
          ok = wait_q(0) && wait_q(1) && acquire(kslot);
          if (!ok) break;
          issue_qk(0, kslot); commit(BAR_S_FULL + 0);
          issue_qk(1, kslot); commit(BAR_S_FULL + 1);
          commit(BAR_KV_EMPTY + kslot);
          if (n == 1) { commit(BAR_Q_EMPTY + 0); commit(BAR_Q_EMPTY + 1); }
        }
        for (int i = 0; ok && i < n; ++i) {
          const bool more = i + 1 < n;
          const bool prime = !more && has_next && ncnt[0] > 0;
          ok = acquire(vslot) && pv(0, vslot, i > 0);
          if (!ok) break;
          if (more) {
            ok = acquire(kslot);
            if (!ok) break;
            issue_qk(0, kslot); commit(BAR_S_FULL + 0);
          } else {
            commit_o(0);
            if (prime) {              // first QK of the next item, stream 0
              ok = wait_q(0) && acquire(kslot);
              if (!ok) break;
              issue_qk(0, kslot); commit(BAR_S_FULL + 0);
            }
          }
          ok = pv(1, vslot, i > 0);
          if (!ok) break;
          commit(BAR_KV_EMPTY + vslot);
          if (more) {
            issue_qk(1, kslot); commit(BAR_S_FULL + 1);
            commit(BAR_KV_EMPTY + kslot);
            if (i + 2 == n) { commit(BAR_Q_EMPTY + 0); commit(BAR_Q_EMPTY + 1); }
          } else {
            commit_o(1);
            if (prime) {              // and stream 1, same K tile
              ok = wait_q(1);
              if (!ok) break;
              issue_qk(1, kslot); commit(BAR_S_FULL + 1);
              commit(BAR_KV_EMPTY + kslot);
              if (ncnt[0] == 1) { commit(BAR_Q_EMPTY + 0); commit(BAR_Q_EMPTY + 1); }
              primed[0] = primed[1] = true;
            }
          }
        }
      } else {
        bool was_primed[2] = {primed[0], primed[1]};
        primed[0] = primed[1] = false;
        for (int q = 0; ok && q < 2; ++q)
          if (cnt[q] > 0 && !was_primed[q]) {
            ok = wait_q(q) && acquire(kslot);
            if (!ok) break;
            issue_qk(q, kslot); commit(BAR_S_FULL + q);
            commit(BAR_KV_EMPTY + kslot);
            if (cnt[q] == 1) commit(BAR_Q_EMPTY + q);
          }
        const int n = max(cnt[0], cnt[1]);
        for (int i = 0; ok && i < n; ++i)
          for (int q = 0; ok && q < 2; ++q)
            if (i < cnt[q]) {
              ok = acquire(vslot) && pv(q, vslot, i > 0);
              if (!ok) break;
              commit(BAR_KV_EMPTY + vslot);
              if (i + 1 < cnt[q]) {
                ok = acquire(kslot);
                if (!ok) break;
                issue_qk(q, kslot); commit(BAR_S_FULL + q);
                commit(BAR_KV_EMPTY + kslot);
                if (i + 2 == cnt[q]) commit(BAR_Q_EMPTY + q);
              } else {
                commit_o(q);
                if (has_next && ncnt[q] > 0) {     // first QK of this stream's next item
                  ok = wait_q(q) && acquire(kslot);
                  if (!ok) break;
                  issue_qk(q, kslot); commit(BAR_S_FULL + q);
                  commit(BAR_KV_EMPTY + kslot);
                  if (ncnt[q] == 1) commit(BAR_Q_EMPTY + q);
                  primed[q] = true;
                }
              }
            }
      }
    }
    }
    __syncwarp();
  }
  } else if (warp < EPI_WARP0) {
    // ------------------------------------------------------------- softmax
    setmaxnreg_inc<SOFTMAX_REGS>();
    const int q = warp >> 2;                       // stream
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + q * TILE;
    const uint32_t t_o = tmem + lane_base + 256 + q * HEAD_DIM;
    uint32_t sphase = 0;
    // items of this stream handed to the epilogue warps so far: kept in shared memory, it is
    // touched once per item and would otherwise occupy a register across the softmax loop
    volatile int* handed_ptr = misc + 4 + warp;
    if (lane == 0) *handed_ptr = 0;
    __syncwarp();
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_virtual; item += gridDim.x) {
      Stream s[2];
      decode_item(p, item, s);
      const Stream& me = s[q];
      if (!me.valid) continue;
      // (scatter launches look their destination up where they store, after the loop: nothing more to keep in
      // registers while the softmax runs)
      const long long orow = me.out_row + row_in_tile;
      float* lse_dst = me.tail ? p.tail_lse : p.lse;
      if (me.count == 0) {
        // empty list: neutral element of the log-sum-exp merge
        if (me.tail) {                           // an empty piece: only its weight matters to the merge
          lse_dst[orow] = -INFINITY;
          continue;
        }
        void* out_base = p.out;
        long long zrow = orow;
        float* zlse = p.lse;
        if constexpr (SCATTER) {
          long long tile_row = me.out_row;
          const int slice = slice_of(sc, tile_row);
          zrow = tile_row + row_in_tile;
          if (slice) {
            out_base = sc.out[slice - 1];
            zlse = sc.lse[slice - 1];
          }
        }
        if (OUT_F32) {
          float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out_base) + zrow * HEAD_DIM);
          for (int c = 0; c < HEAD_DIM / 4; ++c) dst[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out_base) + zrow * HEAD_DIM);
          for (int c = 0; c < HEAD_DIM / 8; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
        }
        if (zlse) zlse[zrow] = -INFINITY;
        continue;
      }
      float row_max = 0.f, row_sum = 0.f;
      for (int i = 0; i < me.count; ++i) {
        bool w = mbar_wait(bar(BAR_S_FULL + q), sphase, guard, 0x300 + q);
        sphase ^= 1;
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, sv[c]);
        tc_wait_ld();
        // four independent running maxima, three-input max: 64 instructions per row
        float mx[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) mx[j] = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int j = 0; j < 32; j += 2)
            mx[(j >> 1) & 3] = max3(mx[(j >> 1) & 3], __uint_as_float(sv[c][j]), __uint_as_float(sv[c][j + 1]));
        float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        tile_max *= p.scale_log2;
        // Lazy rescale: keep a stale row max while the true max is less than
        // 2^RESCALE_LOG2 above it (P stays finite in bf16, the sum in fp32).
        float factor = 1.0f;
        if (i == 0) {
          row_max = tile_max;
        } else if (tile_max - row_max > RESCALE_LOG2) {
          factor = ex2_approx(row_max - tile_max);
          row_max = tile_max;
          row_sum *= factor;
        }
        // O of this stream is idle here: the PV MMA of the previous tile was
        // issued before the QK MMA whose commit released these scores, so it
        // has completed, and the next PV waits for the arrival below.
        if (i > 0 && __any_sync(0xffffffffu, factor != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t ov[32];
            tmem_ld32(t_o + c * 32, ov);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * factor);
            tmem_st32(t_o + c * 32, ov);
          }
        }
        // p = 2^(s*scale - max): packed FMAs, exponentials on the special-function unit (moving a
        // share of them to an FMA-pipe polynomial was measured slower: the softmax warps are
        // issue-bound there).
        float2 part[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 neg_max2 = make_float2(-row_max, -row_max);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 x = fma2(make_float2(__uint_as_float(sv[c][2 * j]), __uint_as_float(sv[c][2 * j + 1])),
                                  scale2, neg_max2);
            const float2 e = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            part[j & 1] = add2(part[j & 1], e);
            pk[j] = pack_bf16x2(e.x, e.y);
          }
          tmem_st16(t_s + c * 16, pk);
          if (c == 2 && p.pair_mode) {
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(BAR_P_HALF + q));
          }
        }
        row_sum += (part[0].x + part[0].y) + (part[1].x + part[1].y);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_P_FULL + q));
      }
      if (!ok) break;
      // Hand the row statistics to the epilogue warps and go on to the next item. A list of
      // one block ends before its PV has been issued, so nothing else orders this write
      // after the epilogue of the stream's previous item: wait for its release.
      const int handed = *handed_ptr;
      if (handed > 0) {
        bool w = mbar_wait(bar(BAR_STATS_EMPTY + q), (handed - 1) & 1, guard, 0x320 + q);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
      }
      __syncwarp();
      if (lane == 0) *handed_ptr = handed + 1;
      stats[q * TILE + row_in_tile] = 1.0f / row_sum;
      if constexpr (SCATTER) {
        long long tile_row = s[q].out_row;
        const int slice = slice_of(sc, tile_row);
        float* dst = slice ? sc.lse[slice - 1] : p.lse;
        dst[tile_row + row_in_tile] = (row_max + log2f(row_sum)) * 0.6931471805599453f;
      } else {
        if (lse_dst) lse_dst[orow] = (row_max + log2f(row_sum)) * 0.6931471805599453f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_STATS_FULL + q));
    }
  } else {
    // ------------------------------------------------------------- epilogue warps
    setmaxnreg_dec<EPI_REGS>();
    // Warp w reads tensor-memory lanes 32 * (w % 4) .. + 31 of O0 and O1: normalise, stage
    // in shared memory in the 128-byte-swizzled box layout, let TMA write the rows out.
    const int quarter = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t stage = base + OFF_STAGE + quarter * STAGE_BYTES;
    unsigned char* stage_g = gbase + OFF_STAGE + quarter * STAGE_BYTES;
    uint32_t done[2] = {0, 0};
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_virtual; item += gridDim.x) {
      Stream s[2];
      decode_item(p, item, s);
#pragma unroll 1
      for (int q = 0; ok && q < 2; ++q) {
        const Stream& me = s[q];
        if (!me.valid || me.count == 0) continue;
        const uint32_t t_o = tmem + lane_base + 256 + q * HEAD_DIM;
        bool w = mbar_wait(bar(BAR_STATS_FULL + q), done[q] & 1, guard, 0x400 + q);
        w = mbar_wait(bar(BAR_O_FULL + q), done[q] & 1, guard, 0x410 + q) && w;
        ++done[q];
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        tc_fence_after();
        const float inv = stats[q * TILE + quarter * 32 + lane];
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_STATS_EMPTY + q));
        long long tile_row = me.out_row;
        const CUtensorMap* out_map = me.tail ? &o_tail_map : &o_map;
        if constexpr (SCATTER) {
          const int slice = slice_of(sc, tile_row);
          if (slice) out_map = &sc.m[slice - 1];
        }
        const int out_row32 = static_cast<int>(tile_row) + quarter * 32;
        if (lane == 0) bulk_wait_read0();            // earlier stores have left the staging tile
        __syncwarp();
        if (OUT_F32) {
          // 512 bytes per row: two rounds of two 128-byte boxes
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            if (half == 1) {
              if (lane == 0) bulk_wait_read0();
              __syncwarp();
            }
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              uint32_t ov[32];
              tmem_ld32(t_o + half * 64 + cc * 32, ov);
              tc_wait_ld();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 val = make_float4(__uint_as_float(ov[4 * j]) * inv, __uint_as_float(ov[4 * j + 1]) * inv,
                                               __uint_as_float(ov[4 * j + 2]) * inv, __uint_as_float(ov[4 * j + 3]) * inv);
                *reinterpret_cast<float4*>(stage_g + cc * 4096 + lane * 128 + ((j ^ (lane & 7)) << 4)) = val;
              }
            }
            if (half == 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar(BAR_O_EMPTY + q));
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(out_map, half * 64, out_row32, stage);
              tma_store_2d(out_map, half * 64 + 32, out_row32, stage + 4096);
              bulk_commit();
            }
          }
        } else {
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
          if (lane == 0) mbar_arrive(bar(BAR_O_EMPTY + q));
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(out_map, 0, out_row32, stage);
            tma_store_2d(out_map, 64, out_row32, stage + 4096);
            bulk_commit();
          }
        }
      }
    }
    if (lane == 0) bulk_wait_all();      // output stores of this warp have completed
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// Merge of the pieces of the tail items (see Params::tail_first): one CTA per (tail item, stream, eight
// query rows), sixteen threads per row (16 bytes each: coalesced). Many small CTAs: a thread makes two
// dependent round trips to memory (LSEs, then partial rows), so the kernel's time is that latency
// plus its launch, whatever the row count.
// out = sum_r exp(L_r - L) O_r / sum_r exp(L_r - L), L = logsumexp_r L_r, pieces in order; a piece with
// L_r = -inf (empty share of the list) has weight 0 whatever it holds. Launched as a programmatic
// dependent of the attention kernel: its prologue overlaps that kernel's tail.
__global__ void __launch_bounds__(128) tail_merge_kernel(const Params p, const __nv_bfloat16* __restrict__ tail_out) {
  const int t = blockIdx.x >> 5, q = (blockIdx.x >> 4) & 1;
  Params real = p;
  real.tail_first = p.num_items;                 // decode the item itself, not a piece of it
  Stream s[2];
  decode_item(real, p.tail_first + t, s);
  asm volatile("griddepcontrol.wait;" ::: "memory");      // the attention kernel's stores are visible from here on
  if (!s[q].valid) return;
  const int part16 = threadIdx.x & 15;
  {
    const int row = (blockIdx.x & 15) * 8 + (threadIdx.x >> 4);
    float L[4], maximum = -INFINITY;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      L[r] = -INFINITY;
      if (r < p.tail_parts) L[r] = p.tail_lse[(static_cast<long long>(t * p.tail_parts + r) * 2 + q) * TILE + row];
      maximum = fmaxf(maximum, L[r]);
    }
    float w[4], denom = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      w[r] = (r < p.tail_parts && L[r] > -INFINITY) ? expf(L[r] - maximum) : 0.f;
      denom += w[r];
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (r < p.tail_parts && w[r] > 0.f) {
        const uint4 raw = *reinterpret_cast<const uint4*>(
            tail_out + ((static_cast<long long>(t * p.tail_parts + r) * 2 + q) * TILE + row) * HEAD_DIM + part16 * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          acc[2 * e] = fmaf(w[r], f.x, acc[2 * e]);
          acc[2 * e + 1] = fmaf(w[r], f.y, acc[2 * e + 1]);
        }
      }
    }
    const long long orow = s[q].out_row + row;
    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + orow * HEAD_DIM + part16 * 8) =
        make_uint4(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv),
                   pack_bf16x2(acc[4] * inv, acc[5] * inv), pack_bf16x2(acc[6] * inv, acc[7] * inv));
    if (part16 == 0 && p.lse) p.lse[orow] = denom > 0.f ? maximum + logf(denom) : -INFINITY;
  }
}

// ------------------------------------------------------------------ host side
// Output map: boxes of 32 rows x 128 bytes, 128-byte swizzle.
static int encode_out_map(CUtensorMap* map, void* ptr, uint64_t rows, bool f32) {
  const cuuint64_t dims[2] = {HEAD_DIM, rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(HEAD_DIM) * (f32 ? 4 : 2)};
  const cuuint32_t box[2] = {f32 ? 32u : 64u, 32};
  const cuuint32_t steps[2] = {1, 1};
  return encode_tiled(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims,
                      strides, box, steps, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE);
}

static int encode_rows_map(CUtensorMap* map, const void* ptr, uint64_t rows) {
  const cuuint64_t dims[2] = {HEAD_DIM, rows};
  const cuuint64_t strides[1] = {HEAD_DIM * 2};
  const cuuint32_t box[2] = {64, TILE};
  const cuuint32_t steps[2] = {1, 1};
  return encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                      steps, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

}  // namespace qc

int launch_q_centric(const QCentricArgs& a, cudaStream_t stream) {
  using namespace qc;
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  const int group = a.hq / a.hkv;
  Params p{};
  p.ids = a.block_idx;
  p.counts = a.block_count;
  p.out = a.out;
  p.lse = a.lse;
  p.status = ctx->status;
  p.batch = a.batch; p.hq = a.hq; p.hkv = a.hkv; p.sq = a.sq; p.skv = a.skv;
  p.topk = a.topk; p.nseg = a.nseg;
  p.group = group;
  p.qt = a.sq / TILE;
  p.pair_mode = (group % 2 == 0) ? 1 : 0;
  p.items_per_seg = p.pair_mode ? a.batch * a.hkv * p.qt * (group / 2)
                                : a.batch * a.hq * ((p.qt + 1) / 2);
  p.num_items = p.items_per_seg * a.nseg;
  p.scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(HEAD_DIM));
  const int grid = p.num_items < ctx->sm_count ? p.num_items : ctx->sm_count;

  // Tail balancing. With few rounds of items per CTA the last, partly filled round costs a whole
  // round: when at most half of the CTAs would work in it, its items are cut into 2-4 pieces (as
  // many as idle CTAs allow), so that the round takes a half to a quarter of the time, and a small
  // kernel merges the pieces. Needs a workspace; single-segment bf16 launches only.
  p.tail_first = p.num_virtual = p.num_items;
  p.tail_parts = 1;
  p.tail_lse = nullptr;
  __nv_bfloat16* tail_out = nullptr;
  const int rounds = p.num_items / grid, rem = p.num_items - rounds * grid;
  if (a.tail_ws && a.owners <= 1 && a.nseg == 1 && !a.out_f32 && rem > 0 && 2 * rem <= grid && rounds >= 1 && rounds <= 8 && a.topk >= 8) {
    int parts = grid / rem;
    if (parts > 4) parts = 4;
    if (parts > a.topk / 4) parts = a.topk / 4;  // at least four blocks per piece
    const long long rows = static_cast<long long>(rem) * parts * 2 * TILE;
    const long long need = rows * (HEAD_DIM * 2 + 4) + 256;
    // worth it when the blocks a CTA no longer walks (about 1.7 us each, measured) outweigh the merge
    // (launch + the partials' round trip through memory: about 4 us + 0.1 us per tail item)
    const bool pays = parts >= 2 && 1.7f * static_cast<float>(a.topk - a.topk / parts) >= 4.f + 0.1f * static_cast<float>(rem);
    if (pays && need <= a.tail_bytes && (reinterpret_cast<uintptr_t>(a.tail_ws) & 15u) == 0) {
      p.tail_first = p.num_items - rem;
      p.tail_parts = parts;
      p.num_virtual = p.tail_first + rem * parts;
      tail_out = static_cast<__nv_bfloat16*>(a.tail_ws);
      p.tail_lse = reinterpret_cast<float*>(static_cast<unsigned char*>(a.tail_ws) + ((rows * HEAD_DIM * 2 + 255) & ~255LL));
    }
  }

  CUtensorMap qm, km, vm, om, omt;
  if (encode_rows_map(&qm, a.q, static_cast<uint64_t>(a.batch) * a.hq * a.sq) ||
      encode_rows_map(&km, a.k, static_cast<uint64_t>(a.batch) * a.hkv * a.skv) ||
      encode_rows_map(&vm, a.v, static_cast<uint64_t>(a.batch) * a.hkv * a.skv) ||
      encode_out_map(&om, a.out, static_cast<uint64_t>(a.nseg) * a.batch * a.hq * a.sq, a.out_f32 != 0))
    return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for q/k/v/out");
  omt = om;
  if (tail_out && encode_out_map(&omt, tail_out, static_cast<uint64_t>(p.num_virtual - p.tail_first) * 2 * TILE, false))
    return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for the tail workspace");

  if (a.owners > 1) {
    // scatter launch: slice j of the rows has a destination of its own (a.out / a.lse are slice 0's)
    const long long rows = static_cast<long long>(a.batch) * a.hq * a.sq;
    if (a.owners > MAX_SLICES || a.nseg != 1 || a.out_f32 || rows % a.owners || (rows / a.owners) % TILE || !a.lse)
      return set_error(SB_ERR_INVALID,
                       "scatter launches: 2 to 4 equal slices of whole 128-row tiles, one segment, bf16, LSE required");
    ScatterOn sc{};
    sc.slices = a.owners;
    sc.slice_tiles = static_cast<int>(rows / a.owners / TILE);
    if (encode_out_map(&om, a.out, static_cast<uint64_t>(rows / a.owners), false))
      return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for slice 0");
    for (int j = 1; j < MAX_SLICES; ++j) sc.m[j - 1] = om;
    for (int j = 1; j < a.owners; ++j) {
      if (!a.owner_out[j] || !a.owner_lse[j] || (reinterpret_cast<uintptr_t>(a.owner_out[j]) & 15u))
        return set_error(SB_ERR_INVALID, "every slice needs a 16-byte aligned output and an LSE pointer");
      sc.out[j - 1] = a.owner_out[j];
      sc.lse[j - 1] = a.owner_lse[j];
      if (encode_out_map(&sc.m[j - 1], a.owner_out[j], static_cast<uint64_t>(rows / a.owners), false))
        return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for a slice's destination");
    }
    if (!(ctx->tc_attr & (1 << 19))) {
      cudaError_t e = cudaFuncSetAttribute(q_centric_kernel<false, ScatterOn>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
      ctx->tc_attr |= (1 << 19);
    }
    q_centric_kernel<false, ScatterOn><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(qm, km, vm, om, om, p, sc);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  }
  auto kernel = a.out_f32 ? q_centric_kernel<true, ScatterOff> : q_centric_kernel<false, ScatterOff>;
  int& configured = a.out_f32 ? ctx->qc_attr_f32 : ctx->qc_attr_bf16;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    configured = 1;
  }
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(qm, km, vm, om, omt, p, ScatterOff{});
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  if (tail_out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.num_items - p.tail_first) * 32);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const __nv_bfloat16* tail_in = tail_out;
    e = cudaLaunchKernelEx(&cfg, tail_merge_kernel, p, tail_in);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  }
  return SB_OK;
}

}  // namespace sb
