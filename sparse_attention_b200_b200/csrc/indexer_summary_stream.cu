// Persistent, warp-specialised form of the tensor-core R1 / R4 summary selector for group
// size x representatives = 32 query descriptors per list (e.g. GQA 8:1 with R4): same block
// ids as the exact kernel (indexer_summary.cu), bit for bit.
//
// One CTA per SM walks work units = (batch, KV head, 8 query blocks). Roles:
//   warp 12       TMA producer: the 256 query descriptors of the unit (B operand, one buffer)
//                 and the key descriptor tiles (A operand, ring of two 32 KiB slots);
//   warp 13       MMA issuer: tcgen05 M128 N256 K16 x 8 per key tile into one of two 256-column
//                 TMEM accumulators (N = 256: 167 cycles per instruction against 2 x 116 at N = 128);
//   warps 0-7     epilogue: lane = key descriptor, warp >> 2 = half of the 256 columns; max over
//                 a list's 32 columns and over the R rows of a KV block -> approximate block
//                 scores, written to one of two CHUNK buffers (16 key tiles) in shared memory;
//   warps 14, 15  chunk filter: a warp keeps the candidate pools of four lists. It never sees all
//                 scores of a list at once: per chunk it keeps what can still belong to the C best
//                 (first chunk: the C-th largest by a bitwise search; later chunks: everything
//                 above the smallest key kept goes to a 256-entry pool that is cut back when it
//                 fills). After the unit's last chunk the C .. C + 16 candidates of a list are
//                 copied to the area of the settle warp that owns the list;
//   warps 8-11    settle: two lists of the unit each, as in indexer_summary_tc.cu: candidates more
//                 than 2 delta apart are ordered by their approximate scores, the others are
//                 re-scored exactly (fp32 FMAs in feature order), ranks by counting, safety test.
// Chunk buffers (epilogue -> filter) and candidate areas (filter -> settle) are the only hand-overs,
// each with a full / empty mbarrier pair, so the scoring of unit u + 1, the filtering of its
// chunks and the settling of unit u run at the same time.
// A list whose result cannot be proven (ties that reach beyond the candidates, a violated
// error bound) gets -1 as its first id; the launcher runs the exact kernel on those afterwards.
// Replaces descriptor_dot + reduce_topk (indexers/r1_r4/gpu_ops.py:19-49).
#include "summary_tc_common.cuh"
#include <climits>
// #define SB_STREAM_CLOCKS
#ifdef SB_STREAM_CLOCKS   // debug build: per-role cycle counts of two CTAs on stdout
#include <cstdio>
#define CLK(...) __VA_ARGS__
#else
#define CLK(...)
#endif

namespace sb {
namespace stc {
namespace stream {

constexpr int TILE_BYTES = 128 * 256;        // 128 key descriptors x 128 bf16
constexpr int A_PANEL = 128 * 128;
constexpr int A_STAGES = 2;
constexpr int B_BYTES = 256 * 256;           // 256 query descriptors
constexpr int B_PANEL = 256 * 128;
constexpr int SC_WORDS = 4096;               // one chunk buffer: lists x blocks of a chunk
constexpr int CAP = 256;                     // pool entries per list
constexpr int SLACK = 16;                    // a cut may keep up to C + SLACK entries (fewer search steps)
constexpr int FIN = C_MAX + SLACK;           // candidates of a list when it is settled
constexpr int QB_MAX = 8;                    // lists of a unit (GR = 32)
constexpr int NUM_THREADS = 512;
// warpgroups: epilogue, epilogue, settle, {TMA, MMA, two chunk-filter warps}
constexpr int EPI_WARPS = 8, SEL_WARP0 = 8, NSEL = 4, TMA_WARP = 12, MMA_WARP = 13, FLT_WARP0 = 14;
constexpr int LPW_MAX = QB_MAX / NSEL;       // lists per selection warp
// registers per thread after the setup barrier (setmaxnreg): 128 * (2 * 104 + 176 + 128) = 65536; the fourth
// warpgroup (roles with different code) keeps the 128 it was launched with
constexpr int EPI_REGS = 104, SEL_REGS = 176;
// per settle warp: the candidates of its lists (ids, approximate scores; written by a filter warp), exact
// scores, the list's query descriptors, work list (bytes), candidates per list and smallest key kept
constexpr int SELW_STATE = LPW_MAX * 2 * FIN + FIN + 2048 + FIN / 4;
constexpr int SELW_WORDS = SELW_STATE + 2 * LPW_MAX;

constexpr int OFF_A = 0;
constexpr int OFF_B = OFF_A + A_STAGES * TILE_BYTES;
constexpr int OFF_SC = OFF_B + B_BYTES;
constexpr int OFF_POOL = OFF_SC + 2 * SC_WORDS * 4;
constexpr int OFF_SELW = OFF_POOL + QB_MAX * CAP * 8;
constexpr int OFF_FST = OFF_SELW + NSEL * SELW_WORDS * 4;   // filter warps: fill and threshold of their pools
constexpr int OFF_BARS = OFF_FST + 2 * 2 * QB_MAX * 4;
constexpr int OFF_MISC = OFF_BARS + 192;
constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;     // + slack for the 1 KiB alignment
static_assert(SMEM_BYTES <= 232448, "shared memory");

enum { A_FULL = 0, A_EMPTY = 3, B_FULL = 6, B_EMPTY = 7, ACC_FULL = 8, ACC_EMPTY = 10, SC_FULL = 12, SC_EMPTY = 14,
       FIN_FULL = 16, FIN_EMPTY = 20 };

// Threshold for cutting n <= 512 unsigned keys (arr[j] ^ xorv) down to about C of them, one
// warp, n >= C >= 1. The keys sit in registers (up to 16 per lane); the value is found bit by
// bit from the top of the keys' range: a bit stays set when at least C keys reach the value it
// gives. The search stops early at a value that C .. C + SLACK keys reach (then all of them are
// kept: need_eq = INT_MAX); run to the end it yields the C-th largest key and `need_eq` = how
// many keys equal to it belong to the C largest.
__device__ __noinline__ unsigned warp_select_threshold(const unsigned* arr, unsigned xorv, int n, int C, int lane,
                                                          int& need_eq) {
  unsigned key[16];
  unsigned umin = 0xffffffffu, umax = 0u;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int j = lane + 32 * i;
    key[i] = j < n ? arr[j] ^ xorv : 0u;
    if (j < n) {
      umin = min(umin, key[i]);
      umax = max(umax, key[i]);
    }
  }
  umin = __reduce_min_sync(0xffffffffu, umin);
  umax = __reduce_max_sync(0xffffffffu, umax);
#pragma unroll
  for (int i = 0; i < 16; ++i) key[i] = lane + 32 * i < n ? key[i] - umin : 0u;   // 0 = padding or the smallest key
  const unsigned span = umax - umin;
  unsigned off = 0;
  for (int bit = 31 - __clz(span | 1u); bit >= 0; --bit) {
    const unsigned cand = off | (1u << bit);
    if (cand > span) continue;
    int c4[4] = {0, 0, 0, 0};                  // four short chains instead of one long one
#pragma unroll
    for (int i = 0; i < 16; ++i) c4[i & 3] += static_cast<int>(key[i] >= cand);     // cand >= 1: padding (0) does not count
    const int c = __reduce_add_sync(0xffffffffu, (c4[0] + c4[1]) + (c4[2] + c4[3]));
    if (c >= C) {
      off = cand;
      if (c <= C + SLACK) {                    // close enough: keep all keys that reach this value
        need_eq = INT_MAX;
        return umin + off;
      }
    }
  }
  int gt = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) gt += static_cast<int>(key[i] > off);
  gt = __reduce_add_sync(0xffffffffu, gt);
  need_eq = C - gt;
  return umin + off;
}

// Cuts a pool of `cnt` > C entries back to its C .. C + SLACK largest keys, in place (one warp).
// Entries are read 32 at a time before anything is written, and an entry never moves to a higher
// position, so nothing is overwritten before it has been read. Returns the smallest key kept
// (every entry dropped is at most that); `cnt` becomes the number of entries kept.
__device__ __noinline__ unsigned warp_compact_pool(int32_t* ids, unsigned* keys, int& cnt, int C, int lane) {
  int need_eq;
  const unsigned T = warp_select_threshold(keys, 0u, cnt, C, lane, need_eq);
  const unsigned lt_mask = (1u << lane) - 1u;
  int out = 0, eq_run = 0;
  for (int j0 = 0; j0 < cnt; j0 += 32) {
    const int j = j0 + lane;
    const unsigned u = j < cnt ? keys[j] : 0u;
    const int32_t id = j < cnt ? ids[j] : 0;
    const bool ge = j < cnt && u >= T, eq = ge && u == T;
    const unsigned eq_ballot = __ballot_sync(0xffffffffu, eq);
    const bool take = ge && (!eq || eq_run + __popc(eq_ballot & lt_mask) < need_eq);
    const unsigned take_ballot = __ballot_sync(0xffffffffu, take);
    eq_run += __popc(eq_ballot);
    __syncwarp();
    if (take) {
      const int pos = out + __popc(take_ballot & lt_mask);
      keys[pos] = u;
      ids[pos] = id;
    }
    out += __popc(take_ballot);
    __syncwarp();
  }
  cnt = out;
  return T;
}

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

template <int GR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
score_stream_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map, const Params p,
                    const int units) {
  constexpr int QB = 256 / GR;                 // lists of a work unit
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw);
  int* sc = reinterpret_cast<int*>(gbase + OFF_SC);                    // [2][QB][chunk_blocks] ordered ints
  const uint32_t bar0 = base + OFF_BARS;
  volatile int* misc = reinterpret_cast<volatile int*>(gbase + OFF_MISC);   // tmem base, abort
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.hq / p.hkv;
  const int n_keys = p.nt * p.r;
  const int num_tiles = (n_keys + 127) >> 7;
  const int r_log2 = 31 - __clz(p.r);          // R is 1, 2 or 4
  const int bpt_log2 = 7 - r_log2;             // KV blocks per key tile
  const int cb_log2 = 31 - __clz(SC_WORDS / QB);          // blocks of a chunk (a whole number of tiles)
  const int ch_tiles = 1 << (cb_log2 - bpt_log2);
  const int num_chunks = (num_tiles + ch_tiles - 1) / ch_tiles;
  Guard guard{misc + 1, p.status};

  if (threadIdx.x == 0) {
    misc[1] = 0;
    for (int i = 0; i < A_STAGES; ++i) {
      mbar_init(bar(A_FULL + i), 1);
      mbar_init(bar(A_EMPTY + i), 1);
    }
    mbar_init(bar(B_FULL), 1);
    mbar_init(bar(B_EMPTY), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(ACC_FULL + i), 1);
      mbar_init(bar(ACC_EMPTY + i), EPI_WARPS);
      mbar_init(bar(SC_FULL + i), EPI_WARPS);
      mbar_init(bar(SC_EMPTY + i), 2);
    }
    for (int i = 0; i < NSEL; ++i) {
      mbar_init(bar(FIN_FULL + i), 1);
      mbar_init(bar(FIN_EMPTY + i), 1);
    }
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = static_cast<uint32_t>(misc[0]);
  const int my_units = blockIdx.x < units ? (units - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;

  if (warp == TMA_WARP) {
    // ------------------------------------------------------------------ producer
    bool ok = true;
    int fills = 0;
    for (int ui = 0; ok && ui < my_units; ++ui) {
      const int unit = blockIdx.x + ui * gridDim.x;
      const int bk = unit / p.q_chunks, chunk = unit - bk * p.q_chunks;
      const int b = bk / p.hkv, kvh = bk - b * p.hkv;
      if (ui > 0) {
        bool w = mbar_wait(bar(B_EMPTY), (ui - 1) & 1, guard, 0x800);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
      }
      if (lane == 0) {
        mbar_expect_tx(bar(B_FULL), B_BYTES);
        tma_load_4d(base + OFF_B, &q_map, 0, 0, b * p.hq + kvh * group, chunk * QB, bar(B_FULL));
        tma_load_4d(base + OFF_B + B_PANEL, &q_map, 64, 0, b * p.hq + kvh * group, chunk * QB, bar(B_FULL));
      }
      // CTAs of one head walk the key tiles from different starting points, so they do not
      // all ask the L2 for the same tile at the same moment (a maximum is order-free)
      const int rot = static_cast<int>((static_cast<unsigned>(chunk) * 37u) % static_cast<unsigned>(num_tiles));
      for (int t = 0; ok && t < num_tiles; ++t, ++fills) {
        const int s = fills % A_STAGES, use = fills / A_STAGES;
        if (use > 0) {
          bool w = mbar_wait(bar(A_EMPTY + s), (use - 1) & 1, guard, 0x810 + s);
          ok = __all_sync(0xffffffffu, w);
          if (!ok) break;
        }
        if (lane == 0) {
          const uint32_t dst = base + OFF_A + s * TILE_BYTES;
          int tt = t + rot;
          if (tt >= num_tiles) tt -= num_tiles;
          const int row = bk * n_keys + tt * 128;
          mbar_expect_tx(bar(A_FULL + s), TILE_BYTES);
          tma_load_2d(dst, &k_map, 0, row, bar(A_FULL + s));
          tma_load_2d(dst + A_PANEL, &k_map, 64, row, bar(A_FULL + s));
        }
      }
    }
    if (!ok) {                                   // let the copies in flight land before the CTA exits
      for (int f = max(0, fills - A_STAGES); f < fills; ++f) mbar_wait_drain(bar(A_FULL + f % A_STAGES), (f / A_STAGES) & 1);
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issue
    const uint32_t idesc = idesc_bf16(128, 256, false);
    bool ok = true;
    int g = 0;                                   // tiles issued so far (ring slot and accumulator follow from it)
    CLK(long long w_a = 0; long long w_acc = 0; long long w_b = 0; const long long t_start = clock64();)
    for (int ui = 0; ok && ui < my_units; ++ui) {
      {
        CLK(const long long c0 = clock64();)
        bool w = mbar_wait(bar(B_FULL), ui & 1, guard, 0x820);
        CLK(w_b += clock64() - c0;)
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        tc_fence_after();
      }
      for (int t = 0; ok && t < num_tiles; ++t, ++g) {
        const int s = g % A_STAGES, acc = g & 1;
        CLK(const long long c0 = clock64();)
        bool w = mbar_wait(bar(A_FULL + s), (g / A_STAGES) & 1, guard, 0x830 + s);
        CLK(const long long c1 = clock64(); w_a += c1 - c0;)
        if (w && g >= 2) w = mbar_wait(bar(ACC_EMPTY + acc), ((g >> 1) - 1) & 1, guard, 0x840 + acc);
        CLK(w_acc += clock64() - c1;)
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint64_t a0 = desc_sw128_kmajor(base + OFF_A + s * TILE_BYTES);
          const uint64_t b0 = desc_sw128_kmajor(base + OFF_B);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t a_step = static_cast<uint64_t>((kk >> 2) * (A_PANEL >> 4) + (kk & 3) * 2);
            const uint64_t b_step = static_cast<uint64_t>((kk >> 2) * (B_PANEL >> 4) + (kk & 3) * 2);
            mma_ss(tmem + acc * 256, a0 + a_step, b0 + b_step, idesc, kk > 0);
          }
          tc_commit(bar(A_EMPTY + s));
          tc_commit(bar(ACC_FULL + acc));
          if (t == num_tiles - 1) tc_commit(bar(B_EMPTY));
        }
      }
    }
    CLK(if (lane == 0 && (blockIdx.x == 0 || blockIdx.x == 100))
          printf("cta %d mma: total %lld wait A %lld wait ACC_EMPTY %lld wait B %lld tiles %d\n", blockIdx.x,
                 clock64() - t_start, w_a, w_acc, w_b, g);)
  } else if (warp < EPI_WARPS) {
    // ------------------------------------------------------------------ epilogue
    setmaxnreg_dec<EPI_REGS>();
    const int quarter = warp & 3, half = warp >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    constexpr int LISTS_PER_HALF = 128 / GR;
    bool ok = true;
    int g = 0, h = 0;                            // tiles and chunks handled so far
    CLK(long long w_full = 0; long long w_sc = 0; const long long t_start = clock64();)
    for (int ui = 0; ok && ui < my_units; ++ui) {
      const int unit = blockIdx.x + ui * gridDim.x;
      const int bk = unit / p.q_chunks, chunk = unit - bk * p.q_chunks;
      const int rot = static_cast<int>((static_cast<unsigned>(chunk) * 37u) % static_cast<unsigned>(num_tiles));
      for (int t = 0; ok && t < num_tiles; ++t, ++g) {
        const int acc = g & 1;
        const int slot = t & (ch_tiles - 1);     // tile of the chunk
        CLK(const long long c0 = clock64();)
        bool w = mbar_wait(bar(ACC_FULL + acc), (g >> 1) & 1, guard, 0x850 + acc);
        CLK(const long long c1 = clock64(); w_full += c1 - c0;)
        if (w && slot == 0 && h >= 2) w = mbar_wait(bar(SC_EMPTY + (h & 1)), ((h >> 1) - 1) & 1, guard, 0x860 + (h & 1));
        CLK(w_sc += clock64() - c1;)
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        tc_fence_after();
        int tt = t + rot;
        if (tt >= num_tiles) tt -= num_tiles;
        const bool row_ok = tt * 128 + quarter * 32 + lane < n_keys;
        int* dst = sc + (h & 1) * SC_WORDS + (slot << bpt_log2) + ((quarter * 32 + lane) >> r_log2);
        const uint32_t t_acc = tmem + lane_base + acc * 256 + half * 128;
        auto flush = [&](int list, float val) {
          for (int d = 1; d < p.r; d <<= 1) val = fmaxf(val, __shfl_xor_sync(0xffffffffu, val, d));
          if ((lane & (p.r - 1)) == 0) dst[(half * LISTS_PER_HALF + list) << cb_log2] = row_ok ? f2ord(val) : INT_MIN;
        };
        // four batches of 32 columns through two register buffers: the next batch is in flight
        // while the maxima of the current one are taken
        float cur = -INFINITY;
        uint32_t va[32], vb[32];
        auto reduce32 = [&](const uint32_t (&v)[32], int batch) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            float m5[5];
#pragma unroll
            for (int j = 0; j < 5; ++j)
              m5[j] = max3(__uint_as_float(v[16 * c + 3 * j]), __uint_as_float(v[16 * c + 3 * j + 1]),
                           __uint_as_float(v[16 * c + 3 * j + 2]));
            const float m = fmaxf(max3(m5[0], m5[1], m5[2]), max3(m5[3], m5[4], __uint_as_float(v[16 * c + 15])));
            cur = fmaxf(cur, m);
            const int col_end = batch * 32 + (c + 1) * 16;
            if ((col_end % GR) == 0) {
              flush(col_end / GR - 1, cur);
              cur = -INFINITY;
            }
          }
        };
        tmem_ld32(t_acc, va);
        tc_wait_ld();
        tmem_ld32(t_acc + 32, vb);
        reduce32(va, 0);
        tc_wait_ld();
        tmem_ld32(t_acc + 64, va);
        reduce32(vb, 1);
        tc_wait_ld();
        tmem_ld32(t_acc + 96, vb);
        reduce32(va, 2);
        tc_wait_ld();
        tc_fence_before();                       // everything is in registers: hand the accumulator back
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(ACC_EMPTY + acc));
        reduce32(vb, 3);
        if (slot == ch_tiles - 1 || t == num_tiles - 1) {     // the chunk is complete
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(SC_FULL + (h & 1)));
          ++h;
        }
      }
    }
    CLK(if (lane == 0 && warp == 0 && (blockIdx.x == 0 || blockIdx.x == 100))
          printf("cta %d epilogue warp 0: total %lld wait ACC_FULL %lld wait SC_EMPTY %lld tiles %d\n", blockIdx.x,
                 clock64() - t_start, w_full, w_sc, g);)
  } else if (warp >= FLT_WARP0) {
    // ------------------------------------------------------------------ chunk filter (warps 14, 15)
    // Filter warp f keeps the pools of the lists of settle warps 2 f and 2 f + 1 (lists w and w + NSEL
    // of a unit belong to settle warp w). Per chunk: what can still belong to the C best of a list
    // goes to its pool; at the end of a unit the pools are cut to C .. C + SLACK candidates and
    // copied to the settle warps' areas (FIN_EMPTY / FIN_FULL barriers, one pair per settle warp).
    const int f = warp - FLT_WARP0;
    const unsigned lt_mask = (1u << lane) - 1u;
    const int C = p.cand;
    const int cb = 1 << cb_log2, bpt_mask = (1 << bpt_log2) - 1;
    const int invalid_blocks = (num_tiles << bpt_log2) - p.nt;   // rows past the end of the last key tile
    int* fst = reinterpret_cast<int*>(gbase + OFF_FST) + f * 2 * QB;   // [QB] pool fill, [QB] threshold (own lists only)
    unsigned* fst_thr = reinterpret_cast<unsigned*>(fst + QB);
    for (int x = lane; x < 2 * QB; x += 32) fst[x] = 0;
    __syncwarp();
    bool ok = true;
    int h = 0;
    CLK(long long w_sc = 0; long long w_fin = 0; long long t_hand = 0; const long long t_start = clock64();)
    for (int ui = 0; ok && ui < my_units; ++ui) {
      const int chunk = (blockIdx.x + ui * gridDim.x) % p.q_chunks;
      const int lists = min(QB, p.qt - chunk * QB);
      const int rot = static_cast<int>((static_cast<unsigned>(chunk) * 37u) % static_cast<unsigned>(num_tiles));
      for (int c = 0; ok && c < num_chunks; ++c, ++h) {
        CLK(const long long c0 = clock64();)
        bool w = mbar_wait(bar(SC_FULL + (h & 1)), (h >> 1) & 1, guard, 0x870 + (h & 1));
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        CLK(w_sc += clock64() - c0;)
        const int tiles_here = min(ch_tiles, num_tiles - c * ch_tiles);
        const int n = tiles_here << bpt_log2;    // entries of the chunk (rows past the end hold the lowest key)
        auto block_of = [&](int j) {             // KV block of entry j of this chunk
          int tt = c * ch_tiles + (j >> bpt_log2) + rot;
          if (tt >= num_tiles) tt -= num_tiles;
          return (tt << bpt_log2) + (j & bpt_mask);
        };
#pragma unroll 1
        for (int x = 0; x < QB / 2; ++x) {       // own lists: settle warps 2 f, 2 f + 1, their lists w and w + NSEL
          const int l = 2 * f + (x & 1) + (x >> 1) * NSEL;
          if (l >= lists) continue;
          const unsigned* keys = reinterpret_cast<const unsigned*>(sc + (h & 1) * SC_WORDS + l * cb);
          int32_t* pool_ids = reinterpret_cast<int32_t*>(gbase + OFF_POOL) + l * 2 * CAP;
          unsigned* pool_keys = reinterpret_cast<unsigned*>(pool_ids + CAP);
          int cnt = fst[l];
          unsigned thr_u = fst_thr[l];
          if (c == 0 && n - invalid_blocks >= C) {
            // first chunk with at least C real blocks: its best entries start the pool
            int need_eq;
            const unsigned T = warp_select_threshold(keys, 0x80000000u, n, C, lane, need_eq);
            int out = 0, eq_run = 0;
#pragma unroll 1
            for (int j0 = 0; j0 < n; j0 += 32) {
              const int j = j0 + lane;
              const unsigned u = j < n ? keys[j] ^ 0x80000000u : 0u;
              const bool ge = j < n && u >= T, eq = ge && u == T;
              const unsigned eq_ballot = __ballot_sync(0xffffffffu, eq);
              const bool take = ge && (!eq || eq_run + __popc(eq_ballot & lt_mask) < need_eq);
              const unsigned take_ballot = __ballot_sync(0xffffffffu, take);
              eq_run += __popc(eq_ballot);
              if (take) {
                const int pos = out + __popc(take_ballot & lt_mask);
                pool_ids[pos] = block_of(j);
                pool_keys[pos] = u;
              }
              out += __popc(take_ballot);
            }
            cnt = out;                           // C .. C + SLACK
            thr_u = T;
          } else {
            // later chunks: only entries above the smallest key kept so far can matter (an entry equal
            // to it is not needed: at least C entries at least as good are in the pool already)
#pragma unroll 1
            for (int j0 = 0; j0 < n; j0 += 128) {          // four groups of 32 entries per step
              unsigned u[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int j = j0 + 32 * i + lane;
                u[i] = j < n ? keys[j] ^ 0x80000000u : 0u;   // 0 never passes
              }
              const unsigned best = max(max(u[0], u[1]), max(u[2], u[3]));
              if (!__any_sync(0xffffffffu, best > thr_u)) continue;   // late in a list most steps hold nothing new
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (__ballot_sync(0xffffffffu, u[i] > thr_u) == 0u) continue;
                if (cnt + 32 > CAP) {            // the pool is full: cut it back, raise the threshold
                  __syncwarp();
                  thr_u = warp_compact_pool(pool_ids, pool_keys, cnt, C, lane);
                  __syncwarp();
                }
                const bool take = u[i] > thr_u;
                const unsigned ballot = __ballot_sync(0xffffffffu, take);
                if (take) {
                  const int pos = cnt + __popc(ballot & lt_mask);
                  pool_ids[pos] = block_of(j0 + 32 * i + lane);
                  pool_keys[pos] = u[i];
                }
                cnt += __popc(ballot);
              }
            }
          }
          __syncwarp();
          if (lane == 0) {
            fst[l] = cnt;
            fst_thr[l] = thr_u;
          }
          __syncwarp();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(SC_EMPTY + (h & 1)));
      }
      if (!ok) break;
      // the unit is complete: hand its candidates to the two settle warps
      CLK(const long long h0 = clock64(); const long long wf0 = w_fin;)
#pragma unroll 1
      for (int y = 0; ok && y < 2; ++y) {
        const int sw = 2 * f + y;
        if (ui > 0) {
          CLK(const long long c0 = clock64();)
          bool w = mbar_wait(bar(FIN_EMPTY + sw), (ui - 1) & 1, guard, 0x880 + sw);
          ok = __all_sync(0xffffffffu, w);
          if (!ok) break;
          CLK(w_fin += clock64() - c0;)
        }
        int* selw = reinterpret_cast<int*>(gbase + OFF_SELW) + sw * SELW_WORDS;
        int32_t* fin_ids = selw;
        float* fin_apx = reinterpret_cast<float*>(selw + LPW_MAX * FIN);
        int* st_nc = selw + SELW_STATE;
        unsigned* st_thr_fin = reinterpret_cast<unsigned*>(st_nc + LPW_MAX);
#pragma unroll 1
        for (int x = 0; x < QB / NSEL; ++x) {
          const int l = sw + x * NSEL;
          if (l >= lists) break;
          int32_t* pool_ids = reinterpret_cast<int32_t*>(gbase + OFF_POOL) + l * 2 * CAP;
          unsigned* pool_keys = reinterpret_cast<unsigned*>(pool_ids + CAP);
          int cnt = fst[l];
          unsigned thr_u = fst_thr[l];
          __syncwarp();
          if (cnt > C + SLACK) {
            thr_u = warp_compact_pool(pool_ids, pool_keys, cnt, C, lane);
            __syncwarp();
          }
          for (int c = lane; c < cnt; c += 32) {
            fin_ids[x * FIN + c] = pool_ids[c];
            fin_apx[x * FIN + c] = ord2f(static_cast<int>(pool_keys[c] ^ 0x80000000u)) * SCALE;
          }
          __syncwarp();
          if (lane == 0) {
            st_nc[x] = cnt;
            st_thr_fin[x] = thr_u;
            fst[l] = 0;
            fst_thr[l] = 0u;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(FIN_FULL + sw));
      }
      CLK(t_hand += clock64() - h0 - (w_fin - wf0);)
    }
    CLK(if (lane == 0 && blockIdx.x == 0)
          printf("cta 0 filter warp %d: total %lld wait SC_FULL %lld wait FIN_EMPTY %lld hand-over %lld\n", f,
                 clock64() - t_start, w_sc, w_fin, t_hand);)
  } else if (warp >= SEL_WARP0 && warp < SEL_WARP0 + NSEL) {
    // ------------------------------------------------------------------ settle (warps 8-11)
    setmaxnreg_inc<SEL_REGS>();
    static_assert(GR == 32, "a lane of a settle warp is one query descriptor of a list");
    constexpr int LPW = QB / NSEL;                 // lists of this warp: sw, sw + NSEL
    const int sw = warp - SEL_WARP0;
    int* selw = reinterpret_cast<int*>(gbase + OFF_SELW) + sw * SELW_WORDS;
    const int32_t* fin_ids = selw;                                    // [LPW][FIN] candidates of the lists being settled
    const float* fin_apx = reinterpret_cast<const float*>(selw + LPW_MAX * FIN);   // [LPW][FIN] their approximate scores
    int* ord = selw + 2 * LPW_MAX * FIN;           // [FIN] exact scores of one list's candidates (ordered ints)
    uint32_t* qs = reinterpret_cast<uint32_t*>(ord + FIN);            // [64][32] feature pairs of the list's 32 query descriptors
    unsigned char* work = reinterpret_cast<unsigned char*>(qs + 2048);     // [FIN] candidates that need an exact score
    const int* st_nc = selw + SELW_STATE;          // [LPW] candidates per list
    const unsigned* st_thr_fin = reinterpret_cast<const unsigned*>(st_nc + LPW_MAX);   // [LPW] smallest key kept
    const unsigned lt_mask = (1u << lane) - 1u;
    bool ok = true;
    CLK(long long w_full = 0; const long long t_start = clock64();)
    for (int ui = 0; ok && ui < my_units; ++ui) {
      {
        CLK(const long long c0 = clock64();)
        bool w = mbar_wait(bar(FIN_FULL + sw), ui & 1, guard, 0x890 + sw);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        CLK(w_full += clock64() - c0;)
      }
      const int unit = blockIdx.x + ui * gridDim.x;
      const int bk = unit / p.q_chunks, chunk = unit - bk * p.q_chunks;
      const int b = bk / p.hkv, kvh = bk - b * p.hkv;
      const int qtile0 = chunk * QB;
      const int lists = min(QB, p.qt - qtile0);
      const __nv_bfloat16* kbase = p.kd + static_cast<long long>(bk) * n_keys * 128;
      const float kabs = p.k_absmax[bk], knorm = sqrtf(p.k_norm2[bk]);
      const long long qrow0 = (static_cast<long long>(b) * p.hq + kvh * group) * p.qt;   // descriptor block of head 0
#pragma unroll 1
      for (int li = 0; li < LPW; ++li) {
        if (sw + li * NSEL >= lists) break;
        const int qtile = qtile0 + sw + li * NSEL;
        const int32_t* ids_l = fin_ids + li * FIN;
        const float* apx = fin_apx + li * FIN;
        const int nc = st_nc[li];                // C .. C + SLACK (all blocks when the list is shorter than C)
        const float thr = ord2f(static_cast<int>(st_thr_fin[li] ^ 0x80000000u)) * SCALE;
        // The list's 32 query descriptors go to shared memory (word i of row r at [i][r]: lane r reads
        // its own row without bank conflicts). Their L1 and L2 norms give the error bound of the
        // list: sum of |q_d k_d| bounded by Hoelder (L1 x max) and by Cauchy-Schwarz.
        {
          const int g = lane >> r_log2, rq = lane & (p.r - 1);     // descriptor = head of the group * R + representative
          const uint4* src = reinterpret_cast<const uint4*>(
              p.qd + (((qrow0 + static_cast<long long>(g) * p.qt + qtile) << r_log2) + rq) * 128);
          uint4 v[16];
#pragma unroll
          for (int cc = 0; cc < 16; ++cc) v[cc] = __ldg(src + cc);
          __syncwarp();
#pragma unroll
          for (int cc = 0; cc < 16; ++cc) {
            qs[(4 * cc) * 32 + lane] = v[cc].x;
            qs[(4 * cc + 1) * 32 + lane] = v[cc].y;
            qs[(4 * cc + 2) * 32 + lane] = v[cc].z;
            qs[(4 * cc + 3) * 32 + lane] = v[cc].w;
          }
        }
        __syncwarp();
        float s4[4] = {0.f, 0.f, 0.f, 0.f}, q4[4] = {0.f, 0.f, 0.f, 0.f};   // any order will do for a bound
#pragma unroll 4
        for (int i = 0; i < 64; ++i) {
          const uint32_t w = qs[i * 32 + lane];
          const float x = bf_lo(w), y = bf_hi(w);
          s4[i & 3] += fabsf(x) + fabsf(y);
          q4[i & 3] = fmaf(x, x, fmaf(y, y, q4[i & 3]));
        }
        float l1 = (s4[0] + s4[1]) + (s4[2] + s4[3]), l2 = (q4[0] + q4[1]) + (q4[2] + q4[3]);
        l1 = __int_as_float(__reduce_max_sync(0xffffffffu, __float_as_int(l1)));   // non-negative floats order as ints
        l2 = __int_as_float(__reduce_max_sync(0xffffffffu, __float_as_int(l2)));
        const float delta = EPS * 1.0001f * fminf(l1 * kabs, sqrtf(l2) * knorm) * SCALE;
        const float two = 2.f * delta;
        // candidates whose order the approximate scores do not settle
        int nwork = 0;
#pragma unroll 1
        for (int c0 = 0; c0 < nc; c0 += 32) {
          const int c = c0 + lane;
          bool near = false;
          if (c < nc) {
            const float a = apx[c];
#pragma unroll 4
            for (int j = 0; j < nc; ++j) near |= (j != c) & !(fabsf(a - apx[j]) > two);
            ord[c] = near ? f2ord(-INFINITY) : INT_MIN;     // INT_MIN = "no exact score": below every ordered float
          }
          const unsigned nb = __ballot_sync(0xffffffffu, near);
          if (near) work[nwork + __popc(nb & lt_mask)] = static_cast<unsigned char>(c);
          nwork += __popc(nb);
        }
        __syncwarp();
        // Exact scores: fp32 FMA chains over the features in order, from zero (the arithmetic that
        // defines a score). A lane takes an item = (four key descriptors, eight query descriptors): the
        // key rows come straight from global memory into its registers (16-byte pieces, requested one
        // piece ahead), the query values from the staging area (the four lanes of a quad read
        // different chunks, lanes of different quads the same words), 64 FMAs per 32 bytes loaded
        // from shared memory.
        const int rows = nwork << r_log2;        // key descriptors to score (R per candidate)
        const int quads = (rows + 3) >> 2;
#pragma unroll 1
        for (int item = lane; item < quads * 4; item += 32) {
          const int quad = item >> 2, qc = item & 3;
          const uint4* krow[4];
          int cand[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = min(4 * quad + j, rows - 1);       // rows past the end repeat the last one
            cand[j] = work[row >> r_log2];
            krow[j] = reinterpret_cast<const uint4*>(
                kbase + ((static_cast<long long>(ids_l[cand[j]]) << r_log2) + (row & (p.r - 1))) * 128);
          }
          float acc[4][8];
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int m = 0; m < 8; ++m) acc[j][m] = 0.f;
          uint4 cur[4], nxt[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) cur[j] = __ldg(krow[j]);
#pragma unroll 1
          for (int pc = 0; pc < 16; ++pc) {
            const int pn = pc < 15 ? pc + 1 : 15;
#pragma unroll
            for (int j = 0; j < 4; ++j) nxt[j] = __ldg(krow[j] + pn);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint4* qp = reinterpret_cast<const uint4*>(qs + (4 * pc + e) * 32 + 8 * qc);
              const uint4 qa = qp[0], qb = qp[1];
              const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
              float klo[4], khi[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t kw = e == 0 ? cur[j].x : e == 1 ? cur[j].y : e == 2 ? cur[j].z : cur[j].w;
                klo[j] = bf_lo(kw);
                khi[j] = bf_hi(kw);
              }
#pragma unroll
              for (int m = 0; m < 8; ++m) {
                const float x = bf_lo(qw[m]);
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j][m] = fmaf(x, klo[j], acc[j][m]);
              }
#pragma unroll
              for (int m = 0; m < 8; ++m) {
                const float y = bf_hi(qw[m]);
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j][m] = fmaf(y, khi[j], acc[j][m]);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float best = acc[j][0];
#pragma unroll
            for (int m = 1; m < 8; ++m) best = fmaxf(best, acc[j][m]);        // fmaxf drops a NaN unless both are
            if (best == best) atomicMax(ord + cand[j], f2ord(best));         // a NaN leaves the slot alone
          }
        }
        __syncwarp();
        // rank of a candidate = number of candidates that beat it in (exact score descending, block id
        // ascending): decided by the approximate scores when they are more than 2 delta apart, else
        // by the exact scores (both candidates have one then)
        float kth = -INFINITY;
        bool viol = false;
        int32_t* out_ids = p.ids + (static_cast<long long>(bk) * p.qt + qtile) * p.topk;
#pragma unroll 1
        for (int c0 = 0; c0 < nc; c0 += 32) {
          const int c = c0 + lane;
          if (c < nc) {
            const float a = apx[c];
            const int o = ord[c], id = ids_l[c];
            const float e = ord2f(o) * SCALE;
            if (o != INT_MIN && e == e) {        // both scores in hand: the bound must hold
              const float diff = fabsf(a - e);
              if (delta > 0.f) atomicMax(p.max_ratio, __float_as_int(diff / delta));
              if (!(diff <= delta)) {
                viol = true;
                atomicAdd(p.violations, 1);
              }
            }
            int rank = 0;
#pragma unroll 4
            for (int j = 0; j < nc; ++j) {
              const float d = apx[j] - a, ej = ord2f(ord[j]) * SCALE;
              const int gt = static_cast<int>(d > two), lt = static_cast<int>(d < -two);
              const int exact = static_cast<int>(ej > e) | (static_cast<int>(ej == e) & static_cast<int>(ids_l[j] < id));
              rank += gt | ((gt | lt) ^ 1) & exact;
            }
            if (rank < p.topk) out_ids[rank] = id;
            if (rank == p.topk - 1) kth = o != INT_MIN ? e : a - delta;   // a lower bound of the k-th exact score
          }
        }
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) kth = fmaxf(kth, __shfl_xor_sync(0xffffffffu, kth, d));
        const bool any_viol = __any_sync(0xffffffffu, viol);
        // safe: no block outside the candidates (exact score <= thr + delta) can reach the top k
        const bool safe = !any_viol && (nc >= p.nt || kth > thr + delta);
        __syncwarp();
        if (!safe && lane == 0) {
          out_ids[0] = -1;                       // the launcher's exact pass re-does this list
          if (p.fallbacks) atomicAdd(p.fallbacks, 1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(FIN_EMPTY + sw));       // the areas may be overwritten
    }
    CLK(if (lane == 0 && blockIdx.x == 0 && (sw == 0 || sw == 3))
          printf("cta 0 settle warp %d: total %lld wait FIN_FULL %lld\n", sw, clock64() - t_start, w_full);)
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int GR>
static int launch_gr(const CUtensorMap& qm, const CUtensorMap& km, const Params& p, int units, DeviceCtx* ctx, int slot,
                     cudaStream_t stream) {
  if (!(ctx->tc_attr & (1 << slot))) {
    cudaError_t e = cudaFuncSetAttribute(score_stream_kernel<GR>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->tc_attr |= (1 << slot);
  }
  const int grid = units < ctx->sm_count ? units : ctx->sm_count;
  score_stream_kernel<GR><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(qm, km, p, units);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace stream

int launch_summary_stream(const void* qd, const void* kd, Params p, int batch, DeviceCtx* ctx, cudaStream_t stream) {
  using namespace stream;
  const int group = p.hq / p.hkv, gr = group * p.r;
  if (gr != 32) return 1;                      // a lane of a selection warp = one query descriptor of a list
  if (p.r != 1 && p.r != 2 && p.r != 4) return 1;
  const int qb = 256 / gr;
  if (p.qt < qb || p.cand > C_MAX || p.cand + SLACK + 32 > CAP) return 1;
  CUtensorMap qm, km;
  {
    const cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(p.r), static_cast<cuuint64_t>(batch) * p.hq,
                                static_cast<cuuint64_t>(p.qt)};
    const cuuint64_t strides[3] = {256, static_cast<cuuint64_t>(p.qt) * p.r * 256, static_cast<cuuint64_t>(p.r) * 256};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(p.r), static_cast<cuuint32_t>(group), static_cast<cuuint32_t>(qb)};
    const cuuint32_t steps[4] = {1, 1, 1, 1};
    if (encode_tiled(&qm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(qd), dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
      return 1;
  }
  {
    const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(batch) * p.hkv * p.nt * p.r};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t steps[2] = {1, 1};
    if (encode_tiled(&km, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kd), dims, strides, box, steps,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
      return 1;
  }
  p.qb = qb;
  p.q_chunks = (p.qt + qb - 1) / qb;
  const int units = batch * p.hkv * p.q_chunks;
  return launch_gr<32>(qm, km, p, units, ctx, 17, stream);
}

}  // namespace stc
}  // namespace sb
