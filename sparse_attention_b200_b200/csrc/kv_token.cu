// KV-centric attention for per-TOKEN selection lists (the reference's KV-centric contract).
//
// A task = (KV-head group, KV block, a chunk of up to 128/G queries that selected the
// block). The CTA loads the block's K and V once by TMA, gathers the G query heads of
// every query of the chunk into a 128-row tile, computes S = QK^T (tcgen05, TMEM), a
// softmax over the single block, O = PV, and scatters the normalised partial row and
// its LSE to the slot (query, rank) the selection list gave the block. Combine
// (combine.cu, rank-inner layout) then merges the TopK partials of every query.
// Persistent CTAs walk the task list built on the GPU (metadata_token.cu); two CTAs
// share an SM (112 KiB shared memory, 256 TMEM columns each) so one CTA's softmax
// overlaps the other's MMAs.
// Same computation as kv_tma11_ops::main_kernel / kv_split9_ops::main_kernel
// (attention/kv_centric/optimization_round11/tma11_kernel.cu:97-390,
// attention/kv_centric/optimization_round9/split9_kernel.cu:79-292) for any TopK, with
// q head-major [B,Hq,Sq,128] and partials [B,Hq,Sq,TopK,128] bf16, LSE [B,Hq,Sq,TopK].
#include "ptx.cuh"
#include "internal.h"

namespace sb {
namespace kvt {

constexpr int TILE_BYTES = 128 * 256;
constexpr int PANEL_BYTES = 128 * 128;
constexpr int NUM_THREADS = 160;
constexpr int ISSUE_WARP = 4;
constexpr int OFF_Q = 0, OFF_K = TILE_BYTES, OFF_V = 2 * TILE_BYTES, OFF_STAGE = 3 * TILE_BYTES;
constexpr int OFF_DST = OFF_STAGE + 4 * 4096;        // 128 destination rows (long long)
constexpr int OFF_BAR = OFF_DST + 128 * 8;
constexpr int SMEM_BYTES = OFF_BAR + 64 + 1024;

struct Params {
  const __nv_bfloat16* q;       // [B, Hq, Sq, 128]
  const int32_t* tasks;         // [T, 4]
  const int32_t* task_count;    // -> task_ptr[rows]
  const int32_t* qids;
  const int32_t* ranks;
  __nv_bfloat16* partial;       // [B, Hq, Sq, TopK, 128]
  float* lses;                  // [B, Hq, Sq, TopK]
  int* status;
  int batch, hq, hkv, sq, skv, topk, group, group_log2, edges;
  int partial_f32;              // the partials are fp32 (the reference's fp32 control variants)
  float scale_log2;
};

__global__ void __launch_bounds__(NUM_THREADS, 2)
kv_token_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw);
  long long* dst_rows = reinterpret_cast<long long*>(gbase + OFF_DST);
  const uint32_t bar0 = base + OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(gbase + OFF_BAR + 32);   // tmem base, abort flag
  auto bar = [&](int i) { return bar0 + 8u * i; };
  enum { KV_FULL = 0, S_FULL = 1, O_FULL = 2 };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Guard guard{misc + 1, p.status};

  if (threadIdx.x == 0) {
    misc[1] = 0;
    mbar_init(bar(KV_FULL), 1);
    mbar_init(bar(S_FULL), 1);
    mbar_init(bar(O_FULL), 1);
    fence_mbar_init();
  }
  if (warp == ISSUE_WARP) {
    tmem_alloc(smem_u32(const_cast<int*>(misc)), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = static_cast<uint32_t>(misc[0]);
  const int total = *p.task_count;
  const uint32_t idesc_qk = idesc_bf16(128, 128, false);
  const uint32_t idesc_pv = idesc_bf16(128, 128, true);
  const int rows_per_chunk = 128 >> p.group_log2;      // queries per task

  // Each CTA takes a contiguous range of the task list: tasks are ordered by (group,
  // block), so consecutive tasks mostly share their K/V block and skip the reload.
  const int per_cta = (total + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int t_begin = blockIdx.x * per_cta, t_end = min(total, t_begin + per_cta);
  uint32_t phase = 0, kv_phase = 0;
  int loaded_group = -1, loaded_block = -1;
  for (int t = t_begin; t < t_end; ++t) {
    const int4 task = *reinterpret_cast<const int4*>(p.tasks + static_cast<long long>(t) * 4);
    const int group = task.x, block = task.y, start = task.z, count = task.w;
    const bool valid = group >= 0 && group < p.batch * p.hkv && block >= 0 && block < p.skv / 128 && start >= 0 &&
                       count > 0 && count <= rows_per_chunk && static_cast<long long>(start) + count <= p.edges;
    if (!valid) continue;                                   // block-uniform
    const int b = group / p.hkv, kvh = group - b * p.hkv;
    bool ok = true;
    const bool reload = group != loaded_group || block != loaded_block;
    loaded_group = group;
    loaded_block = block;
    if (warp == ISSUE_WARP) {
      if (reload && lane == 0) {
        const int kv_row = group * p.skv + block * 128;
        mbar_expect_tx(bar(KV_FULL), 2 * TILE_BYTES);
        tma_load_2d(base + OFF_K, &k_map, 0, kv_row, bar(KV_FULL));
        tma_load_2d(base + OFF_K + PANEL_BYTES, &k_map, 64, kv_row, bar(KV_FULL));
        tma_load_2d(base + OFF_V, &v_map, 0, kv_row, bar(KV_FULL));
        tma_load_2d(base + OFF_V + PANEL_BYTES, &v_map, 64, kv_row, bar(KV_FULL));
      }
    } else {
      // gather: thread = row of the Q tile = (query of the chunk, head of the group)
      const int r = threadIdx.x;
      const int tl = r >> p.group_log2, g = r & (p.group - 1);
      int qi = -1, rank = -1;
      if (tl < count) {
        qi = p.qids[start + tl];
        rank = p.ranks[start + tl];
        if (qi < 0 || qi >= p.sq || rank < 0 || rank >= p.topk) qi = rank = -1;
      }
      const int head = kvh * p.group + g;
      const long long qrow = (static_cast<long long>(b) * p.hq + head) * p.sq + (qi >= 0 ? qi : 0);
      dst_rows[r] = qi >= 0 ? qrow * p.topk + rank : -1;
      const uint4* src = reinterpret_cast<const uint4*>(p.q + qrow * 128);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 v = qi >= 0 ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
        // K-major 128-byte-swizzled operand: panel = c / 8, 16-byte chunk (c % 8) ^ (r % 8)
        *reinterpret_cast<uint4*>(gbase + OFF_Q + (c >> 3) * PANEL_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
      }
      fence_async_smem();
    }
    __syncthreads();                                         // (A) Q tile gathered, K/V requested
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float row_max = 0.f, row_sum = 1.f;
    if (warp == ISSUE_WARP) {
      bool w = true;
      if (reload) {
        w = mbar_wait(bar(KV_FULL), kv_phase, guard, 0xa00);
        kv_phase ^= 1;
      }
      ok = __all_sync(0xffffffffu, w);
      tc_fence_after();
      if (ok && lane == 0) {
        const uint64_t a0 = desc_sw128_kmajor(base + OFF_Q);
        const uint64_t b0 = desc_sw128_kmajor(base + OFF_K);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t step = static_cast<uint64_t>((kk >> 2) * (PANEL_BYTES >> 4) + (kk & 3) * 2);
          mma_ss(tmem, a0 + step, b0 + step, idesc_qk, kk > 0);
        }
        tc_commit(bar(S_FULL));
      }
    } else {
      bool w = mbar_wait(bar(S_FULL), phase, guard, 0xa10);
      ok = __all_sync(0xffffffffu, w);
      if (ok) {
        // softmax over the single block, P (bf16 pairs) back into the first 64 columns of S
        tc_fence_after();
        uint32_t sv[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tmem + lane_base + c * 32, sv[c]);
        tc_wait_ld();
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int j = 0; j < 32; j += 2)
            mx[(j >> 1) & 3] = max3(mx[(j >> 1) & 3], __uint_as_float(sv[c][j]), __uint_as_float(sv[c][j + 1]));
        row_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
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
          tmem_st16(tmem + lane_base + c * 16, pk);
        }
        row_sum = (part[0].x + part[0].y) + (part[1].x + part[1].y);
        tc_wait_st();
        tc_fence_before();
      }
    }
    __syncthreads();                                         // (B) P is in tensor memory
    if (warp == ISSUE_WARP) {
      tc_fence_after();
      if (ok && !misc[1] && lane == 0) {
        const uint64_t b0 = desc_sw128_mnmajor(base + OFF_V, PANEL_BYTES, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          mma_ts(tmem + 128, tmem + kk * 8, b0 + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_pv, kk > 0 ? 1u : 0u);
        tc_commit(bar(O_FULL));
      }
    } else if (ok && !misc[1]) {
      bool w = mbar_wait(bar(O_FULL), phase, guard, 0xa20);
      ok = __all_sync(0xffffffffu, w);
      if (ok) {
        tc_fence_after();
        const float inv = 1.0f / row_sum;
        unsigned char* stage_g = gbase + OFF_STAGE + warp * 4096;
        const long long my_dst = dst_rows[threadIdx.x];
        if (my_dst >= 0) p.lses[my_dst] = (row_max + log2f(row_sum)) * 0.6931471805599453f;
        if (p.partial_f32) {
          // fp32 partials: every thread writes its own row (512 contiguous bytes) straight from tensor memory
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.partial) + (my_dst >= 0 ? my_dst : 0) * 128);
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t ov[32];
            tmem_ld32(tmem + lane_base + 128 + cc * 32, ov);
            tc_wait_ld();
            if (my_dst >= 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                dst[cc * 8 + j] = make_float4(__uint_as_float(ov[4 * j]) * inv, __uint_as_float(ov[4 * j + 1]) * inv,
                                              __uint_as_float(ov[4 * j + 2]) * inv, __uint_as_float(ov[4 * j + 3]) * inv);
            }
          }
        } else {
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              uint32_t ov[32];
              tmem_ld32(tmem + lane_base + 128 + pass * 64 + cc * 32, ov);
              tc_wait_ld();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 val = make_uint4(
                    pack_bf16x2(__uint_as_float(ov[8 * j]) * inv, __uint_as_float(ov[8 * j + 1]) * inv),
                    pack_bf16x2(__uint_as_float(ov[8 * j + 2]) * inv, __uint_as_float(ov[8 * j + 3]) * inv),
                    pack_bf16x2(__uint_as_float(ov[8 * j + 4]) * inv, __uint_as_float(ov[8 * j + 5]) * inv),
                    pack_bf16x2(__uint_as_float(ov[8 * j + 6]) * inv, __uint_as_float(ov[8 * j + 7]) * inv));
                *reinterpret_cast<uint4*>(stage_g + lane * 128 + (((cc * 4 + j) ^ (lane & 7)) << 4)) = val;
              }
            }
            __syncwarp();
            // eight lanes write one 128-byte row segment: four destination rows per instruction
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + (lane >> 3), ch = lane & 7;
              const long long d = dst_rows[warp * 32 + rr];
              if (d >= 0) {
                const uint4 val = *reinterpret_cast<const uint4*>(stage_g + rr * 128 + ((ch ^ (rr & 7)) << 4));
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(p.partial) + d * 256 + pass * 128 + ch * 16) = val;
              }
            }
            __syncwarp();
          }
        }
        tc_fence_before();
      }
    }
    __syncthreads();                                         // (C) task done: buffers and TMEM reusable
    phase ^= 1;
    if (misc[1]) break;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == ISSUE_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace kvt

int launch_kv_token_main(const void* q, const void* k, const void* v, const int32_t* tasks, const int32_t* task_count,
                         const int32_t* qids, const int32_t* ranks, void* partial, float* lses, int batch, int hq,
                         int hkv, int sq, int skv, int topk, int partial_f32, cudaStream_t stream) {
  using namespace kvt;
  const int group = hq / hkv;
  // groups of 8 or 16 heads take the pipelined kernel (kv_token_pipe.cu); this one serves
  // the smaller groups, whose Q rows cannot be fetched as 1024-byte-aligned TMA boxes
  if (group == 8 || group == 16)
    return launch_kv_token_pipe(q, k, v, tasks, task_count, qids, ranks, partial, lses, batch, hq, hkv, sq, skv, topk,
                                partial_f32 ? 4 : 0, stream);
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  Params p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.tasks = tasks; p.task_count = task_count; p.qids = qids; p.ranks = ranks;
  p.partial = static_cast<__nv_bfloat16*>(partial);
  p.partial_f32 = partial_f32;
  p.lses = lses;
  p.status = ctx->status;
  p.batch = batch; p.hq = hq; p.hkv = hkv; p.sq = sq; p.skv = skv; p.topk = topk; p.group = group;
  p.group_log2 = 0;
  while ((1 << p.group_log2) < group) ++p.group_log2;
  p.edges = static_cast<int>(static_cast<long long>(batch) * hkv * sq * topk);
  p.scale_log2 = 1.4426950408889634f / sqrtf(128.0f);
  CUtensorMap km, vm;
  const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(batch) * hkv * skv};
  const cuuint64_t strides[1] = {256};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t steps[2] = {1, 1};
  if (encode_tiled(&km, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(k), dims, strides, box, steps,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
      encode_tiled(&vm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(v), dims, strides, box, steps,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
    return set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed for k/v");
  if (!(ctx->tc_attr & (1 << 9))) {
    cudaError_t e = cudaFuncSetAttribute(kv_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->tc_attr |= (1 << 9);
  }
  kv_token_kernel<<<ctx->sm_count * 2, NUM_THREADS, SMEM_BYTES, stream>>>(km, vm, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
