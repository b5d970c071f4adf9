// R1 / R4 summary selector for SMALL problems (few lists, few KV blocks): the same
// arithmetic as indexer_summary.cu, cut so that a problem of 64 lists fills the GPU.
//
//   pool_small_kernel   one CTA per descriptor: the 128/R token rows (contiguous in
//                       memory) are fetched into shared memory in ONE round trip by all
//                       threads, then 64 threads add them in token order (the canonical
//                       sequential fp32 sum, so the descriptors are bit-identical with
//                       pool_kernel, which keeps 16 lanes per descriptor and pays one
//                       memory round trip per 8 tokens).
//   score_cluster_kernel  a cluster of 8 CTAs per list (batch, KV head, query block).
//                       Each CTA scores chunks of key descriptors against all query
//                       descriptors of the list with a 4 x NKT register tile per thread
//                       (dot products accumulate feature by feature in fp32, as in
//                       score_topk_kernel), reduces to one score per KV block and writes
//                       it into the shared memory of the cluster's first CTA, which runs
//                       the top-k after a cluster barrier. No global workspace.
// Same results as pool_blocks / descriptor_dot / reduce_topk
// (indexers/r1_r4/gpu_ops.py:6-49): ids in score-descending order, ties to the lower id.
#include "internal.h"
#include "topk.cuh"
#include <cooperative_groups.h>
#include <cuda_bf16.h>

namespace sb {
namespace {

namespace cg = cooperative_groups;

// ---------------------------------------------------------------- pooling
// Descriptors 0 .. first - 1 come from x, the rest from x2 (queries and keys in one launch).
__global__ void __launch_bounds__(256) pool_small_kernel(const __nv_bfloat16* __restrict__ x,
                                                         __nv_bfloat16* __restrict__ desc, long long first,
                                                         const __nv_bfloat16* __restrict__ x2,
                                                         __nv_bfloat16* __restrict__ desc2, int n) {
  extern __shared__ uint4 tile[];                 // n token rows x 16 uint4
  long long vec = blockIdx.x;
  if (vec >= first) {
    vec -= first;
    x = x2;
    desc = desc2;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + vec * n * 128);
  for (int i = threadIdx.x; i < n * 16; i += blockDim.x) tile[i] = __ldcs(src + i);
  __syncthreads();
  if (threadIdx.x < 64) {
    const __nv_bfloat162* rows = reinterpret_cast<const __nv_bfloat162*>(tile) + threadIdx.x;
    float2 acc = make_float2(0.f, 0.f);
#pragma unroll 8
    for (int t = 0; t < n; ++t) {
      const float2 f = __bfloat1622float2(rows[t * 64]);
      acc.x += f.x;
      acc.y += f.y;
    }
    const float inv = 1.0f / static_cast<float>(n);
    reinterpret_cast<__nv_bfloat162*>(desc + vec * 128)[threadIdx.x] = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
  }
}

// ---------------------------------------------------------------- score + top-k
constexpr int CLUSTER = 8;

// MPAD = padded number of query descriptors (group heads x R): 16, 32 or 64.
// Thread (tq, tk) holds queries QT tq .. QT tq + QT - 1 and key descriptors NKT tk .. NKT tk + NKT - 1;
// a chunk is KD = (256 / (MPAD / QT)) * NKT key descriptors (a multiple of 4, hence of R).
template <int MPAD, int QT, int NKT>
__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(256)
score_cluster_kernel(const __nv_bfloat16* __restrict__ qd, const __nv_bfloat16* __restrict__ kd,
                     float* __restrict__ scores_out, int32_t* __restrict__ ids_out,
                     int32_t* __restrict__ fallback_counter, int hq, int hkv, int qt, int nt, int r, int topk) {
  constexpr int TQ = MPAD / QT, TK = 256 / TQ, KD = TK * NKT;
  static_assert(TQ <= 32 && (KD % 4) == 0, "query threads must fit a warp; chunks hold whole blocks");
  extern __shared__ __align__(16) float smem[];
  float* q_s = smem;                         // [128][MPAD]
  float* k_s = q_s + 128 * MPAD;             // [128][KD]
  float* kbest = k_s + 128 * KD;             // [KD]
  float* scores = kbest + KD;                // [nt]  (used in the cluster's first CTA)
  float* scratch_f = scores + nt;            // [10]
  int* scratch_i = reinterpret_cast<int*>(scratch_f + 10);

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const int list = blockIdx.x / CLUSTER;     // (b * hkv + kvh) * qt + qtile
  const int group = hq / hkv;
  const int m_real = group * r;
  const int qtile = list % qt;
  const int bk = list / qt;
  const int b = bk / hkv, kvh = bk - b * hkv;

  // query descriptors, transposed to [feature][descriptor]: thread <-> (descriptor, 16-byte piece)
  for (int e = threadIdx.x; e < MPAD * 16; e += blockDim.x) {
    const int m = e % MPAD, c = e / MPAD;
    const int mm = m < m_real ? m : 0;       // padding repeats descriptor 0: the maximum is unchanged
    const int g = mm / r, rq = mm - g * r;
    const long long row = ((static_cast<long long>(b) * hq + kvh * group + g) * qt + qtile) * r + rq;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qd + row * 128) + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float2 f = __bfloat1622float2(h[p]);
      q_s[(c * 8 + 2 * p) * MPAD + m] = f.x;
      q_s[(c * 8 + 2 * p + 1) * MPAD + m] = f.y;
    }
  }

  if (fallback_counter && blockIdx.x == 0 && threadIdx.x == 0) *fallback_counter = 0;   // every list is exact here
  cluster.sync();                              // all CTAs of the cluster run: their shared memory may be addressed
  const int n_keys = nt * r;
  const __nv_bfloat16* kbase = kd + static_cast<long long>(bk) * n_keys * 128;
  float* leader_scores = cluster.map_shared_rank(scores, 0);
  const float scale = 0.08838834764831845f;   // fp32(128^-0.5)
  const int tq = threadIdx.x % TQ, tk = threadIdx.x / TQ;

  for (int base = rank * KD; base < n_keys; base += CLUSTER * KD) {
    __syncthreads();                           // q_s staged (first pass) / k_s and kbest free again
    // stage the chunk transposed: thread <-> (key descriptor, 16-byte piece); consecutive
    // threads take consecutive descriptors, so the shared-memory stores do not conflict
    for (int e = threadIdx.x; e < KD * 16; e += blockDim.x) {
      const int kdi = e % KD, c = e / KD;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (base + kdi < n_keys) raw = __ldg(reinterpret_cast<const uint4*>(kbase + static_cast<long long>(base + kdi) * 128) + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 f = __bfloat1622float2(h[p]);
        k_s[(c * 8 + 2 * p) * KD + kdi] = f.x;
        k_s[(c * 8 + 2 * p + 1) * KD + kdi] = f.y;
      }
    }
    __syncthreads();
    float acc[QT][NKT];
#pragma unroll
    for (int i = 0; i < QT; ++i)
#pragma unroll
      for (int j = 0; j < NKT; ++j) acc[i][j] = 0.f;
#pragma unroll 8
    for (int d = 0; d < 128; ++d) {
      float qa[QT], kv[NKT];
#pragma unroll
      for (int i = 0; i < QT; ++i) qa[i] = q_s[d * MPAD + tq * QT + i];
#pragma unroll
      for (int j = 0; j < NKT; ++j) kv[j] = k_s[d * KD + tk * NKT + j];
#pragma unroll
      for (int i = 0; i < QT; ++i)
#pragma unroll
        for (int j = 0; j < NKT; ++j) acc[i][j] = fmaf(qa[i], kv[j], acc[i][j]);
    }
    // best over this thread's queries, then over the TQ threads that share the key descriptors
#pragma unroll
    for (int j = 0; j < NKT; ++j) {
      float best = acc[0][j];
#pragma unroll
      for (int i = 1; i < QT; ++i) best = fmaxf(best, acc[i][j]);
#pragma unroll
      for (int dlt = 1; dlt < TQ; dlt <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, dlt));
      if (tq == 0) kbest[tk * NKT + j] = best;
    }
    __syncthreads();
    // one score per KV block: maximum over its R representatives, then the scale
    for (int blk = threadIdx.x; blk * r < KD; blk += blockDim.x) {
      const int first = base + blk * r;
      if (first < n_keys) {
        float best = kbest[blk * r];
        for (int e = 1; e < r; ++e) best = fmaxf(best, kbest[blk * r + e]);
        leader_scores[first / r] = best * scale;
      }
    }
  }
  cluster.sync();                              // every block's score is in the first CTA's shared memory
  if (rank != 0) return;
  if (scores_out)
    for (int j = threadIdx.x; j < nt; j += blockDim.x) scores_out[static_cast<long long>(list) * nt + j] = scores[j];
  // Few blocks: every score counts the scores that beat it (score descending, id ascending is
  // a total order, so the counts are the ranks). NaN scores would break the order: then, and
  // for long lists, the round-by-round arg-max is used.
  bool plain = nt <= 1024;
  if (plain) {
    bool has_nan = false;
    for (int j = threadIdx.x; j < nt; j += blockDim.x) has_nan |= scores[j] != scores[j];
    plain = !__syncthreads_or(has_nan);
  } else {
    __syncthreads();
  }
  if (plain) {
    for (int j = threadIdx.x; j < nt; j += blockDim.x) {
      const float mine = scores[j];
      int rank = 0;
      for (int i = 0; i < nt; ++i) rank += better(scores[i], i, mine, j) ? 1 : 0;
      if (rank < topk) ids_out[static_cast<long long>(list) * topk + rank] = j;
    }
    return;
  }
  block_topk(scores, nt, topk, ids_out + static_cast<long long>(list) * topk, scratch_f, scratch_i);
}

template <int MPAD, int QT, int NKT>
int launch_cluster(const __nv_bfloat16* qd, const __nv_bfloat16* kd, float* scores, int32_t* ids, int32_t* counter,
                   int lists, int hq, int hkv, int qt, int nt, int r, int topk, DeviceCtx* ctx, int slot,
                   cudaStream_t stream) {
  constexpr int KD = (256 / (MPAD / QT)) * NKT;
  const size_t smem = (128 * MPAD + 128 * KD + KD + nt + 10) * sizeof(float) + 16 * sizeof(int);
  if (!(ctx->small_attr & (1 << slot))) {
    cudaError_t e = cudaFuncSetAttribute(score_cluster_kernel<MPAD, QT, NKT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         100 * 1024);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->small_attr |= (1 << slot);
  }
  score_cluster_kernel<MPAD, QT, NKT><<<lists * CLUSTER, 256, smem, stream>>>(qd, kd, scores, ids, counter, hq, hkv, qt,
                                                                          nt, r, topk);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace

// Small problems only: at most four waves of 16-descriptor CTAs of pool_kernel.
bool pool_small_eligible(long long num_desc) {
  DeviceCtx* ctx = device_ctx();
  return ctx && (num_desc + 15) / 16 < 4LL * ctx->sm_count;
}

int launch_pool_small(const void* x, void* desc, long long num_desc, int tokens_per_desc, cudaStream_t stream) {
  return launch_pool_small_pair(x, desc, num_desc, nullptr, nullptr, 0, tokens_per_desc, stream);
}

// Two tensors in one launch (x2 may be null with num_desc2 = 0).
int launch_pool_small_pair(const void* x, void* desc, long long num_desc, const void* x2, void* desc2,
                           long long num_desc2, int tokens_per_desc, cudaStream_t stream) {
  pool_small_kernel<<<static_cast<unsigned>(num_desc + num_desc2), 256, static_cast<size_t>(tokens_per_desc) * 256,
                      stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(desc), num_desc,
                                static_cast<const __nv_bfloat16*>(x2), static_cast<__nv_bfloat16*>(desc2),
                                tokens_per_desc);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

// Returns 1 when the problem is not a small one (the caller then takes the other kernels).
int launch_summary_small(const void* qd, const void* kd, float* scores, int32_t* ids, int32_t* fallback_counter,
                         int batch, int hq, int hkv, int qt, int nt, int r, int topk, cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  const long long lists = static_cast<long long>(batch) * hkv * qt;
  const int m = (hq / hkv) * r;
  if (lists * CLUSTER > 8LL * ctx->sm_count || nt > 2048 || m > 64) return 1;
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(qd);
  const __nv_bfloat16* k = static_cast<const __nv_bfloat16*>(kd);
  const int n = static_cast<int>(lists);
  if (m <= 16) return launch_cluster<16, 1, 1>(q, k, scores, ids, fallback_counter, n, hq, hkv, qt, nt, r, topk, ctx, 0, stream);
  if (m <= 32) return launch_cluster<32, 2, 2>(q, k, scores, ids, fallback_counter, n, hq, hkv, qt, nt, r, topk, ctx, 1, stream);
  return launch_cluster<64, 4, 4>(q, k, scores, ids, fallback_counter, n, hq, hkv, qt, nt, r, topk, ctx, 2, stream);
}

}  // namespace sb
