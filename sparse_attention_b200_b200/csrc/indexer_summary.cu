// R1 / R4 block-summary indexer: pooled bf16 descriptors, descriptor scores,
// group max and top-k, with a fixed arithmetic so the emitted block ids are
// reproducible bit for bit:
//   descriptor = bf16_rne((x_0 + x_1 + ... + x_{n-1}) * (1/n)), fp32 adds in
//                token order, n = 128/R;
//   raw        = sum over the 128 features in feature order (fp32 FMA; every
//                bf16 x bf16 product is exact in fp32);
//   score      = max over (heads of the KV group, R query reps, R key reps) of
//                raw, times fp32(128^-0.5);
//   ids        = top-k by (score descending, block id ascending).
// Replaces pool_blocks, descriptor_dot and reduce_topk
// (indexers/r1_r4/gpu_ops.py:6-49) and SummarySelector
// (indexers/r1_r4/block_selectors.py:9-45); the raw score matrix is never
// written to memory, any Hkv / group size <= 16 / top-k / block count.
#include "internal.h"
#include "topk.cuh"
#include <cuda_bf16.h>

namespace sb {
namespace {

// ---------------------------------------------------------------- pooling
// 16 threads per descriptor (8 features each), tokens summed sequentially.
__global__ void __launch_bounds__(256) pool_kernel(const __nv_bfloat16* __restrict__ x,
                                                   __nv_bfloat16* __restrict__ desc, long long num_desc, int n) {
  const long long vec = static_cast<long long>(blockIdx.x) * 16 + (threadIdx.x >> 4);
  if (vec >= num_desc) return;
  const int part = threadIdx.x & 15;
  const uint4* src = reinterpret_cast<const uint4*>(x + vec * n * 128 + part * 8);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int t0 = 0; t0 < n; t0 += 8) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldcs(src + static_cast<long long>(t0 + j) * 16);   // 16 uint4 per token row
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
  }
  const float inv = 1.0f / static_cast<float>(n);
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
    ow[e] = *reinterpret_cast<uint32_t*>(&p);
  }
  *reinterpret_cast<uint4*>(desc + vec * 128 + part * 8) = o;
}

// ---------------------------------------------------------------- score + top-k
// One CTA per (batch, KV head, query block). MP = padded number of query
// descriptors (group heads x R). Thread t scores key descriptor base + t against
// all MP query descriptors (accumulators in registers, query descriptors read
// from shared memory as broadcasts), feature by feature.
template <int MP>
__global__ void __launch_bounds__(256) score_topk_kernel(const __nv_bfloat16* __restrict__ qd,
                                                         const __nv_bfloat16* __restrict__ kd,
                                                         float* __restrict__ scores_out, int32_t* __restrict__ ids_out,
                                                         int hq, int hkv, int qt, int nt, int r, int topk,
                                                         int flagged_only) {
  // second pass after a pre-filter kernel: only lists it marked with -1 as their first id
  if (flagged_only && ids_out[static_cast<long long>(blockIdx.x) * topk] != -1) return;
  extern __shared__ float smem[];
  float* q_s = smem;                         // [128][MP]
  float* scores = q_s + 128 * MP;            // [nt]
  float* scratch_f = scores + nt;            // [10]
  int* scratch_i = reinterpret_cast<int*>(scratch_f + 10);

  const int group = hq / hkv;
  const int m_real = group * r;
  const int list = blockIdx.x;               // (b * hkv + kvh) * qt + qtile
  const int qtile = list % qt;
  const int bk = list / qt;
  const int b = bk / hkv, kvh = bk - b * hkv;

  for (int e = threadIdx.x; e < 128 * MP; e += blockDim.x) {
    const int m = e % MP, d = e / MP;
    const int mm = m < m_real ? m : 0;
    const int g = mm / r, rq = mm - g * r;
    const long long row = ((static_cast<long long>(b) * hq + kvh * group + g) * qt + qtile) * r + rq;
    q_s[d * MP + m] = __bfloat162float(qd[row * 128 + d]);
  }
  __syncthreads();

  const int n_keys = nt * r;
  const __nv_bfloat16* kbase = kd + static_cast<long long>(bk) * n_keys * 128;
  const float scale = 0.08838834764831845f;   // fp32(128^-0.5)
  for (int base = 0; base < n_keys; base += blockDim.x) {
    const int n = base + threadIdx.x;
    const bool valid = n < n_keys;
    float best = -CUDART_INF_F;
    if (valid) {
      float acc[MP];
#pragma unroll
      for (int m = 0; m < MP; ++m) acc[m] = 0.f;
      const uint4* krow = reinterpret_cast<const uint4*>(kbase + static_cast<long long>(n) * 128);
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
#pragma unroll
      for (int m = 0; m < MP; ++m) best = fmaxf(best, acc[m]);
    }
    // max over the R key representatives of a block: adjacent lanes
    for (int d = 1; d < r; d <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, d));
    if (valid && (n % r) == 0) scores[n / r] = best * scale;
  }
  __syncthreads();
  if (scores_out)
    for (int j = threadIdx.x; j < nt; j += blockDim.x) scores_out[static_cast<long long>(list) * nt + j] = scores[j];
  __syncthreads();
  block_topk(scores, nt, topk, ids_out + static_cast<long long>(list) * topk, scratch_f, scratch_i);
}

template <int MP>
int launch_score(const __nv_bfloat16* qd, const __nv_bfloat16* kd, float* scores, int32_t* ids, int batch, int hq,
                 int hkv, int qt, int nt, int r, int topk, DeviceCtx* ctx, int slot, cudaStream_t stream,
                 int flagged_only) {
  const size_t smem = (128 * MP + nt + 10) * sizeof(float) + 16 * sizeof(int);
  if (smem > 200 * 1024) return set_error(SB_ERR_INVALID, "too many KV blocks for the summary indexer (shared memory)");
  if (!ctx->misc_attr[slot]) {
    cudaError_t e = cudaFuncSetAttribute(score_topk_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    ctx->misc_attr[slot] = 1;
  }
  score_topk_kernel<MP><<<batch * hkv * qt, 256, smem, stream>>>(qd, kd, scores, ids, hq, hkv, qt, nt, r, topk,
                                                                  flagged_only);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace

int launch_pool(const void* x, void* desc, long long num_desc, int tokens_per_desc, cudaStream_t stream) {
  const long long blocks = (num_desc + 15) / 16;
  pool_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                  static_cast<__nv_bfloat16*>(desc), num_desc,
                                                                  tokens_per_desc);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

int launch_summary_score_topk(const void* qd, const void* kd, float* scores, int32_t* ids, int batch, int hq, int hkv,
                              int qt, int nt, int r, int topk, cudaStream_t stream, int flagged_only) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  const int m = (hq / hkv) * r;
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(qd);
  const __nv_bfloat16* k = static_cast<const __nv_bfloat16*>(kd);
  if (m <= 4) return launch_score<4>(q, k, scores, ids, batch, hq, hkv, qt, nt, r, topk, ctx, 0, stream, flagged_only);
  if (m <= 8) return launch_score<8>(q, k, scores, ids, batch, hq, hkv, qt, nt, r, topk, ctx, 1, stream, flagged_only);
  if (m <= 16) return launch_score<16>(q, k, scores, ids, batch, hq, hkv, qt, nt, r, topk, ctx, 2, stream, flagged_only);
  if (m <= 32) return launch_score<32>(q, k, scores, ids, batch, hq, hkv, qt, nt, r, topk, ctx, 3, stream, flagged_only);
  if (m <= 64) return launch_score<64>(q, k, scores, ids, batch, hq, hkv, qt, nt, r, topk, ctx, 4, stream, flagged_only);
  return set_error(SB_ERR_INVALID, "group size x representatives must not exceed 64");
}

}  // namespace sb
