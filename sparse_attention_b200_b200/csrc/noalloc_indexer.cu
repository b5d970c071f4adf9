// R1 / R4 summary indexer for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they
// need block ids: code running under a framework memory pool that owns the
// device and forbids outside allocations, a serving loop with a fixed
// device-memory budget, or a plugin that is handed its inputs and outputs and
// nothing else. The regular entry point (sparse_b200_indexer_summary) makes the
// caller supply two descriptor workspaces; this variant keeps those pooled
// descriptors in a fixed array that is part of the library image instead.
//
// Cost and limits: every GPU that loads the library holds NOALLOC_SCRATCH_BYTES
// (8 MiB) until the process exits. A call needs 256 bytes per pooled descriptor,
// (B*Hq*Sq/128 + B*Hkv*Skv/128) * R descriptors in total, so at most 32768 of
// them; also group size x R <= 16 and at most 4096 KV blocks. Larger problems
// are rejected with SPARSE_B200_ERR_INVALID; use the regular entry point.
//
// The array is shared by every call on a device and keeps the previous call's
// descriptors. Nothing in it has to start at zero: a call overwrites every
// descriptor it later reads. Two calls that overlap on one GPU (different
// streams, or different host threads) race on the array: serialise them.
//
// The first call on each device looks up the array's device address (host code
// only sees a host-side stand-in for a __device__ symbol, so the address is
// obtained with cudaGetSymbolAddress and passed to the kernels). Make that
// first call outside any stream capture.
//
// Arithmetic is that of indexer_summary.cu, so ids and scores are identical.
#include "internal.h"
#include "topk.cuh"
#include "../../include/sparse_b200.h"
#include <cuda_bf16.h>
#include <mutex>

namespace sb {
namespace {

constexpr size_t NOALLOC_SCRATCH_BYTES = 8u << 20;
constexpr long long NOALLOC_MAX_DESCRIPTORS = NOALLOC_SCRATCH_BYTES / 256;
constexpr int NOALLOC_MAX_KV_BLOCKS = 4096;
constexpr int NOALLOC_MP = 16;   // padded (group size x R)

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// fp32 mean of n consecutive tokens, summed in token order, rounded to bf16.
__global__ void __launch_bounds__(256) noalloc_pool_kernel(const __nv_bfloat16* __restrict__ x,
                                                           __nv_bfloat16* __restrict__ desc, long long num_desc,
                                                           int n) {
  const long long vec = static_cast<long long>(blockIdx.x) * 16 + (threadIdx.x >> 4);
  if (vec >= num_desc) return;
  const int part = threadIdx.x & 15;
  const uint4* src = reinterpret_cast<const uint4*>(x + vec * n * 128 + part * 8);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int t = 0; t < n; ++t) {
    const uint4 v = __ldg(src + static_cast<long long>(t) * 16);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      acc[2 * e] += f.x;
      acc[2 * e + 1] += f.y;
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

// One CTA per (batch, KV head, query block); descriptors come from the scratch array.
__global__ void __launch_bounds__(256) noalloc_score_topk_kernel(const __nv_bfloat16* __restrict__ qd,
                                                                 const __nv_bfloat16* __restrict__ kd,
                                                                 float* __restrict__ scores_out,
                                                                 int32_t* __restrict__ ids_out, int hq, int hkv,
                                                                 int qt, int nt, int r, int topk) {
  __shared__ float q_s[128 * NOALLOC_MP];
  __shared__ float scores[NOALLOC_MAX_KV_BLOCKS];
  __shared__ float scratch_f[10];
  __shared__ int scratch_i[10];
  const int group = hq / hkv, m_real = group * r;
  const int list = blockIdx.x;
  const int qtile = list % qt, bk = list / qt;
  const int b = bk / hkv, kvh = bk - b * hkv;
  for (int e = threadIdx.x; e < 128 * NOALLOC_MP; e += blockDim.x) {
    const int m = e % NOALLOC_MP, d = e / NOALLOC_MP;
    const int mm = m < m_real ? m : 0;
    const int g = mm / r, rq = mm - g * r;
    const long long row = ((static_cast<long long>(b) * hq + kvh * group + g) * qt + qtile) * r + rq;
    q_s[d * NOALLOC_MP + m] = __bfloat162float(qd[row * 128 + d]);
  }
  __syncthreads();
  const int n_keys = nt * r;
  const __nv_bfloat16* kbase = kd + static_cast<long long>(bk) * n_keys * 128;
  for (int base = 0; base < n_keys; base += blockDim.x) {
    const int n = base + threadIdx.x;
    const bool valid = n < n_keys;
    float best = -CUDART_INF_F;
    if (valid) {
      float acc[NOALLOC_MP];
#pragma unroll
      for (int m = 0; m < NOALLOC_MP; ++m) acc[m] = 0.f;
      const uint4* krow = reinterpret_cast<const uint4*>(kbase + static_cast<long long>(n) * 128);
      for (int c = 0; c < 16; ++c) {
        const uint4 kv = krow[c];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&kv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 kf = __bfloat1622float2(h[e]);
          const float* q0 = q_s + (c * 8 + 2 * e) * NOALLOC_MP;
#pragma unroll
          for (int m = 0; m < NOALLOC_MP; ++m) acc[m] = fmaf(q0[m], kf.x, acc[m]);
#pragma unroll
          for (int m = 0; m < NOALLOC_MP; ++m) acc[m] = fmaf(q0[NOALLOC_MP + m], kf.y, acc[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < NOALLOC_MP; ++m) best = fmaxf(best, acc[m]);
    }
    for (int d = 1; d < r; d <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, d));
    if (valid && (n % r) == 0) scores[n / r] = best * 0.08838834764831845f;
  }
  __syncthreads();
  if (scores_out)
    for (int j = threadIdx.x; j < nt; j += blockDim.x) scores_out[static_cast<long long>(list) * nt + j] = scores[j];
  __syncthreads();
  block_topk(scores, nt, topk, ids_out + static_cast<long long>(list) * topk, scratch_f, scratch_i);
}

std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_ptr[64] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
int noalloc_scratch(unsigned char** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return set_error(SB_ERR_CUDA, "no current CUDA device");
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return SB_OK;
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" int sparse_b200_indexer_summary_noalloc(const void* q, const void* k, float* scores, int32_t* block_idx,
                                                   int batch, int hq, int hkv, int sq, int skv, int representatives,
                                                   int topk, void* stream) {
  if (!q || !k || !block_idx) return set_error(SB_ERR_INVALID, "q, k and block_idx must be non-null device pointers");
  if (batch <= 0 || hkv <= 0 || hq < hkv || hq % hkv) return set_error(SB_ERR_INVALID, "Hq must be a positive multiple of Hkv");
  if (sq < 128 || sq % 128 || skv < 128 || skv % 128)
    return set_error(SB_ERR_INVALID, "Sq and Skv must be positive multiples of 128");
  const int r = representatives;
  if (r != 1 && r != 2 && r != 4) return set_error(SB_ERR_INVALID, "representatives must be 1, 2 or 4");
  const int qt = sq / 128, nt = skv / 128;
  if (topk <= 0 || topk > nt) return set_error(SB_ERR_INVALID, "top-k must be in [1, number of KV blocks]");
  if ((reinterpret_cast<uintptr_t>(q) & 15u) || (reinterpret_cast<uintptr_t>(k) & 15u))
    return set_error(SB_ERR_INVALID, "q and k must be 16-byte aligned");
  const long long nq = static_cast<long long>(batch) * hq * qt * r, nk = static_cast<long long>(batch) * hkv * nt * r;
  if ((hq / hkv) * r > NOALLOC_MP)
    return set_error(SB_ERR_INVALID, "no-alloc indexer: group size x representatives must not exceed 16");
  if (nt > NOALLOC_MAX_KV_BLOCKS)
    return set_error(SB_ERR_INVALID, "no-alloc indexer: at most 4096 KV blocks");
  if (nq + nk > NOALLOC_MAX_DESCRIPTORS)
    return set_error(SB_ERR_INVALID,
                     "no-alloc indexer: the pooled descriptors exceed the 8 MiB built-in scratch "
                     "(32768 descriptors); use sparse_b200_indexer_summary with caller workspaces");
  unsigned char* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  __nv_bfloat16* qd = reinterpret_cast<__nv_bfloat16*>(scratch);
  __nv_bfloat16* kd = qd + nq * 128;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  noalloc_pool_kernel<<<static_cast<unsigned>((nq + 15) / 16), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(q), qd,
                                                                            nq, 128 / r);
  noalloc_pool_kernel<<<static_cast<unsigned>((nk + 15) / 16), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(k), kd,
                                                                            nk, 128 / r);
  noalloc_score_topk_kernel<<<batch * hkv * qt, 256, 0, st>>>(qd, kd, scores, block_idx, hq, hkv, qt, nt, r, topk);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}
