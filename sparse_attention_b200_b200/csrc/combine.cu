// Log-sum-exp merge of partial (O, LSE): HBM-bound streaming kernel.
//   m = max_r L_r, w_r = exp(L_r - m), O = sum_r w_r O_r / sum_r w_r,
//   LSE = m + log(sum_r w_r)            (ranks accumulated in order 0..R-1)
// Half a warp per output row, eight features per lane, a whole batch of ranks in
// flight per lane. Partials may be fp32 or
// bf16 and are addressed with strides, so both the rank-major layout
// [R, rows, 128] written by the segment kernel and the rank-inner layout
// [rows, R, 128] of the reference are accepted.
// Same arithmetic as kv_combine11::kernel
// (attention/kv_centric/optimization_round11/combine11.cu:23-60), any R.
#include "internal.h"
#include <cuda_bf16.h>
#include <math_constants.h>

namespace sb {
namespace {

// eight consecutive features of one partial row, kept raw until the weights are known
template <typename T>
struct Raw8;
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = __ldcs(reinterpret_cast<const float4*>(p));
    b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static constexpr int BATCH = 8;      // ranks in flight per lane (64 registers)
};
template <>
struct Raw8<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(h[e]);
      f[2 * e] = v.x;
      f[2 * e + 1] = v.y;
    }
  }
  static constexpr int BATCH = 16;
};

// Half a warp (16 lanes x 8 features) per output row. The raw partial rows of a whole
// batch of ranks (16 for bf16, 8 for fp32) are requested first; the LSEs of the row are
// fetched one rank per lane (coalesced) and reduced with shuffles while those loads are
// in flight, so a row costs one memory round trip per batch instead of several dependent
// ones. A rank of weight 0 is dropped with a select, whatever it holds.
template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ partial, const float* __restrict__ lses,
                                                      __nv_bfloat16* __restrict__ out, float* __restrict__ out_lse,
                                                      long long rows, int ranks, long long p_stride_rank,
                                                      long long p_stride_row, long long l_stride_rank,
                                                      long long l_stride_row) {
  constexpr int BATCH = Raw8<T>::BATCH;
  const int sub = threadIdx.x & 15;
  const unsigned half_mask = 0xffffu << (threadIdx.x & 16);
  const long long halves_total = static_cast<long long>(gridDim.x) * (blockDim.x >> 4);
  const long long first = static_cast<long long>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4);
  // every lane of a warp runs the same number of iterations (the shuffles need both halves)
  const long long iters = (rows + halves_total - 1) / halves_total;
  for (long long it = 0; it < iters; ++it) {
    const long long row_raw = first + it * halves_total;
    const bool live = row_raw < rows;
    const long long row = live ? row_raw : rows - 1;
    const T* base = partial + row * p_stride_row + sub * 8;
    const float* lbase = lses + row * l_stride_row;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float denom = 0.f;
    Raw8<T> val[BATCH];
#pragma unroll
    for (int j = 0; j < BATCH; ++j)
      if (j < ranks) val[j].load(base + j * p_stride_rank);
    // row maximum of the LSEs: lane `sub` takes ranks sub, sub + 16, ...
    float maximum = -CUDART_INF_F;
    for (int r = sub; r < ranks; r += 16) maximum = fmaxf(maximum, __ldg(lbase + r * l_stride_rank));
#pragma unroll
    for (int d = 8; d >= 1; d >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, d));
    if (maximum > -CUDART_INF_F) {            // uniform within the half warp
      for (int r0 = 0; r0 < ranks; r0 += BATCH) {
        if (r0 > 0) {
#pragma unroll
          for (int j = 0; j < BATCH; ++j)
            if (r0 + j < ranks) val[j].load(base + (r0 + j) * p_stride_rank);
        }
        // weight of rank r0 + (sub % BATCH) in this lane (ranks of a batch sit in lanes 0..BATCH-1)
        float mine = 0.f;
        if (sub < BATCH && r0 + sub < ranks) mine = expf(__ldg(lbase + (r0 + sub) * l_stride_rank) - maximum);
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
          const float w = __shfl_sync(half_mask, mine, (threadIdx.x & 16) + j);   // exp(-inf) = 0
          if (r0 + j < ranks) {
            float f[8];
            val[j].unpack(f);
            denom += w;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, w > 0.f ? f[e] : 0.f, acc[e]);
          }
        }
      }
      const float inv = 1.0f / denom;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= inv;
    }
    if (live) {
      uint4 packed;
      uint32_t* pw = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        pw[e] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(out + row * 128 + sub * 8) = packed;
      if (sub == 0 && out_lse) out_lse[row] = (maximum > -CUDART_INF_F) ? maximum + logf(denom) : -CUDART_INF_F;
    }
  }
}

}  // namespace

int launch_combine(const void* partial, int partial_is_f32, const float* lses, void* out, float* out_lse,
                   long long rows, int ranks, long long p_stride_rank, long long p_stride_row,
                   long long l_stride_rank, long long l_stride_row, cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  const long long blocks_needed = (rows + 15) / 16;
  const long long cap = static_cast<long long>(ctx->sm_count) * 64;
  const int grid = static_cast<int>(blocks_needed < cap ? blocks_needed : cap);
  if (partial_is_f32)
    combine_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(partial), lses,
                                                    static_cast<__nv_bfloat16*>(out), out_lse, rows, ranks,
                                                    p_stride_rank, p_stride_row, l_stride_rank, l_stride_row);
  else
    combine_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(partial), lses,
                                                            static_cast<__nv_bfloat16*>(out), out_lse, rows, ranks,
                                                            p_stride_rank, p_stride_row, l_stride_rank,
                                                            l_stride_row);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
