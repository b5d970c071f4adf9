// Log-sum-exp merge of partial (O, LSE): HBM-bound streaming kernel.
//   m = max_r L_r, w_r = exp(L_r - m), O = sum_r w_r O_r / sum_r w_r,
//   LSE = m + log(sum_r w_r)            (ranks accumulated in order 0..R-1)
// One warp per output row, four features per lane. Partials may be fp32 or
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

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return __ldcs(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ partial, const float* __restrict__ lses,
                                                      __nv_bfloat16* __restrict__ out, float* __restrict__ out_lse,
                                                      long long rows, int ranks, long long p_stride_rank,
                                                      long long p_stride_row, long long l_stride_rank,
                                                      long long l_stride_row) {
  const int lane = threadIdx.x & 31;
  const long long warps_total = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += warps_total) {
    float maximum = -CUDART_INF_F;
    for (int r = lane; r < ranks; r += 32)
      maximum = fmaxf(maximum, lses[r * l_stride_rank + row * l_stride_row]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, d));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float denom = 0.f;
    if (maximum > -CUDART_INF_F) {
      const T* base = partial + row * p_stride_row + lane * 4;
      for (int r0 = 0; r0 < ranks; r0 += 4) {
        float4 val[4];
        float wgt[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = r0 + j;
          if (r < ranks) {
            const float l = lses[r * l_stride_rank + row * l_stride_row];
            wgt[j] = (l > -CUDART_INF_F) ? expf(l - maximum) : 0.f;
            // A rank with weight 0 may hold anything (even NaN): skip its load.
            val[j] = (wgt[j] > 0.f) ? load4<T>(base + r * p_stride_rank) : make_float4(0.f, 0.f, 0.f, 0.f);
          } else {
            wgt[j] = 0.f;
            val[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          denom += wgt[j];
          acc.x = fmaf(wgt[j], val[j].x, acc.x);
          acc.y = fmaf(wgt[j], val[j].y, acc.y);
          acc.z = fmaf(wgt[j], val[j].z, acc.z);
          acc.w = fmaf(wgt[j], val[j].w, acc.w);
        }
      }
      const float inv = 1.0f / denom;
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + row * 128 + lane * 4) = packed;
    if (lane == 0 && out_lse) out_lse[row] = (maximum > -CUDART_INF_F) ? maximum + logf(denom) : -CUDART_INF_F;
  }
}

}  // namespace

int launch_combine(const void* partial, int partial_is_f32, const float* lses, void* out, float* out_lse,
                   long long rows, int ranks, long long p_stride_rank, long long p_stride_row,
                   long long l_stride_rank, long long l_stride_row, cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  const long long blocks_needed = (rows + 7) / 8;
  const long long cap = static_cast<long long>(ctx->sm_count) * 32;
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
