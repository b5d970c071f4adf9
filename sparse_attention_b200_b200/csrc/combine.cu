// Log-sum-exp merge of partial (O, LSE): HBM-bound streaming kernel.
//   m = max_r L_r, w_r = exp(L_r - m), O = sum_r w_r O_r / sum_r w_r,
//   LSE = m + log(sum_r w_r)            (ranks accumulated in order 0..R-1)
// Half a warp per output row, eight features per lane. Partials may be fp32 or
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

// eight consecutive features of one partial row as fp32
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 v = __bfloat1622float2(h[e]);
    f[2 * e] = v.x;
    f[2 * e + 1] = v.y;
  }
}

// Half a warp (16 lanes x 8 features) per output row. The partial rows of up to
// four ranks are requested before the weights are known, so the two dependent
// memory round trips (LSE, then partials) overlap; a rank of weight 0 is then
// dropped with a select, whatever it holds.
template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ partial, const float* __restrict__ lses,
                                                      __nv_bfloat16* __restrict__ out, float* __restrict__ out_lse,
                                                      long long rows, int ranks, long long p_stride_rank,
                                                      long long p_stride_row, long long l_stride_rank,
                                                      long long l_stride_row) {
  const int sub = threadIdx.x & 15;
  const long long halves_total = static_cast<long long>(gridDim.x) * (blockDim.x >> 4);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4); row < rows;
       row += halves_total) {
    const T* base = partial + row * p_stride_row + sub * 8;
    const float* lbase = lses + row * l_stride_row;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float denom = 0.f;
    // Requests first, arithmetic later: the partial rows of the first four ranks and
    // every rank's LSE (a broadcast within the half warp) are all in flight together.
    float val[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < ranks) {
        load8<T>(base + j * p_stride_rank, val[j]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) val[j][e] = 0.f;
      }
    }
    float maximum = -CUDART_INF_F;
    for (int r = 0; r < ranks; ++r) maximum = fmaxf(maximum, __ldg(lbase + r * l_stride_rank));
    if (maximum > -CUDART_INF_F) {
      for (int r0 = 0; r0 < ranks; r0 += 4) {
        float wgt[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (r0 + j < ranks) {
            if (r0 > 0) load8<T>(base + (r0 + j) * p_stride_rank, val[j]);
            wgt[j] = expf(__ldg(lbase + (r0 + j) * l_stride_rank) - maximum);   // exp(-inf) = 0
          } else {
            wgt[j] = 0.f;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          denom += wgt[j];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(wgt[j], wgt[j] > 0.f ? val[j][e] : 0.f, acc[e]);
        }
      }
      const float inv = 1.0f / denom;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= inv;
    }
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
