// Log-sum-exp merge of partial (O, LSE): HBM-bound streaming kernel.
//   m = max_r L_r, w_r = exp(L_r - m), O = sum_r w_r O_r / sum_r w_r,
//   LSE = m + log(sum_r w_r)            (ranks accumulated in order 0..R-1)
// One warp per output row, four features per lane, a whole batch of ranks in
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

// four consecutive features of one partial row, kept raw until the weights are known
template <typename T>
struct Raw4;
template <>
struct Raw4<float> {
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = __ldcs(reinterpret_cast<const float4*>(p)); }
  __device__ __forceinline__ void unpack(float (&f)[4]) const { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
};
template <>
struct Raw4<__nv_bfloat16> {
  uint2 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = __ldcs(reinterpret_cast<const uint2*>(p)); }
  __device__ __forceinline__ void unpack(float (&f)[4]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
};

// One warp per output row (RPW rows at a time when there are few ranks), four features per
// lane, four warps per block and no persistent loop: registers stay low (16 (row, rank) pieces
// of raw data per lane = 32-64 registers), so an SM keeps 32-64 rows x R ranks of loads in
// flight, which is what a streaming kernel with two dependent round trips (LSEs, partial rows)
// needs to approach HBM bandwidth. The raw partial rows are requested first; the LSEs of a row
// are fetched one rank per lane and reduced with shuffles while those loads fly. A rank of
// weight 0 is dropped with a select, whatever it holds.
// Offset of a row's first partial. Rows are (batch, head, token) in that order everywhere; with
// tm_h > 0 the partials are token-major [B, S, ranks, H, 128] (the caller passes H * 128 as the
// rank stride), else `row * p_stride_row`.
__device__ __forceinline__ long long partial_base(long long row, long long p_stride_row, int ranks, int tm_h, int tm_s) {
  if (tm_h == 0) return row * p_stride_row;
  const long long bh = row / tm_s;
  const long long s = row - bh * tm_s, b = bh / tm_h, h = bh - b * tm_h;
  return ((b * tm_s + s) * ranks * tm_h + h) * 128;
}

template <typename T, int RPW>
__global__ void __launch_bounds__(128) combine_kernel(const T* __restrict__ partial, const float* __restrict__ lses,
                                                      __nv_bfloat16* __restrict__ out, float* __restrict__ out_lse,
                                                      long long rows, int ranks, long long p_stride_rank,
                                                      long long p_stride_row, long long l_stride_rank,
                                                      long long l_stride_row, int tm_h, int tm_s) {
  constexpr int CB = 16 / RPW;                   // ranks per batch
  const int lane = threadIdx.x & 31;
  const long long row0 = (static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5)) * RPW;
  if (row0 >= rows) return;                      // whole warps leave together
  Raw4<T> val[RPW][CB];
#pragma unroll
  for (int rr = 0; rr < RPW; ++rr) {
    const long long row = min(row0 + rr, rows - 1);
#pragma unroll
    for (int j = 0; j < CB; ++j)
      if (j < ranks) val[rr][j].load(partial + partial_base(row, p_stride_row, ranks, tm_h, tm_s) + lane * 4 + j * p_stride_rank);
  }
#pragma unroll
  for (int rr = 0; rr < RPW; ++rr) {
    const bool live = row0 + rr < rows;
    const long long row = live ? row0 + rr : rows - 1;
    const T* base = partial + partial_base(row, p_stride_row, ranks, tm_h, tm_s) + lane * 4;
    const float* lbase = lses + row * l_stride_row;
    // row maximum of the LSEs: lane l takes ranks l, l + 32, ...
    float maximum = -CUDART_INF_F;
    for (int r = lane; r < ranks; r += 32) maximum = fmaxf(maximum, __ldg(lbase + r * l_stride_rank));
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, d));
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float denom = 0.f;
    if (maximum > -CUDART_INF_F) {               // uniform within the warp
      for (int r0 = 0; r0 < ranks; r0 += CB) {
        if (r0 > 0) {
#pragma unroll
          for (int j = 0; j < CB; ++j)
            if (r0 + j < ranks) val[rr][j].load(base + (r0 + j) * p_stride_rank);
        }
        // weight of rank r0 + lane in lane `lane` (the ranks of a batch sit in lanes 0..CB-1)
        float mine = 0.f;
        if (lane < CB && r0 + lane < ranks) mine = expf(__ldg(lbase + (r0 + lane) * l_stride_rank) - maximum);
#pragma unroll
        for (int j = 0; j < CB; ++j) {
          const float w = __shfl_sync(0xffffffffu, mine, j);   // exp(-inf) = 0
          if (r0 + j < ranks) {
            float f[4];
            val[rr][j].unpack(f);
            denom += w;
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(w, w > 0.f ? f[e] : 0.f, acc[e]);
          }
        }
      }
      const float inv = 1.0f / denom;
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] *= inv;
    }
    if (live) {
      uint2 packed;
      __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0], acc[1]), h1 = __floats2bfloat162_rn(acc[2], acc[3]);
      packed.x = *reinterpret_cast<uint32_t*>(&h0);
      packed.y = *reinterpret_cast<uint32_t*>(&h1);
      *reinterpret_cast<uint2*>(out + row * 128 + lane * 4) = packed;
      if (lane == 0 && out_lse) out_lse[row] = (maximum > -CUDART_INF_F) ? maximum + logf(denom) : -CUDART_INF_F;
    }
  }
}

// Eight consecutive features of one partial row.
template <typename T>
struct Raw8;
template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = __ldcs(reinterpret_cast<const float4*>(p));
    b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void clear() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};
template <>
struct Raw8<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void clear() { raw = make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
};

// Rank counts compiled in (1-4: KV-range segments, KV splits across GPUs; 8 and 16 bf16 ranks:
// per-token selection lists): the kernel above spends its time issuing instructions there
// (shuffles for the weights, 64-bit address arithmetic per 8-byte load), not waiting for
// memory. Here sixteen threads share a row, eight features each, every thread reads the
// row's R LSEs itself (one broadcast transaction) and computes the weights redundantly: no
// shuffles, 16-byte loads. U rows per thread keep U R loads of 16 bytes in flight. Same
// operations in the same order as combine_kernel, so the results are bit-identical.
template <typename T, int R, int U>
__global__ void __launch_bounds__(256) combine_few_kernel(const T* __restrict__ partial, const float* __restrict__ lses,
                                                          __nv_bfloat16* __restrict__ out, float* __restrict__ out_lse,
                                                          long long rows, long long p_stride_rank, long long p_stride_row,
                                                          long long l_stride_rank, long long l_stride_row, int tm_h,
                                                          int tm_s) {
  const int slot = threadIdx.x >> 4, part = threadIdx.x & 15;
  const long long row_base = static_cast<long long>(blockIdx.x) * (16 * U) + slot;
  Raw8<T> val[U][R];
  float L[U][R];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const long long row = min(row_base + 16 * u, rows - 1);
    const T* src = partial + partial_base(row, p_stride_row, R, tm_h, tm_s) + part * 8;
    const float* lsrc = lses + row * l_stride_row;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      val[u][r].load(src + r * p_stride_rank);
      L[u][r] = __ldg(lsrc + r * l_stride_rank);
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const long long row = row_base + 16 * u;
    if (row >= rows) continue;
    float maximum = L[u][0];
#pragma unroll
    for (int r = 1; r < R; ++r) maximum = fmaxf(maximum, L[u][r]);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float denom = 0.f;
    if (maximum > -CUDART_INF_F) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float w = expf(L[u][r] - maximum);   // exp(-inf) = 0
        if (!(w > 0.f)) val[u][r].clear();         // a rank of weight 0 is dropped, whatever it holds
        float f[8];
        val[u][r].unpack(f);
        denom += w;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, f[e], acc[e]);
      }
      const float inv = 1.0f / denom;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= inv;
    }
    uint4 packed;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0], acc[1]), h1 = __floats2bfloat162_rn(acc[2], acc[3]);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[4], acc[5]), h3 = __floats2bfloat162_rn(acc[6], acc[7]);
    packed.x = *reinterpret_cast<uint32_t*>(&h0);
    packed.y = *reinterpret_cast<uint32_t*>(&h1);
    packed.z = *reinterpret_cast<uint32_t*>(&h2);
    packed.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(out + row * 128 + part * 8) = packed;
    if (part == 0 && out_lse) out_lse[row] = (maximum > -CUDART_INF_F) ? maximum + logf(denom) : -CUDART_INF_F;
  }
}

template <typename T, int R>
static void combine_few_launch(const void* partial, const float* lses, void* out, float* out_lse, long long rows,
                               long long psr, long long psw, long long lsr, long long lsw, int tm_h, int tm_s, cudaStream_t stream) {
  constexpr int U = R <= 4 ? 2 : 1;
  combine_few_kernel<T, R, U><<<static_cast<unsigned>((rows + 16 * U - 1) / (16 * U)), 256, 0, stream>>>(
      static_cast<const T*>(partial), lses, static_cast<__nv_bfloat16*>(out), out_lse, rows, psr, psw, lsr, lsw, tm_h, tm_s);
}

template <typename T>
static void combine_few_dispatch(int ranks, const void* partial, const float* lses, void* out, float* out_lse,
                                 long long rows, long long psr, long long psw, long long lsr, long long lsw,
                                 int tm_h, int tm_s, cudaStream_t stream) {
  switch (ranks) {
    case 1: combine_few_launch<T, 1>(partial, lses, out, out_lse, rows, psr, psw, lsr, lsw, tm_h, tm_s, stream); break;
    case 2: combine_few_launch<T, 2>(partial, lses, out, out_lse, rows, psr, psw, lsr, lsw, tm_h, tm_s, stream); break;
    case 3: combine_few_launch<T, 3>(partial, lses, out, out_lse, rows, psr, psw, lsr, lsw, tm_h, tm_s, stream); break;
    case 4: combine_few_launch<T, 4>(partial, lses, out, out_lse, rows, psr, psw, lsr, lsw, tm_h, tm_s, stream); break;
    case 8: combine_few_launch<T, 8>(partial, lses, out, out_lse, rows, psr, psw, lsr, lsw, tm_h, tm_s, stream); break;
    default: combine_few_launch<T, 16>(partial, lses, out, out_lse, rows, psr, psw, lsr, lsw, tm_h, tm_s, stream); break;
  }
}

template <typename T, int RPW>
static void combine_launch(const void* partial, const float* lses, void* out, float* out_lse, long long rows, int ranks,
                           long long psr, long long psw, long long lsr, long long lsw, int tm_h, int tm_s, cudaStream_t stream) {
  const long long blocks = (rows + 4 * RPW - 1) / (4 * RPW);
  combine_kernel<T, RPW><<<static_cast<unsigned>(blocks), 128, 0, stream>>>(
      static_cast<const T*>(partial), lses, static_cast<__nv_bfloat16*>(out), out_lse, rows, ranks, psr, psw, lsr, lsw, tm_h, tm_s);
}

}  // namespace

int launch_combine(const void* partial, int partial_is_f32, const float* lses, void* out, float* out_lse,
                   long long rows, int ranks, long long p_stride_rank, long long p_stride_row,
                   long long l_stride_rank, long long l_stride_row, cudaStream_t stream, int tm_h, int tm_s) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  if ((rows + 3) / 4 > 0x7fffffffLL) return set_error(SB_ERR_INVALID, "too many rows for one combine launch");
  // 16-byte accesses of the specialised kernel: every stride must keep them aligned
  const long long esz = partial_is_f32 ? 4 : 2;
  const bool aligned = ((reinterpret_cast<uintptr_t>(partial) & 15u) == 0) && ((p_stride_rank * esz) & 15) == 0 &&
                       ((p_stride_row * esz) & 15) == 0 && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
  const bool compiled_in = (ranks >= 1 && ranks <= 4) || (!partial_is_f32 && (ranks == 8 || ranks == 16));
  if (compiled_in && aligned) {
    if (partial_is_f32) combine_few_dispatch<float>(ranks, partial, lses, out, out_lse, rows, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
    else combine_few_dispatch<__nv_bfloat16>(ranks, partial, lses, out, out_lse, rows, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  }
  // few ranks: several rows per warp, so that every lane still has 16 loads in flight
  if (partial_is_f32) {
    if (ranks <= 4) combine_launch<float, 4>(partial, lses, out, out_lse, rows, ranks, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
    else if (ranks <= 8) combine_launch<float, 2>(partial, lses, out, out_lse, rows, ranks, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
    else combine_launch<float, 1>(partial, lses, out, out_lse, rows, ranks, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
  } else {
    if (ranks <= 4) combine_launch<__nv_bfloat16, 4>(partial, lses, out, out_lse, rows, ranks, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
    else if (ranks <= 8) combine_launch<__nv_bfloat16, 2>(partial, lses, out, out_lse, rows, ranks, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
    else combine_launch<__nv_bfloat16, 1>(partial, lses, out, out_lse, rows, ranks, p_stride_rank, p_stride_row, l_stride_rank, l_stride_row, tm_h, tm_s, stream);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
