// Block-wide top-k over scores held in shared memory: k rounds of arg-max keyed
// on (score descending, index ascending), so ties go to the lower block index
// and ids come out in score-descending order (the order of reduce_topk,
// indexers/r1_r4/gpu_ops.py:44-49, and tile_max_topk16_kernel,
// indexers/fp4/tile_topk.cu:98-124). Taken entries are overwritten with NaN
// (skipped by the scan), so a genuine -inf or -FLT_MAX score is still picked once.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <climits>
#include <cstdint>

namespace sb {

__device__ __forceinline__ bool better(float s, int i, float bs, int bi) {
  return s > bs || (s == bs && i < bi);
}

// scores: shared memory [n]; scratch_f / scratch_i: shared memory, blockDim.x / 32 + 1 words each.
// All threads of the block must call. ids_out may point to global memory.
// vals_out (optional, may be shared memory): the scores of the winners, same order.
__device__ __forceinline__ void block_topk_ex(float* scores, int n, int k, int32_t* ids_out, float* vals_out,
                                              float* scratch_f, int* scratch_i) {
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
  float my_s = -CUDART_INF_F;
  int my_i = INT_MAX;
  bool dirty = true;
  for (int rank = 0; rank < k; ++rank) {
    if (dirty) {
      my_s = -CUDART_INF_F;
      my_i = INT_MAX;
      for (int j = tid; j < n; j += nthreads) {
        const float s = scores[j];
        if (s != s) continue;                  // retired
        if (better(s, j, my_s, my_i)) { my_s = s; my_i = j; }
      }
      dirty = false;
    }
    float bs = my_s;
    int bi = my_i;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float os = __shfl_xor_sync(0xffffffffu, bs, d);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
      if (better(os, oi, bs, bi)) { bs = os; bi = oi; }
    }
    if (lane == 0) { scratch_f[warp] = bs; scratch_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bs = lane < nwarps ? scratch_f[lane] : -CUDART_INF_F;
      bi = lane < nwarps ? scratch_i[lane] : INT_MAX;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, bs, d);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
        if (better(os, oi, bs, bi)) { bs = os; bi = oi; }
      }
      if (lane == 0) { scratch_i[nwarps] = bi; scratch_f[nwarps] = bs; }
    }
    __syncthreads();
    const int winner = scratch_i[nwarps];
    if (winner != INT_MAX && (winner % nthreads) == tid) {
      scores[winner] = __int_as_float(0x7fc00000);   // NaN = retired
      dirty = true;
    }
    if (tid == 0) {
      ids_out[rank] = winner == INT_MAX ? 0 : winner;
      if (vals_out) vals_out[rank] = scratch_f[nwarps];
    }
    __syncthreads();
  }
}

__device__ __forceinline__ void block_topk(float* scores, int n, int k, int32_t* ids_out, float* scratch_f,
                                           int* scratch_i) {
  block_topk_ex(scores, n, k, ids_out, nullptr, scratch_f, scratch_i);
}

}  // namespace sb
