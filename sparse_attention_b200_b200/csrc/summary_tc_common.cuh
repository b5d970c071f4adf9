// Shared by the two tensor-core forms of the R1 / R4 summary selector
// (indexer_summary_tc.cu: one CTA per work unit, phases in series; indexer_summary_stream.cu:
// persistent CTAs, scoring and selection overlapped).
#pragma once
#include "ptx.cuh"
#include "internal.h"
#include <cuda_bf16.h>

namespace sb {
namespace stc {

constexpr int C_MAX = 192;                 // candidates per list
constexpr float EPS = 6.103515625e-05f;    // 2^-14
constexpr float SCALE = 0.08838834764831845f;

struct Params {
  const __nv_bfloat16* qd;     // [B, Hq, qt, R, 128]
  const __nv_bfloat16* kd;     // [B, Hkv, nt, R, 128]
  const float* k_absmax;       // [B * Hkv] max |element| of the key descriptors of a head
  const float* k_norm2;        // [B * Hkv] max squared L2 norm of a key descriptor of the head
  int32_t* ids;                // [B, Hkv, qt, topk]
  int* status;
  int* fallbacks;              // optional counter of lists that took the exact fallback
  int* violations;             // re-scored candidates whose two scores differed by more than delta
  int* max_ratio;              // largest observed |approximate - exact| / delta (float bits)
  int hq, hkv, qt, nt, r, topk, qb, cand;
  int q_chunks;                // ceil(qt / qb)
};

// monotone float <-> int mapping so integer comparisons and atomicMax work on scores
__device__ __forceinline__ int f2ord(float f) {
  const int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// Key descriptor rows (KV blocks x R) from which the persistent form is preferred. 0 = always.
#ifndef SB_STREAM_MIN_KEY_ROWS
#define SB_STREAM_MIN_KEY_ROWS 0
#endif
constexpr long long STREAM_MIN_KEY_ROWS = SB_STREAM_MIN_KEY_ROWS;

// Persistent form (indexer_summary_stream.cu). Returns SB_OK when it ran, 1 when the problem
// is not eligible, negative on error. `p` arrives with everything but qb / q_chunks filled in.
int launch_summary_stream(const void* qd, const void* kd, Params p, int batch, DeviceCtx* ctx, cudaStream_t stream);

}  // namespace stc
}  // namespace sb
