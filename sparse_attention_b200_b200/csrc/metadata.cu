// Scheduling metadata for the KV-centric operator: cut every selection list
// into KV-range segments. Segment s owns KV blocks [s*W, (s+1)*W),
// W = ceil(kv_blocks / nseg); the ids a segment owns keep their original order
// and are packed to the front of seg_ids[s, list, :], the tail repeats the
// segment's first block id. One warp per list. Plays the role of the
// reference's reverse index (kv4_build_metadata,
// attention/kv_centric/optimization_round4/gpu_metadata.cu:82-108) for
// per-query-block lists: a (query block, KV range) pair is one task.
// An id outside [0, kv_blocks) sets bit 1 of the error word and is dropped.
#include "internal.h"

namespace sb {
namespace {

__global__ void __launch_bounds__(256) split_segments_kernel(const int32_t* __restrict__ ids,
                                                             const int32_t* __restrict__ counts,
                                                             int32_t* __restrict__ seg_ids,
                                                             int32_t* __restrict__ seg_counts, int* __restrict__ error,
                                                             long long lists, int topk, int kv_blocks, int nseg) {
  const int lane = threadIdx.x & 31;
  const long long list = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (list >= lists) return;
  const int width = (kv_blocks + nseg - 1) / nseg;
  int live = counts ? counts[list] : topk;
  live = min(max(live, 0), topk);
  const int32_t* src = ids + list * topk;
  for (int s = 0; s < nseg; ++s) {
    const int lo = s * width, hi = min(lo + width, kv_blocks);
    int32_t* dst = seg_ids + (static_cast<long long>(s) * lists + list) * topk;
    int kept = 0;
    for (int base = 0; base < live; base += 32) {
      const int i = base + lane;
      const int id = (i < live) ? src[i] : -1;
      if (s == 0 && i < live && (id < 0 || id >= kv_blocks)) atomicOr(error, 1);
      const bool mine = (i < live) && id >= lo && id < hi;
      const unsigned ballot = __ballot_sync(0xffffffffu, mine);
      if (mine) dst[kept + __popc(ballot & ((1u << lane) - 1u))] = id;
      kept += __popc(ballot);
    }
    for (int i = kept + lane; i < topk; i += 32) dst[i] = lo < kv_blocks ? lo : 0;
    if (lane == 0) seg_counts[static_cast<long long>(s) * lists + list] = kept;
  }
}

}  // namespace

int launch_split_segments(const int32_t* ids, const int32_t* counts, int32_t* seg_ids, int32_t* seg_counts,
                          int* error, long long lists, int topk, int kv_blocks, int nseg, cudaStream_t stream) {
  const long long blocks = (lists + 7) / 8;
  split_segments_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(ids, counts, seg_ids, seg_counts, error,
                                                                           lists, topk, kv_blocks, nseg);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
