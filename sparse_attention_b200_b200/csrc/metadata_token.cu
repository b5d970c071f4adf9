// Per-TOKEN selection lists -> reverse index for the KV-centric token kernel.
//
// selected [B, Hkv, Sq, TopK] int32 holds, for every query token and KV-head group,
// the KV blocks it attends to. The reverse index lists, for every row
// (group = b*Hkv + kvh, block), the (query, rank) edges that chose the block:
//   row_ptr [rows + 1], query_ids [E], ranks [E]   (E = B*Hkv*Sq*TopK edges)
// and cuts every row into tasks of at most 128 / group_size queries:
//   task_ptr [rows + 1] (task_ptr[rows] = number of tasks), tasks [T, 4] =
//   (group, block, first edge, edge count).
// Same structure as the reference's build (kv4_build_metadata,
// attention/kv_centric/optimization_round4/gpu_metadata.cu:82-108; CPU statement
// attention/kv_centric/metadata.py:43-72), for any TopK and block count, with its own
// scans instead of a library call. Edge order inside a row is arbitrary (atomics).
// error word: bit 1 = an id outside [0, kv_blocks).
#include <algorithm>
#include "internal.h"

namespace sb {
namespace {

__global__ void __launch_bounds__(256) count_edges_kernel(const int32_t* __restrict__ selected, int32_t* counts,
                                                          int32_t* error, long long edges, long long group_edges,
                                                          int kv_blocks) {
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < edges;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int key = selected[e];
    if (static_cast<unsigned>(key) < static_cast<unsigned>(kv_blocks))
      atomicAdd(counts + (e / group_edges) * kv_blocks + key, 1);
    else
      atomicOr(error, 1);
  }
}

// Shared-memory variants for up to SMEM_BINS KV blocks: a CTA takes a contiguous span of edges
// (one KV-head group, or a few), histograms it in shared memory and touches global memory once
// per (CTA, non-empty bin) instead of once per edge: with 256 rows and half a million edges the
// per-edge atomics of the plain kernels serialise on a few hundred addresses.
constexpr int SMEM_BINS = 2048;
constexpr int EDGES_PER_CTA = 4096;

__global__ void __launch_bounds__(256) count_edges_smem_kernel(const int32_t* __restrict__ selected, int32_t* counts,
                                                               int32_t* error, long long edges,
                                                               long long group_edges, int kv_blocks) {
  __shared__ int hist[SMEM_BINS];
  const long long e0 = static_cast<long long>(blockIdx.x) * EDGES_PER_CTA;
  const long long e1 = min(edges, e0 + EDGES_PER_CTA);
  for (long long seg = e0; seg < e1;) {
    const long long g = seg / group_edges;
    const long long seg_end = min(e1, (g + 1) * group_edges);
    for (int i = threadIdx.x; i < kv_blocks; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (long long e = seg + threadIdx.x; e < seg_end; e += blockDim.x) {
      const int key = selected[e];
      if (static_cast<unsigned>(key) < static_cast<unsigned>(kv_blocks))
        atomicAdd(&hist[key], 1);
      else
        atomicOr(error, 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kv_blocks; i += blockDim.x)
      if (hist[i] > 0) atomicAdd(counts + g * kv_blocks + i, hist[i]);
    __syncthreads();
    seg = seg_end;
  }
}

__global__ void __launch_bounds__(256) scatter_edges_smem_kernel(const int32_t* __restrict__ selected,
                                                                 const int32_t* __restrict__ row_ptr, int32_t* cursors,
                                                                 int32_t* __restrict__ qids, int32_t* __restrict__ ranks,
                                                                 long long edges, long long group_edges, int kv_blocks,
                                                                 int topk) {
  __shared__ int hist[SMEM_BINS];      // edges of this span per bin, then the running local cursor
  __shared__ int first[SMEM_BINS];     // first slot of this CTA's edges inside the row
  const long long e0 = static_cast<long long>(blockIdx.x) * EDGES_PER_CTA;
  const long long e1 = min(edges, e0 + EDGES_PER_CTA);
  for (long long seg = e0; seg < e1;) {
    const long long g = seg / group_edges;
    const long long seg_end = min(e1, (g + 1) * group_edges);
    for (int i = threadIdx.x; i < kv_blocks; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (long long e = seg + threadIdx.x; e < seg_end; e += blockDim.x) {
      const int key = selected[e];
      if (static_cast<unsigned>(key) < static_cast<unsigned>(kv_blocks)) atomicAdd(&hist[key], 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kv_blocks; i += blockDim.x) {
      const int c = hist[i];
      if (c > 0) first[i] = row_ptr[g * kv_blocks + i] + atomicAdd(cursors + g * kv_blocks + i, c);
      hist[i] = 0;
    }
    __syncthreads();
    for (long long e = seg + threadIdx.x; e < seg_end; e += blockDim.x) {
      const int key = selected[e];
      if (static_cast<unsigned>(key) >= static_cast<unsigned>(kv_blocks)) continue;
      const int dst = first[key] + atomicAdd(&hist[key], 1);
      const long long in_group = e - g * group_edges;
      qids[dst] = static_cast<int32_t>(in_group / topk);
      ranks[dst] = static_cast<int32_t>(in_group % topk);
    }
    __syncthreads();
    seg = seg_end;
  }
}

// Exclusive scan of n + 1 values by one CTA of 1024 threads (n is at most a few 10^5 rows).
// With `capacity` > 0 the scanned values are ceil(in / capacity) (tasks per row).
__global__ void __launch_bounds__(1024) scan_kernel(const int32_t* __restrict__ in, int32_t* __restrict__ out, int n,
                                                    int capacity) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base <= n; base += 1024) {
    const int i = base + threadIdx.x;
    int v = 0;
    if (i < n) v = capacity > 0 ? (in[i] + capacity - 1) / capacity : in[i];
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += o;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int prefix = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - v;
    if (i <= n) out[i] = prefix;
    __syncthreads();
    if (threadIdx.x == 1023) carry = prefix + v;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256) scatter_edges_kernel(const int32_t* __restrict__ selected,
                                                            const int32_t* __restrict__ row_ptr, int32_t* cursors,
                                                            int32_t* __restrict__ qids, int32_t* __restrict__ ranks,
                                                            long long edges, long long group_edges, int kv_blocks,
                                                            int topk) {
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < edges;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int key = selected[e];
    if (static_cast<unsigned>(key) >= static_cast<unsigned>(kv_blocks)) continue;
    const long long row = (e / group_edges) * kv_blocks + key;
    const int dst = row_ptr[row] + atomicAdd(cursors + row, 1);
    const long long in_group = e % group_edges;
    qids[dst] = static_cast<int32_t>(in_group / topk);
    ranks[dst] = static_cast<int32_t>(in_group % topk);
  }
}

// One thread per task. The owning row of task t is the last row whose first task is <= t, found
// by bisection over task_ptr (rows with no edges own no task and are skipped by the search), so a
// row with thousands of tasks is spread over many CTAs. A task record is (KV-head group, KV
// block, first edge, edge count).
__global__ void __launch_bounds__(256) emit_tasks_kernel(const int32_t* __restrict__ row_ptr,
                                                         const int32_t* __restrict__ task_ptr,
                                                         int4* __restrict__ tasks, int rows, int kv_blocks,
                                                         int edges_per_task) {
  const int n_tasks = task_ptr[rows];
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n_tasks; t += gridDim.x * blockDim.x) {
    int lo = 0, hi = rows;                       // invariant: task_ptr[lo] <= t < task_ptr[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (task_ptr[mid] <= t) lo = mid; else hi = mid;
    }
    const int first_edge = row_ptr[lo] + (t - task_ptr[lo]) * edges_per_task;
    const int left = row_ptr[lo + 1] - first_edge;
    tasks[t] = make_int4(lo / kv_blocks, lo % kv_blocks, first_edge, left < edges_per_task ? left : edges_per_task);
  }
}

}  // namespace

// counts / cursors [rows + 1], row_ptr / task_ptr [rows + 1], qids / ranks [E], tasks [max_tasks, 4].
int launch_token_metadata(const int32_t* selected, int32_t* counts, int32_t* cursors, int32_t* row_ptr,
                          int32_t* qids, int32_t* ranks, int32_t* task_ptr, int32_t* tasks, int32_t* error,
                          int groups, int sq, int topk, int kv_blocks, int group_size, cudaStream_t stream) {
  const int rows = groups * kv_blocks;
  const long long group_edges = static_cast<long long>(sq) * topk;
  const long long edges = group_edges * groups;
  const int capacity = 128 / group_size;
  if (cudaMemsetAsync(counts, 0, static_cast<size_t>(rows + 1) * 4, stream) != cudaSuccess ||
      cudaMemsetAsync(cursors, 0, static_cast<size_t>(rows + 1) * 4, stream) != cudaSuccess ||
      cudaMemsetAsync(error, 0, 4, stream) != cudaSuccess)
    return set_error(SB_ERR_CUDA, "memset failed");
  const int grid = static_cast<int>(edges / 256 + 1 < 4096 ? edges / 256 + 1 : 4096);
  const bool in_smem = kv_blocks <= SMEM_BINS && (edges + EDGES_PER_CTA - 1) / EDGES_PER_CTA < (1LL << 30);
  const int span_grid = static_cast<int>((edges + EDGES_PER_CTA - 1) / EDGES_PER_CTA);
  if (in_smem)
    count_edges_smem_kernel<<<span_grid, 256, 0, stream>>>(selected, counts, error, edges, group_edges, kv_blocks);
  else
    count_edges_kernel<<<grid, 256, 0, stream>>>(selected, counts, error, edges, group_edges, kv_blocks);
  scan_kernel<<<1, 1024, 0, stream>>>(counts, row_ptr, rows, 0);
  if (in_smem)
    scatter_edges_smem_kernel<<<span_grid, 256, 0, stream>>>(selected, row_ptr, cursors, qids, ranks, edges,
                                                             group_edges, kv_blocks, topk);
  else
    scatter_edges_kernel<<<grid, 256, 0, stream>>>(selected, row_ptr, cursors, qids, ranks, edges, group_edges,
                                                   kv_blocks, topk);
  scan_kernel<<<1, 1024, 0, stream>>>(counts, task_ptr, rows, capacity);
  const long long task_bound = std::min<long long>((edges + capacity - 1) / capacity + rows, edges);
  const int task_grid = static_cast<int>(std::min<long long>((task_bound + 255) / 256, 2048));
  emit_tasks_kernel<<<task_grid > 0 ? task_grid : 1, 256, 0, stream>>>(row_ptr, task_ptr, reinterpret_cast<int4*>(tasks),
                                                                     rows, kv_blocks, capacity);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
