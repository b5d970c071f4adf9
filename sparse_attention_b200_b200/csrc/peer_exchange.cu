// Cross-GPU merge of the KV-range split without a copy step: every rank keeps its partial
// (O_r, LSE_r) in memory that the other ranks of the machine have mapped (CUDA IPC over
// NVLink), tells them with a flag word when the partial is complete, and the merge kernel of
// the rank that owns a slice of rows reads the R partials of that slice where they lie - its
// own from local memory, the others with plain loads from the peers' memory - and writes
// the merged rows. No library kernel touches peer memory, no multicast, and every wait on a
// flag that another GPU writes has a time limit after which the kernel records a status code
// and returns.
//
// Protocol of one step (epoch e = 1, 2, ...), all on one stream per rank:
//   peer_wait(done[*] >= e - 1)      every reader of my previous partial has finished
//   attention kernel                 writes my partial into my exchange memory
//   peer_signal(ready[me] := e)      into every rank's flag block (after the kernel, stream order)
//   combine_peer(waits ready[*] >= e, then merges my slice of rows from all R partials)
//   peer_signal(done[me] := e)       into every rank's flag block
// The flag words a rank polls live in its OWN memory; peers write them remotely.
//
// The reference has no multi-GPU path; this serves the KV split of the 1 Mi-token
// configuration next to the NCCL send/recv form (sharding.py).
#include "internal.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <cstdint>
#include <cstring>

namespace sb {
namespace {

constexpr int MAX_PEERS = 8;
constexpr int CODE_WAIT_KERNEL = 0xb00;    // status codes of the two waits (peer_wait, combine_peer)
constexpr int CODE_COMBINE = 0xb10;

struct PeerPtrs {
  const __nv_bfloat16* part[MAX_PEERS];    // [rows, 128] bf16, already at the first row of the slice
  const float* lse[MAX_PEERS];             // [rows]
};
struct FlagPtrs {
  int32_t* word[2 * MAX_PEERS];
};

__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// plain (coherent) 16-byte and 4-byte loads: the data was written by another GPU during this kernel's lifetime
__device__ __forceinline__ uint4 ld_plain_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_plain_f32(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// One thread: waits until each of n flag words is >= value. False (and the status word set) when limit_ns ran out.
__device__ bool wait_flags(const int32_t* flags, int n, int value, unsigned long long limit_ns, int* status, int code) {
  const unsigned long long t0 = global_ns();
  for (int i = 0; i < n; ++i) {
    int spins = 0;
    while (ld_acquire_sys(flags + i) < value) {
      if ((++spins & 63) == 0) {
        if (*reinterpret_cast<volatile int*>(status) != 0) return false;      // another CTA already gave up
        if (global_ns() - t0 > limit_ns) {
          atomicCAS(status, 0, code + i);
          return false;
        }
        __nanosleep(200);
      }
    }
  }
  return true;
}

__global__ void peer_signal_kernel(FlagPtrs f, int n, int value) {
  if (threadIdx.x < n) {
    __threadfence_system();                  // everything earlier on this stream is visible before the flag
    st_release_sys(f.word[threadIdx.x], value);
  }
}

__global__ void peer_wait_kernel(const int32_t* flags, int n, int value, unsigned long long limit_ns, int* status) {
  if (threadIdx.x == 0) wait_flags(flags, n, value, limit_ns, status, CODE_WAIT_KERNEL);
}

// Sixteen threads per row, eight features each; the operations and their order are those of the
// single-GPU Combine kernels (combine.cu), so the merged rows equal the send/recv form bit for bit.
template <int R>
__global__ void __launch_bounds__(256) combine_peer_kernel(PeerPtrs src, const int32_t* ready, int value,
                                                           unsigned long long limit_ns, int* status,
                                                           __nv_bfloat16* __restrict__ out, float* __restrict__ out_lse,
                                                           long long rows) {
  __shared__ int go;
  if (ready != nullptr) {
    if (threadIdx.x == 0) go = wait_flags(ready, R, value, limit_ns, status, CODE_COMBINE) ? 1 : 0;
    __syncthreads();
    if (!go) return;
  }
  const int slot = threadIdx.x >> 4, part = threadIdx.x & 15;
  const long long row = static_cast<long long>(blockIdx.x) * 16 + slot;
  if (row >= rows) return;
  uint4 raw[R];
  float L[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    raw[r] = ld_plain_v4(src.part[r] + row * 128 + part * 8);
    L[r] = ld_plain_f32(src.lse[r] + row);
  }
  float maximum = L[0];
#pragma unroll
  for (int r = 1; r < R; ++r) maximum = fmaxf(maximum, L[r]);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float denom = 0.f;
  if (maximum > -CUDART_INF_F) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float w = expf(L[r] - maximum);            // exp(-inf) = 0
      if (!(w > 0.f)) raw[r] = make_uint4(0u, 0u, 0u, 0u);   // a rank of weight 0 is dropped, whatever it holds
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
      denom += w;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(h[i]);
        acc[2 * i] = fmaf(w, x.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(w, x.y, acc[2 * i + 1]);
      }
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

template <int R>
void launch_r(const PeerPtrs& src, const int32_t* ready, int value, unsigned long long limit_ns, int* status, void* out,
              float* out_lse, long long rows, cudaStream_t stream) {
  combine_peer_kernel<R><<<static_cast<unsigned>((rows + 15) / 16), 256, 0, stream>>>(
      src, ready, value, limit_ns, status, static_cast<__nv_bfloat16*>(out), out_lse, rows);
}

unsigned long long to_ns(int wait_ms) {
  return static_cast<unsigned long long>(wait_ms < 1 ? 1 : wait_ms) * 1000000ULL;
}

}  // namespace

int peer_alloc(long long bytes, void** ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is handed around as 64 bytes");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  }
  std::memcpy(handle64, &h, 64);
  *ptr = p;
  return SB_OK;
}

int peer_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return set_error(SB_ERR_CUDA, cudaGetErrorString(e));
  *ptr = p;
  return SB_OK;
}

int peer_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

int peer_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

int launch_peer_signal(int32_t* const* flags, int n, int value, cudaStream_t stream) {
  if (n < 1 || n > 2 * MAX_PEERS) return set_error(SB_ERR_INVALID, "1 to 16 flag words per signal");
  FlagPtrs f{};
  for (int i = 0; i < n; ++i) {
    if (!flags[i]) return set_error(SB_ERR_INVALID, "null flag pointer");
    f.word[i] = flags[i];
  }
  peer_signal_kernel<<<1, 32, 0, stream>>>(f, n, value);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

int launch_peer_wait(const int32_t* flags, int n, int value, int wait_ms, cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  peer_wait_kernel<<<1, 32, 0, stream>>>(flags, n, value, to_ns(wait_ms), ctx->status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

int launch_combine_peer(const void* const* partials, const float* const* lses, const int32_t* ready, int value,
                        int wait_ms, void* out, float* out_lse, long long rows, int ranks, cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  if (ranks != 1 && ranks != 2 && ranks != 4 && ranks != 8)
    return set_error(SB_ERR_INVALID, "the peer merge is compiled for 1, 2, 4 and 8 ranks");
  if ((rows + 15) / 16 > 0x7fffffffLL) return set_error(SB_ERR_INVALID, "too many rows for one combine launch");
  PeerPtrs src{};
  for (int r = 0; r < ranks; ++r) {
    if (!partials[r] || !lses[r] || (reinterpret_cast<uintptr_t>(partials[r]) & 15u))
      return set_error(SB_ERR_INVALID, "partials must be 16-byte aligned device pointers, one per rank");
    src.part[r] = static_cast<const __nv_bfloat16*>(partials[r]);
    src.lse[r] = lses[r];
  }
  const unsigned long long ns = to_ns(wait_ms);
  switch (ranks) {
    case 1: launch_r<1>(src, ready, value, ns, ctx->status, out, out_lse, rows, stream); break;
    case 2: launch_r<2>(src, ready, value, ns, ctx->status, out, out_lse, rows, stream); break;
    case 4: launch_r<4>(src, ready, value, ns, ctx->status, out, out_lse, rows, stream); break;
    default: launch_r<8>(src, ready, value, ns, ctx->status, out, out_lse, rows, stream); break;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
