// C-ABI of libsparse_b200.so: argument checks, per-device state, error text.
// No entry point throws, synchronises the device or allocates on the stream
// path (the only allocation is a 4-byte status word per device, on first use).
#include "internal.h"
#include "../../include/sparse_b200.h"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace sb {

static thread_local char g_error[512] = "";

int set_error(int code, const char* message) {
  snprintf(g_error, sizeof(g_error), "%s", message ? message : "");
  return code;
}

static std::mutex g_mutex;
static DeviceCtx g_ctx[64];
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn g_encode = nullptr;

DeviceCtx* device_ctx() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error(SB_ERR_CUDA, "no current CUDA device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceCtx& c = g_ctx[dev];
  if (c.device == dev) return &c;
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
      set_error(SB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
      return nullptr;
    }
    g_encode = reinterpret_cast<EncodeFn>(fn);
  }
  if (cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaMalloc(&c.status, sizeof(int)) != cudaSuccess ||
      cudaMemset(c.status, 0, sizeof(int)) != cudaSuccess) {
    set_error(SB_ERR_CUDA, "device state initialisation failed");
    return nullptr;
  }
  c.device = dev;
  return &c;
}

int encode_tiled(CUtensorMap* map, CUtensorMapDataType type, int rank, void* ptr, const cuuint64_t* dims,
                 const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* steps,
                 CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo) {
  if (!g_encode) return 1;
  CUresult r = g_encode(map, type, rank, ptr, dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace sb

using namespace sb;

#define REQUIRE(cond, msg) \
  do {                     \
    if (!(cond)) return set_error(SB_ERR_INVALID, msg); \
  } while (0)

extern "C" {

const char* sparse_b200_last_error(void) { return g_error; }

int sparse_b200_device_status(int reset) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  int value = 0;
  if (cudaMemcpy(&value, ctx->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return set_error(SB_ERR_CUDA, "status read failed");
  if (reset && value != 0) cudaMemset(ctx->status, 0, sizeof(int));
  return value;
}

static int check_attention(const void* q, const void* k, const void* v, const int32_t* block_idx,
                           const void* out, int batch, int hq, int hkv, int sq, int skv, int topk, int nseg) {
  REQUIRE(q && k && v && block_idx && out, "q, k, v, block_idx and out must be non-null device pointers");
  REQUIRE(batch > 0 && hkv > 0, "batch and KV heads must be positive");
  REQUIRE(hq >= hkv && hq % hkv == 0, "Hq must be a multiple of and at least Hkv");
  REQUIRE(sq >= 128 && sq % 128 == 0, "Sq must be a positive multiple of 128");
  REQUIRE(skv >= 128 && skv % 128 == 0, "Skv must be a positive multiple of 128");
  REQUIRE(topk > 0, "selected_count must be positive");
  REQUIRE(topk <= skv / 128, "selected_count cannot exceed the number of KV tiles");
  REQUIRE(nseg >= 1, "segment count must be positive");
  REQUIRE(static_cast<long long>(batch) * hq * sq < (1LL << 31) &&
              static_cast<long long>(batch) * hkv * skv < (1LL << 31),
          "flattened Q / KV row counts must fit int32 (TMA row coordinates)");
  REQUIRE(static_cast<long long>(nseg) * batch * hkv * (sq / 128) * topk < (1LL << 40), "block_idx too large");
  REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), "q, k, v, out must be 16-byte aligned");
  REQUIRE(out != q && out != k && out != v && out != static_cast<const void*>(block_idx),
          "output must not alias inputs");
  return SB_OK;
}

int sparse_b200_q_centric(const void* q, const void* k, const void* v, const int32_t* block_idx,
                          const int32_t* block_count, void* out, float* lse, int batch, int hq, int hkv,
                          int sq, int skv, int topk, void* stream) {
  int rc = check_attention(q, k, v, block_idx, out, batch, hq, hkv, sq, skv, topk, 1);
  if (rc) return rc;
  QCentricArgs a{q, k, v, block_idx, block_count, out, lse, batch, hq, hkv, sq, skv, topk, 1, 0};
  return launch_q_centric(a, static_cast<cudaStream_t>(stream));
}

int sparse_b200_q_centric_partial(const void* q, const void* k, const void* v, const int32_t* seg_block_idx,
                                  const int32_t* seg_block_count, void* partial_out, float* partial_lse,
                                  int nseg, int partial_is_f32, int batch, int hq, int hkv, int sq, int skv,
                                  int topk, void* stream) {
  int rc = check_attention(q, k, v, seg_block_idx, partial_out, batch, hq, hkv, sq, skv, topk, nseg);
  if (rc) return rc;
  REQUIRE(seg_block_count && partial_lse, "segment counts and partial LSE are required");
  QCentricArgs a{q, k, v, seg_block_idx, seg_block_count, partial_out, partial_lse,
                 batch, hq, hkv, sq, skv, topk, nseg, partial_is_f32 ? 1 : 0};
  return launch_q_centric(a, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
