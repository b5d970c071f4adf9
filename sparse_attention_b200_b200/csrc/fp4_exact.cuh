// Exact NVFP4 scoring arithmetic shared by the plain scorer and by the re-scoring
// stage of the tensor-core indexer. With integer codes c = 2 * e2m1 value,
//   t_g = (sum_{i in 16-feature group g} cq_i * ck_i) * (0.25 * qs_g * ks_g)   exact in fp32
//   dot = ((t_0 + t_1) + t_2) + ... + t_7                                       fp32, in order
// A 128 x 128 (query tile x key page) block is computed by 256 threads, thread
// (ty, tx) = (tid / 16, tid % 16) owning queries ty*8..ty*8+7 and keys tx + 16*j.
#pragma once
#include <cuda_fp8.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace sb {

constexpr int FP4_ROW_WORDS = 36;   // 128 int8 = 32 words, padded to 36 for conflict-free 16-byte reads

__device__ __forceinline__ float e4m3_to_float(uint8_t bits) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(bits, __NV_E4M3)));
}
// eight e2m1 codes (one 32-bit word) -> eight signed bytes 2*value, as two dp4a operands
__device__ __forceinline__ void codes_to_int8(uint32_t w, uint32_t& lo4, uint32_t& hi4) {
  const unsigned long long lut = 0x0C08060403020100ULL;
  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t c = (w >> (4 * i)) & 15u;
    int m = static_cast<int>((lut >> (8 * (c & 7u))) & 0xFFu);
    if (c & 8u) m = -m;
    out[i >> 2] |= (static_cast<uint32_t>(m) & 0xFFu) << (8 * (i & 3));
  }
  lo4 = out[0];
  hi4 = out[1];
}

// Stage 128 index vectors (codes row pitch `code_pitch` bytes, scales row pitch
// `scale_pitch` bytes) as int8 rows + fp32 scales (times `fold`). All threads of the block.
__device__ __forceinline__ void fp4_stage_rows(uint32_t* rows_i8, float* rows_sc, const uint8_t* codes,
                                               long long code_pitch, const uint8_t* scales, long long scale_pitch,
                                               float fold) {
  for (int e = threadIdx.x; e < 128 * 16; e += blockDim.x) {
    const int r = e >> 4, w = e & 15;
    const uint32_t word = __ldg(reinterpret_cast<const uint32_t*>(codes + r * code_pitch + w * 4));
    uint32_t a, c;
    codes_to_int8(word, a, c);
    rows_i8[r * FP4_ROW_WORDS + 2 * w] = a;
    rows_i8[r * FP4_ROW_WORDS + 2 * w + 1] = c;
  }
  for (int e = threadIdx.x; e < 128 * 8; e += blockDim.x)
    rows_sc[e] = fold * e4m3_to_float(scales[(e >> 3) * scale_pitch + (e & 7)]);
}

// The 8 x 8 dots of thread (ty, tx); q scales must carry the 0.25 factor.
__device__ __forceinline__ void fp4_block_dots(const uint32_t* q_i8, const float* q_sc, const uint32_t* k_i8,
                                               const float* k_sc, int ty, int tx, float (&acc)[8][8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
#pragma unroll 1
  for (int g = 0; g < 8; ++g) {
    uint4 qv[8], kv[8];
    float qsc[8], ksc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      qv[i] = *reinterpret_cast<const uint4*>(&q_i8[(ty * 8 + i) * FP4_ROW_WORDS + g * 4]);
      qsc[i] = q_sc[(ty * 8 + i) * 8 + g];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      kv[j] = *reinterpret_cast<const uint4*>(&k_i8[(tx + 16 * j) * FP4_ROW_WORDS + g * 4]);
      ksc[j] = k_sc[(tx + 16 * j) * 8 + g];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // The integer sum is accumulated on top of the bit pattern of 1.5 * 2^23: the result
        // IS the float 12582912 + sum (|sum| <= 2304), and one exact subtraction gives
        // float(sum) without an int-to-float conversion (a quarter-rate instruction).
        int isum = __dp4a(static_cast<int>(qv[i].x), static_cast<int>(kv[j].x), 0x4B400000);
        isum = __dp4a(static_cast<int>(qv[i].y), static_cast<int>(kv[j].y), isum);
        isum = __dp4a(static_cast<int>(qv[i].z), static_cast<int>(kv[j].z), isum);
        isum = __dp4a(static_cast<int>(qv[i].w), static_cast<int>(kv[j].w), isum);
        // exact product (<= 12 + 8 significant bits), one rounding in the add
        acc[i][j] = fmaf(__int_as_float(isum) - 12582912.0f, qsc[i] * ksc[j], acc[i][j]);
      }
  }
}

}  // namespace sb
