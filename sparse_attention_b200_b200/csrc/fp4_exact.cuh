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
#include "ptx.cuh"

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

// Maximum over the 16 x 128 (query, key) scores of one warp: queries 16 * warp .. + 15 of the staged
// query tile against the 128 staged keys, with the integer group sums on the tensor cores
// (mma.sync m16n8k16, s8 x s8 -> s32, one scale group per instruction). Same arithmetic as
// fp4_block_dots: acc = fma(float(group sum), qs * ks, acc) in group order, so the scores are
// bit-identical; the accumulator starts at the bit pattern of 1.5 * 2^23 and one exact
// subtraction turns the result into float(group sum). Returns this thread's partial maximum.
__device__ __forceinline__ float fp4_block_max_mma(const uint32_t* q_i8, const float* q_sc, const uint32_t* k_i8,
                                                   const float* k_sc, int warp, int lane) {
  const int gid = lane >> 2, tig = lane & 3, m0 = warp * 16;
  const unsigned long long magic2 = f32x2_pack(12582912.0f, 12582912.0f);
  float m = -INFINITY;
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {         // 64 keys at a time: 32 accumulators per thread
    unsigned long long acc[8][2];
#pragma unroll
    for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = 0ull;
#pragma unroll 1
    for (int g = 0; g < 8; ++g) {
      const uint32_t a0 = q_i8[(m0 + gid) * FP4_ROW_WORDS + g * 4 + tig];
      const uint32_t a1 = q_i8[(m0 + 8 + gid) * FP4_ROW_WORDS + g * 4 + tig];
      const float qs0 = q_sc[(m0 + gid) * 8 + g], qs1 = q_sc[(m0 + 8 + gid) * 8 + g];
      const unsigned long long q0 = f32x2_pack(qs0, qs0), q1 = f32x2_pack(qs1, qs1);
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int key0 = half * 64 + n * 8;
        const uint32_t b0 = k_i8[(key0 + gid) * FP4_ROW_WORDS + g * 4 + tig];
        const unsigned long long kk =
            f32x2_pack(k_sc[(key0 + tig * 2) * 8 + g], k_sc[(key0 + tig * 2 + 1) * 8 + g]);
        int d0, d1, d2, d3;
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};"
            : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
            : "r"(a0), "r"(a1), "r"(b0), "r"(0x4B400000));
        acc[n][0] = f32x2_fma(f32x2_sub(f32x2_pack_bits(d0, d1), magic2), f32x2_mul(q0, kk), acc[n][0]);
        acc[n][1] = f32x2_fma(f32x2_sub(f32x2_pack_bits(d2, d3), magic2), f32x2_mul(q1, kk), acc[n][1]);
      }
    }
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      float x0, x1, x2, x3;
      f32x2_unpack(acc[n][0], x0, x1);
      f32x2_unpack(acc[n][1], x2, x3);
      m = fmaxf(m, fmaxf(fmaxf(x0, x1), fmaxf(x2, x3)));
    }
  }
  return m;
}

}  // namespace sb
