/* libsparse_b200.so -- C ABI of the B200 block-sparse attention hot path.
 *
 * Plain pointers and sizes only. Every pointer is a DEVICE pointer unless the
 * comment says otherwise; `stream` is a cudaStream_t passed as void*. Calls are
 * asynchronous on that stream, never synchronise, never throw. Return value:
 * 0 on success, negative on error (SPARSE_B200_ERR_*), with a message from
 * sparse_b200_last_error(). The device that is current when a function is
 * called is the device it launches on.
 *
 * Layouts (d = 128, bf16 unless stated, all contiguous):
 *   q, out        [B, Hq, Sq, 128]
 *   k, v          [B, Hkv, Skv, 128]
 *   block_idx     [B, Hkv, Sq/128, TopK] int32: KV-block ids chosen for a query
 *                 block, shared by the Hq/Hkv query heads of the KV-head group
 *   block_count   [B, Hkv, Sq/128] int32 or NULL: live entries per list
 *   lse           [B, Hq, Sq] fp32, natural log, or NULL
 */
#ifndef SPARSE_B200_H
#define SPARSE_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPARSE_B200_OK 0
#define SPARSE_B200_ERR_INVALID (-1)
#define SPARSE_B200_ERR_CUDA (-2)
#define SPARSE_B200_ERR_TIMEOUT (-3)

/* Text of the last error raised on the calling thread (host pointer). */
const char* sparse_b200_last_error(void);

/* Reads (and with reset != 0 clears) the device status word. 0 = healthy;
 * a positive value names the bounded wait a kernel abandoned. Synchronises the
 * device; meant for tests and post-mortems, not for the hot path. */
int sparse_b200_device_status(int reset);

/* Q-centric block-sparse attention forward.
 * Replaces the launch functions behind xomtention_progression::attention_out
 * (attention/q_centric/progression_attention.cpp:11-15, 96-108:
 * dense14_sparse_two_q_launch / dense14_sparse_gqa_launch), same argument
 * order with block_count and lse added. Group sizes Hq/Hkv that are even share
 * each selected K/V tile between two heads; others pair neighbouring query
 * blocks. A list with count 0 yields out = 0 and lse = -inf. */
int sparse_b200_q_centric(const void* q, const void* k, const void* v, const int32_t* block_idx,
                          const int32_t* block_count, void* out, float* lse, int batch, int hq, int hkv,
                          int sq, int skv, int topk, void* stream);

/* Same kernel over `nseg` list sets at once, writing normalised partial
 * outputs [nseg, B, Hq, Sq, 128] (bf16, or fp32 when partial_is_f32) and
 * partial LSE [nseg, B, Hq, Sq]. seg_block_idx is [nseg, B, Hkv, Sq/128, TopK],
 * seg_block_count [nseg, B, Hkv, Sq/128]. This is the "main" stage of the
 * KV-centric operator (role of kv11_launch,
 * attention/kv_centric/optimization_round11/tma11_kernel.cu:439-452): segment
 * s holds the ids of one KV range, segments run KV-range-outer. */
int sparse_b200_q_centric_partial(const void* q, const void* k, const void* v, const int32_t* seg_block_idx,
                                  const int32_t* seg_block_count, void* partial_out, float* partial_lse,
                                  int nseg, int partial_is_f32, int batch, int hq, int hkv, int sq, int skv,
                                  int topk, void* stream);

#ifdef __cplusplus
}
#endif
#endif
