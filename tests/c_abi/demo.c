/*
 * The C ABI used from plain C99, without Python or PyTorch: allocates a small paged cache
 * with the CUDA runtime, writes rows through lms_reshape_and_cache, duplicates blocks with
 * lms_copy_blocks_host, derives a step's index arrays with lms_build_step_indices, and checks
 * everything on the host.  Built and run by
 * tests/test_c_abi_from_c.py; exit code 0 = all checks passed.
 */
#include <cuda_runtime_api.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "lmserve_kv.h"
#include "lmserve_kv_bench.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
  fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 2; } } while (0)
#define CHECK_LMS(x) do { int s_ = (x); if (s_ != LMS_OK) { \
  fprintf(stderr, "%s: %s %s\n", #x, lms_strerror(s_), lms_last_cuda_error()); return 3; } } while (0)

int main(void) {
  enum { NB = 8, BS = 4, ROW = 64, T = 5 };           /* 64-byte rows, 4 slots per block */
  const int64_t chunk = 2 * BS * ROW;                  /* K plane + V plane of one block */
  unsigned char *cache, *key, *value;
  int64_t *slots;
  unsigned char h_key[T * ROW], h_val[T * ROW], h_cache[NB * 2 * BS * ROW];
  const int64_t h_slots[T] = {5, -1, 0, 31, 14};
  const int64_t pairs[4] = {1, 6, 1, 2};               /* block 1 -> blocks 6 and 2 */
  int t, i, bad = 0;

  if (lms_version() != LMS_VERSION) return 1;
  for (i = 0; i < T * ROW; ++i) { h_key[i] = (unsigned char)(i * 7 + 1); h_val[i] = (unsigned char)(i * 13 + 5); }
  CHECK_CUDA(cudaMalloc((void**)&cache, NB * chunk));
  CHECK_CUDA(cudaMalloc((void**)&key, sizeof h_key));
  CHECK_CUDA(cudaMalloc((void**)&value, sizeof h_val));
  CHECK_CUDA(cudaMalloc((void**)&slots, sizeof h_slots));
  CHECK_CUDA(cudaMemset(cache, 0, NB * chunk));
  CHECK_CUDA(cudaMemcpy(key, h_key, sizeof h_key, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(value, h_val, sizeof h_val, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(slots, h_slots, sizeof h_slots, cudaMemcpyHostToDevice));

  CHECK_LMS(lms_init_device());
  CHECK_LMS(lms_reshape_and_cache(key, value, ROW, ROW, cache, cache + BS * ROW, chunk, ROW,
                                  slots, T, ROW, BS, NB * BS, NULL));
  CHECK_LMS(lms_copy_blocks_host(cache, NB * chunk, chunk, chunk, 1, pairs, 2, NB, NULL));
  CHECK_LMS(lms_check_device_errors(NULL, NULL, NULL));
  CHECK_CUDA(cudaMemcpy(h_cache, cache, sizeof h_cache, cudaMemcpyDeviceToHost));

  for (t = 0; t < T; ++t) {
    const int64_t s = h_slots[t];
    const unsigned char *k, *v;
    if (s < 0) continue;
    k = h_cache + (s / BS) * chunk + (s % BS) * ROW;
    v = k + BS * ROW;
    if (memcmp(k, h_key + t * ROW, ROW) || memcmp(v, h_val + t * ROW, ROW)) ++bad;
  }
  /* slot 5 lives in block 1, which was copied to blocks 6 and 2 */
  if (memcmp(h_cache + 6 * chunk, h_cache + 1 * chunk, chunk)) ++bad;
  if (memcmp(h_cache + 2 * chunk, h_cache + 1 * chunk, chunk)) ++bad;
  /* padded token 1 wrote nothing: block 4 is still zero */
  for (i = 0; i < chunk; ++i) if (h_cache[4 * chunk + i]) { ++bad; break; }
  /* argument errors come back as statuses */
  if (lms_reshape_and_cache(key + 1, value, ROW, ROW, cache, cache, chunk, ROW, slots, T, ROW, BS, 0, NULL) != LMS_ERR_ALIGN) ++bad;
  if (lms_copy_blocks_host(cache, NB * chunk, chunk, chunk, 1, NULL, 2, NB, NULL) != LMS_ERR_NULL) ++bad;
  {
    /* three requests, sorted by descending input_len: a 4-token prefill chunk (14 cached
       tokens, blocks 3 and 8), a decode at position 16 (blocks 5, 9), a decode at position 2
       (block 6); page size 16 */
    enum { B = 3, TOK = 6, NBLK = 5 };
    const int32_t h_in[4 * B + NBLK] = {4, 1, 1, 14, 16, 2, 18, 17, 3, 2, 2, 1, 3, 8, 5, 9, 6};
    const int64_t want_slots[TOK] = {3 * 16 + 14, 3 * 16 + 15, 8 * 16, 8 * 16 + 1, 9 * 16, 6 * 16 + 2};
    const int32_t want_cu[B + 1] = {0, 4, 5, 6};
    int32_t *d_in, *d_cu, h_cu[B + 1];
    int64_t *d_slots, h_out[TOK];
    CHECK_CUDA(cudaMalloc((void**)&d_in, sizeof h_in));
    CHECK_CUDA(cudaMalloc((void**)&d_cu, sizeof h_cu));
    CHECK_CUDA(cudaMalloc((void**)&d_slots, sizeof h_out));
    CHECK_CUDA(cudaMemcpy(d_in, h_in, sizeof h_in, cudaMemcpyHostToDevice));
    CHECK_LMS(lms_build_step_indices(d_in, d_in + B, d_in + 2 * B, d_in + 3 * B, d_in + 4 * B, NULL,
                                     B, TOK, NBLK, 16, NULL, d_cu, NULL, NULL, NULL, NULL, NULL,
                                     d_slots, NULL, 1, 2, NULL, NULL));
    CHECK_CUDA(cudaMemcpy(h_out, d_slots, sizeof h_out, cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(h_cu, d_cu, sizeof h_cu, cudaMemcpyDeviceToHost));
    if (memcmp(h_out, want_slots, sizeof h_out) || memcmp(h_cu, want_cu, sizeof h_cu)) ++bad;
    if (lms_build_step_indices(d_in, d_in + B, d_in + 2 * B, d_in + 3 * B, d_in + 4 * B, NULL,
                               LMS_STEP_MAX_BATCH + 1, TOK, NBLK, 16, NULL, d_cu, NULL, NULL, NULL,
                               NULL, NULL, d_slots, NULL, 0, 0, NULL, NULL) != LMS_ERR_TOO_LARGE) ++bad;
    cudaFree(d_in); cudaFree(d_cu); cudaFree(d_slots);
  }
  printf("c abi demo: %s, %lld launches\n", bad ? "FAILED" : "ok", (long long)lms_launch_count());
  cudaFree(cache); cudaFree(key); cudaFree(value); cudaFree(slots);
  return bad ? 4 : 0;
}
