/*
 * lmserve_kv_bench.h — measurement and test instruments of liblmserve_kv.so.
 *
 * Not part of the drop-in boundary (include/lmserve_kv.h): these entry points exist so that
 * the benchmark can sweep launch parameters and count launches, and so that the tests can
 * exercise the bounded device-side wait.  A deployment does not need this header.  None of
 * them has a counterpart in the reference.
 */
#ifndef LMSERVE_KV_BENCH_H_
#define LMSERVE_KV_BENCH_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Tunables for lms_set_tuning (a negative value restores the built-in choice; for the
 * non-variant keys 0 does too). */
#define LMS_TUNE_WRITE_VARIANT 1 /* 0 = tiled 16-byte ld/st, 1 = tiled 32-byte, 2 = bulk-copy (TMA) rows,
                                    3 = untiled one-vector-per-thread 32-byte, 4 = untiled 16-byte,
                                    5 = one wave: a thread moves the K and the V vector of
                                    LMS_TUNE_WRITE_VPT (1, 2, 4) tokens, 6 = one wave: a thread moves
                                    LMS_TUNE_WRITE_VPT independent vectors, 7 = as 5 on a persistent
                                    grid with a two-deep register pipeline */
#define LMS_TUNE_WRITE_TILE_BYTES 2 /* payload bytes read per CTA of the tiled cache write; for variant 7
                                       the CTAs per SM of the persistent grid */
#define LMS_TUNE_COPY_VARIANT 3  /* 0 = persistent 16-byte ld/st, 1 = persistent 32-byte, 2 = bulk-copy (TMA),
                                    3 = untiled one-vector-per-thread, 4 = persistent 16-byte with
                                    1024-thread CTAs (128 KiB in flight per CTA, for grids of a few CTAs) */
#define LMS_TUNE_COPY_CTAS_PER_SM 4
#define LMS_TUNE_SWAP_OUT_CTAS 5 /* total CTAs of the GPU->host kernel; built-in 3 (of 1024 threads), which
                                    fills a PCIe Gen5 x16 link and leaves the SMs to concurrent GEMMs -
                                    raise it on a faster host link */
#define LMS_TUNE_SWAP_IN_CTAS 6  /* total CTAs of the host->GPU kernel */
#define LMS_TUNE_XFER_CTAS_PER_SM 7
#define LMS_TUNE_XFER_VARIANT 8  /* as LMS_TUNE_COPY_VARIANT */
#define LMS_TUNE_WRITE_VPT 9     /* vectors per thread per pipeline batch of the cache write: 2, 4, 8 */
#define LMS_TUNE_SWAP_VARIANT 10 /* as LMS_TUNE_COPY_VARIANT, both directions */
#define LMS_TUNE_WRITE_PDL 11    /* 1 (built-in) = launch the untiled cache write, the untiled chunk copy and the rotary kernel
                                    with programmatic stream serialization: the grid becomes resident
                                    while the previous kernel drains and still waits for that kernel
                                    before touching memory, so stream order is unchanged; 2 = off */
#define LMS_TUNE_SWAP_ENGINE 12  /* lms_swap_blocks_host only: 1 (built-in) = the SM kernel, 2 = the copy
                                    engines: one strided DMA copy per block (all layers of the range),
                                    no SM is used, so a concurrent GEMM keeps every SM */
#define LMS_TUNE_WRITE_PREFETCH 13 /* 1 (built-in) = the untiled cache-write kernels prefetch their source
                                     lines into L2 before the programmatic-launch wait (a hint: it
                                     cannot change a result); 2 = off */
#define LMS_TUNE_STAGED_STREAMS 14 /* copy streams lms_swap_blocks_staged spreads its transfers over: 1
                                      (built-in) or 2 */
#define LMS_TUNE__COUNT 15

/* Overrides a launch tunable for every later call in this process. */
int lms_set_tuning(int key, int value);
int lms_get_tuning(int key);

/* Name of the kernel a cache write of `row_bytes`-byte rows and `total_bytes` payload bytes
 * would launch under the current tuning ("write_rows_direct", "write_rows_pair", ...): lets the
 * benchmark label its numbers with the kernel that produced them. */
const char* lms_write_kernel_name(int64_t row_bytes, int64_t total_bytes);

/*
 * Self-test of the bounded device-side wait used by the bulk-copy (TMA) kernel variants: one
 * warp waits on a shared-memory barrier that nothing ever completes, gives up after
 * `limit_us` microseconds, records the time-out in the device error record and returns.  The
 * kernel neither traps nor spins forever, and the context stays usable;
 * lms_check_device_errors afterwards returns LMS_ERR_CUDA with a "gave up waiting" message.
 * `limit_us` is clamped to [1, 1000000].  No counterpart in the reference.
 */
int lms_selftest_bounded_wait(int64_t limit_us, void* stream);

/*
 * Plain cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault) on `stream`: the copy-engine
 * baseline the swap and transfer kernels are measured against (one contiguous DMA).  No
 * counterpart in the reference, which issues its copies through pycuda
 * (runtime/worker/llm_worker/kv_worker.py:206-211,222-227).
 */
int lms_memcpy_async(void* dst, const void* src, int64_t bytes, void* stream);

/* Number of kernels this library has launched in this process (all threads). */
int64_t lms_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* LMSERVE_KV_BENCH_H_ */
