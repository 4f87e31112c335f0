/*
 * lmserve_kv.h — C ABI of the B200 (sm_100a) KV-cache data-movement library.
 *
 * The library replaces the GPU data path of LMServe's Python worker: the paged
 * cache write, the copy-on-write block copy, the GPU<->pinned-host block swap
 * and the prefill->decode block transfer.  LMServe itself has no C interface;
 * each entry point below names the Python callable (path inside the LMServe
 * source tree, file:line) whose device work it performs.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; nothing is allocated, owned or freed on
 *     behalf of the caller unless the function name says so (lms_host_alloc,
 *     lms_ipc_open);
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); work is enqueued asynchronously on it and the call returns
 *     without synchronising;
 *   - the CUDA device of the calling thread must be the device that owns the
 *     (local) cache pointer;
 *   - all byte strides, row sizes and chunk sizes must be multiples of 16 and
 *     all data pointers 16-byte aligned (LMS_ERR_ALIGN otherwise);
 *   - the return value is LMS_OK (0) or a negative lms_status; no exceptions,
 *     no abort, no device-side trap.
 *
 * Paged layout (runtime/worker/llm_worker/model_worker.py:221-228): one GPU
 * tensor [num_layers, num_blocks, 2, block_size, num_kv_heads, head_dim], K in
 * plane 0 and V in plane 1 of every block.  A "row" is one token's K (or V),
 * row_bytes = num_kv_heads*head_dim*elem.  A "chunk" is one (layer, block) =
 * 2*block_size*row_bytes contiguous bytes.  The pinned host pool is
 * block-major, [num_host_blocks, num_layers, chunk]
 * (runtime/worker/llm_worker/kv_worker.py:123-130).
 */
#ifndef LMSERVE_KV_H_
#define LMSERVE_KV_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LMS_VERSION 200 /* major*10000 + minor*100 + patch */

typedef enum lms_status {
  LMS_OK = 0,
  LMS_ERR_NULL = -1,      /* a required pointer is NULL                      */
  LMS_ERR_ALIGN = -2,     /* pointer / stride / size not a multiple of 16    */
  LMS_ERR_RANGE = -3,     /* negative count, empty layer range, bad enum ... */
  LMS_ERR_CUDA = -4,      /* a CUDA runtime call failed (see lms_last_cuda_error) */
  LMS_ERR_INDEX = -5,     /* debug checks: an index was out of range         */
  LMS_ERR_PEER = -6,      /* peer access between the two devices unavailable */
  LMS_ERR_UNSUPPORTED = -7,
  LMS_ERR_TOO_LARGE = -8  /* more pairs than a fixed-size table holds        */
} lms_status;

/* Direction of lms_swap_blocks. */
#define LMS_SWAP_OUT 0 /* GPU  -> host (kv_worker.py "save")  */
#define LMS_SWAP_IN 1  /* host -> GPU  (kv_worker.py "load")  */

/* Library version (LMS_VERSION of the build). */
int lms_version(void);

/* Static, NUL-terminated description of a status code. */
const char* lms_strerror(int status);

/* Text of the last CUDA error seen by the calling thread inside this library. */
const char* lms_last_cuda_error(void);

/*
 * Per-device set-up for the CURRENT device: queries the SM count and allocates the 32-byte
 * device error record (cudaMalloc).  Every entry point does this on its first call on a
 * device; call it explicitly first when that first call would otherwise fall inside a CUDA
 * graph capture, where allocation is not permitted.  Idempotent.
 */
int lms_init_device(void);

/*
 * Debug checks.  When enabled, every kernel verifies each slot / block index
 * against the bounds the caller passed (num_slots, num_*_blocks > 0), skips the
 * offending access instead of performing it, and records the first offender in
 * a per-device error record: 32 bytes of device memory owned by the library,
 * allocated with cudaMalloc by the first call of any entry point on a device
 * (so make that first call outside stream capture).
 * lms_check_device_errors synchronises `stream`, reads the record back, clears
 * it, and returns LMS_ERR_INDEX if a kernel reported an index; `index` / `value`
 * (optional) receive the position in the index table and the bad value.
 */
int lms_set_debug_checks(int enable);
int lms_check_device_errors(void* stream, int64_t* index, int64_t* value);

/*
 * Paged cache write for one layer — replaces
 *   fill_key_cache            runtime/worker/llm_worker/ops/cache_ops.py:39-59
 *   fill_key_cache_kernel     runtime/worker/llm_worker/ops/triton/cache_kernels.py:39-58
 * and the live per-layer call flashinfer.append_paged_kv_cache at
 *   runtime/worker/llm_worker/models/layers/attention.py:76-85.
 *
 * For every token t with slot = slot_mapping[t] >= 0:
 *   key_cache  [(slot / block_size) * block_stride + (slot % block_size) * slot_stride] <- key  [t]
 *   value_cache[ same offset ]                                                         <- value[t]
 * (row_bytes bytes each).  slot < 0 marks padding and is skipped.  Slots must be
 * distinct.  With block_stride = block_size*slot_stride the caches are the flat
 * [num_slots, H, D] arrays of fill_key_cache; with key_cache = &kv[layer][0][0],
 * value_cache = &kv[layer][0][1] and block_stride = chunk bytes they are the
 * interleaved per-layer cache that attention reads.
 * num_slots is used by the debug checks only (0 = unknown).
 */
int lms_reshape_and_cache(const void* key, const void* value,
                          int64_t key_token_stride, int64_t value_token_stride,
                          void* key_cache, void* value_cache,
                          int64_t block_stride, int64_t slot_stride,
                          const int64_t* slot_mapping, int64_t num_tokens,
                          int64_t row_bytes, int32_t block_size,
                          int64_t num_slots, void* stream);

/*
 * The same write for num_layers layers in ONE launch (the per-layer loop of
 * runtime/worker/llm_worker/models/llama.py:236-242 collapsed): layer l reads
 * key + l*key_layer_stride, value + l*value_layer_stride and writes the caches
 * at + l*cache_layer_stride.  slot_layer_stride is in elements; 0 shares one
 * slot_mapping between all layers, as the reference's block tables do.
 */
int lms_reshape_and_cache_layers(const void* key, const void* value,
                                 int64_t key_token_stride, int64_t value_token_stride,
                                 int64_t key_layer_stride, int64_t value_layer_stride,
                                 void* key_cache, void* value_cache,
                                 int64_t cache_layer_stride,
                                 int64_t block_stride, int64_t slot_stride,
                                 const int64_t* slot_mapping, int64_t slot_layer_stride,
                                 int64_t num_tokens, int32_t num_layers,
                                 int64_t row_bytes, int32_t block_size,
                                 int64_t num_slots, void* stream);

/*
 * Planned write.  A decode loop issues the same write — same buffers, refilled in place —
 * once per layer per step, and at 2 MiB per layer the host's argument marshalling costs more
 * than the kernel.  lms_write_plan_create validates and stores the arguments of
 * lms_reshape_and_cache_layers once; lms_write_plan_run enqueues the write on `stream` with
 * the CUDA device the plan was created on current.  The plan holds no device memory and does
 * not own any buffer; destroy it with lms_write_plan_destroy.  (The reference has no such
 * object: it re-derives its launch arguments in Python on every call,
 * runtime/worker/llm_worker/ops/cache_ops.py:46-59.)
 */
typedef struct lms_write_plan lms_write_plan;
int lms_write_plan_create(const void* key, const void* value,
                          int64_t key_token_stride, int64_t value_token_stride,
                          int64_t key_layer_stride, int64_t value_layer_stride,
                          void* key_cache, void* value_cache,
                          int64_t cache_layer_stride,
                          int64_t block_stride, int64_t slot_stride,
                          const int64_t* slot_mapping, int64_t slot_layer_stride,
                          int64_t num_tokens, int32_t num_layers,
                          int64_t row_bytes, int32_t block_size,
                          int64_t num_slots, lms_write_plan** plan);
int lms_write_plan_run(const lms_write_plan* plan, void* stream);
int lms_write_plan_destroy(lms_write_plan* plan);

/*
 * The same write addressed the way the reference's live call site addresses it —
 *   flashinfer.append_paged_kv_cache(key, value, batch_indices, positions, kv_cache,
 *                                    kv_indices, kv_indptr, kv_last_page_len)
 *   runtime/worker/llm_worker/models/layers/attention.py:76-85
 * (flashinfer-python, pinned 0.3.1.post1 by runtime/worker/uv.lock; kernel
 * AppendPagedKVCacheKernel in its include/flashinfer/page.cuh) — so the index tensors that
 * model_worker.py:399-433 already builds are used as they are, all int32 on the device:
 *   page  = kv_indices[kv_indptr[batch_indices[t]] + positions[t] / block_size]
 *   entry = positions[t] % block_size
 *   key_cache  [page * block_stride + entry * slot_stride] <- key[t]   (value likewise)
 * kv_last_page_len plays no part in the write and is not passed.  A negative batch index or
 * position marks padding and is skipped.  num_layers > 1 writes all layers in one launch
 * with the layer strides of lms_reshape_and_cache_layers; the per-layer call of the
 * reference is num_layers = 1.  num_blocks: debug checks only (0 = unknown).
 */
int lms_append_paged_kv_cache(const void* key, const void* value,
                              int64_t key_token_stride, int64_t value_token_stride,
                              int64_t key_layer_stride, int64_t value_layer_stride,
                              const int32_t* batch_indices, const int32_t* positions,
                              void* key_cache, void* value_cache,
                              int64_t cache_layer_stride, int64_t block_stride,
                              int64_t slot_stride, const int32_t* kv_indices,
                              const int32_t* kv_indptr, int64_t num_tokens,
                              int32_t num_layers, int64_t row_bytes,
                              int32_t block_size, int64_t num_blocks, void* stream);

/*
 * lms_append_paged_kv_cache with its arguments validated and resolved once: the per-layer
 * call of runtime/worker/llm_worker/models/layers/attention.py:76-85 passes the same buffers
 * every step (the index arrays are refilled in place), so the plan is built once per layer and
 * lms_write_plan_run is then the whole per-call cost.  Run and destroy with
 * lms_write_plan_run / lms_write_plan_destroy.  `num_requests` = entries of kv_indptr minus
 * one (0 = not known): with it the kernel fetches kv_indptr[t] together with batch_indices[t]
 * and positions[t] on the guess that token t belongs to request t - true for every token of a
 * decode step - which leaves one dependent load (the page id) before the store instead of
 * two; a wrong guess falls back to the plain walk, so the result never depends on it.
 */
int lms_paged_write_plan_create(const void* key, const void* value,
                                int64_t key_token_stride, int64_t value_token_stride,
                                int64_t key_layer_stride, int64_t value_layer_stride,
                                const int32_t* batch_indices, const int32_t* positions,
                                void* key_cache, void* value_cache,
                                int64_t cache_layer_stride, int64_t block_stride,
                                int64_t slot_stride, const int32_t* kv_indices,
                                const int32_t* kv_indptr, int64_t num_requests,
                                int64_t num_tokens, int32_t num_layers, int64_t row_bytes,
                                int32_t block_size, int64_t num_blocks,
                                lms_write_plan** plan);

/*
 * Per-step index preparation on the device — replaces the host-side list building and the ten
 * separate uploads of
 *   ModelWorker._make_inputs      runtime/worker/llm_worker/model_worker.py:310-433
 * including its calls of flashinfer.get_seq_lens and flashinfer.get_batch_indices_positions
 * (model_worker.py:425-433).  The caller sorts the requests as the reference does (descending
 * input_len, model_worker.py:328) and uploads, per request b: input_len[b] (new tokens),
 * filled_len[b] (InferInput.filled_token_len), context_len[b], num_blocks[b] =
 * len(InferInput.block_ids); the block tables concatenated in block_ids[total_blocks]; and
 * optionally the new token ids in token_ids[total_tokens].  All pointers are device pointers
 * (int32, slot_mapping / input_ids int64); any output may be NULL.  One launch writes
 *   cu_seqlens_q[batch+1], kv_block_indptrs[batch+1]   exclusive prefix sums
 *   kv_last_block_lens[b] = (context_len[b]-1) mod block_size + 1      (floor modulo, as Python)
 *   kv_block_indices      = block_ids
 *   position_ids[i]       = filled_len[b] + off          for token i = cu_seqlens_q[b] + off
 *   batch_indices[i] = b, positions[i] = seq_len[b] - input_len[b] + off with
 *                         seq_len[b] = max(num_blocks[b]-1, 0)*block_size + kv_last_block_lens[b]
 *   slot_mapping[i]       = block_ids[kv_block_indptrs[b] + positions[i]/block_size]*block_size
 *                           + positions[i] % block_size, or -1 when that page is not in the
 *                           request's table (reported as LMS_ERR_INDEX with debug checks on)
 *   input_ids[i]          = token_ids[i] widened to int64
 *   decode_kv_block_indptrs[d] = kv_block_indptrs[num_prefill+d] - kv_block_indptrs[num_prefill],
 *                           d = 0..num_decode: the page-table offsets of the decode requests
 *                           alone (requests [num_prefill, num_prefill+num_decode) of the sorted
 *                           batch), which the reference builds a second time for its decode
 *                           attention plan (build_decode_wrapper, model_worker.py:83-140); the
 *                           prefill requests' arrays are prefixes of the batch arrays
 * total_tokens must equal the sum of input_len and total_blocks the sum of num_blocks.
 * batch <= LMS_STEP_MAX_BATCH, else LMS_ERR_TOO_LARGE.
 */
#define LMS_STEP_MAX_BATCH 4096
int lms_build_step_indices(const int32_t* input_len, const int32_t* filled_len,
                           const int32_t* context_len, const int32_t* num_blocks,
                           const int32_t* block_ids, const int32_t* token_ids,
                           int32_t batch, int64_t total_tokens, int64_t total_blocks,
                           int32_t block_size, int32_t* position_ids,
                           int32_t* cu_seqlens_q, int32_t* kv_block_indptrs,
                           int32_t* kv_block_indices, int32_t* kv_last_block_lens,
                           int32_t* batch_indices, int32_t* positions,
                           int64_t* slot_mapping, int64_t* input_ids, int32_t num_prefill,
                           int32_t num_decode, int32_t* decode_kv_block_indptrs, void* stream);

/*
 * Rotary position embedding, optionally fused with the cache write that follows it in the
 * attention layer — replaces
 *   rotary_pos_emb               runtime/worker/llm_worker/ops/rotary_embedding_ops.py:8-38
 *   apply_rotary_pos_emb_kernel  runtime/worker/llm_worker/ops/triton/rotary_embedding.py:5-66
 * and, when key_cache / value_cache are given, the cache write of
 *   runtime/worker/llm_worker/models/layers/attention.py:76-85
 * in the same launch (call order in runtime/worker/llm_worker/models/llama.py:156-167).
 *
 * query [T, num_heads*head_dim], key / value [T, num_kv_heads*head_dim] (token strides in
 * bytes), positions int32 (positions_are_int64 = 0) or int64 [T], cos_sin_cache
 * [max_position, 2*head_dim] = the cos row then the sin row of a position (row stride in
 * bytes).  For every head, x = first half, y = second half:
 *   out_x = x*cos[i] - y*sin[i],  out_y = y*cos[D/2+i] + x*sin[D/2+i]
 * in the element type (dtype 0 = fp16, 1 = bf16).  `arithmetic` selects how the two lines are
 * rounded: LMS_ROPE_CONTRACTED = as the Triton compiler emits them for a GPU, the first product
 * of each line fused into the sum, out_x = fma(x, cos[i], -rn(y*sin[i])), out_y =
 * fma(y, cos[D/2+i], rn(x*sin[D/2+i])) — the results the reference produces when it runs;
 * LMS_ROPE_ROUND_EACH = every product and sum rounded on its own, the Triton language
 * semantics and the result of the Triton interpreter.  Rotated Q goes to q_out;
 * rotated K goes to k_out if it is not NULL and, if the caches are not NULL, to the key-cache
 * row of slot_mapping[t]; V is copied to the value-cache row.  Cache addressing, the slot < 0
 * padding rule and num_slots are those of lms_reshape_and_cache.  Only the full rotary
 * dimension (rotary_dim == head_dim, a multiple of 16) is supported, which covers the Llama
 * and Qwen2 models of the reference.  max_position: debug checks only (0 = unknown).
 */
#define LMS_ROPE_CONTRACTED 0
#define LMS_ROPE_ROUND_EACH 1
int lms_rope_and_cache(const void* query, const void* key, const void* value,
                       int64_t query_token_stride, int64_t key_token_stride,
                       int64_t value_token_stride, const void* positions,
                       int32_t positions_are_int64, const void* cos_sin_cache,
                       int64_t cos_sin_row_stride, void* q_out,
                       int64_t q_out_token_stride, void* k_out,
                       int64_t k_out_token_stride, void* key_cache,
                       void* value_cache, int64_t block_stride, int64_t slot_stride,
                       const int64_t* slot_mapping, int64_t num_tokens,
                       int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                       int32_t dtype, int32_t arithmetic, int32_t block_size,
                       int64_t num_slots, int64_t max_position, void* stream);

/*
 * Copy-on-write block copy — replaces
 *   copy_blocks               runtime/worker/llm_worker/ops/cache_ops.py:8-36
 *   copy_blocks_kernel        runtime/worker/llm_worker/ops/triton/cache_kernels.py:5-36
 * For every pair p and every layer l:
 *   kv[l*layer_stride + dst_p*block_stride ...] <- kv[l*layer_stride + src_p*block_stride ...]
 * (chunk_bytes bytes).  `pairs` is a device array of n_pairs (src, dst) int64
 * couples, 16-byte aligned.  Destinations must be distinct and no destination
 * may also be a source in the same call.  num_blocks: debug checks only.
 */
int lms_copy_blocks(void* kv, int64_t layer_stride, int64_t block_stride,
                    int64_t chunk_bytes, int32_t num_layers,
                    const int64_t* pairs, int64_t n_pairs,
                    int64_t num_blocks, void* stream);

/*
 * GPU <-> pinned-host block swap for layers [layer_begin, layer_end) — replaces
 *   KVWorker._save_layer_kv_blocks_to_host   runtime/worker/llm_worker/kv_worker.py:213-227
 *   KVWorker._load_layer_kv_blocks_from_host runtime/worker/llm_worker/kv_worker.py:197-211
 * (one cuMemcpy{DtoH,HtoD}Async per (layer, block) there; one kernel here).
 *   LMS_SWAP_OUT: host[dst_p][l] <- gpu[l][src_p]      LMS_SWAP_IN: gpu[l][dst_p] <- host[src_p][l]
 * gpu chunk address  = gpu  + l*gpu_layer_stride  + block*gpu_block_stride
 * host chunk address = host + block*host_block_stride + l*host_layer_stride
 * `host` must be the DEVICE-visible address of page-locked, mapped host memory
 * (lms_host_alloc / lms_host_register return it).  `pairs` (src, dst) int64
 * couples must be readable by the GPU (device memory or mapped host memory).
 * The layer range keeps the reference's layer-pipelined swap possible
 * (kv_worker.py:249-295 records / waits one event per layer).
 */
int lms_swap_blocks(int direction, void* gpu, int64_t gpu_layer_stride,
                    int64_t gpu_block_stride, void* host,
                    int64_t host_block_stride, int64_t host_layer_stride,
                    int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                    const int64_t* pairs, int64_t n_pairs,
                    int64_t num_gpu_blocks, int64_t num_host_blocks,
                    void* stream);

/*
 * Prefill -> decode block transfer — replaces the three hops of
 *   KVWorker.push_kv / _push_kv   runtime/worker/llm_worker/kv_worker.py:358-415
 * (GPU -> host write-through, NIXL/UCX host -> host WRITE, host -> GPU fetch)
 * with one kernel on the source GPU that reads local chunks and stores them
 * into the destination GPU's cache over NVLink:
 *   dst[l][dst_p] <- src[l][src_p]   for every pair p and layer l < num_layers.
 * `dst` is the peer cache as mapped into this process (peer access enabled on
 * a same-process pointer, or the result of lms_ipc_open).  Completion is
 * ordered by `stream` like any kernel; there is no device-side handshake.
 */
int lms_transfer_blocks(const void* src, int64_t src_layer_stride,
                        int64_t src_block_stride, void* dst,
                        int64_t dst_layer_stride, int64_t dst_block_stride,
                        int64_t chunk_bytes, int32_t num_layers,
                        const int64_t* pairs, int64_t n_pairs,
                        int64_t num_src_blocks, int64_t num_dst_blocks,
                        void* stream);

/*
 * The three chunk-copy operations with the (src, dst) table in HOST memory, which is where
 * LMServe's callers have it: copy_blocks flattens a Python dict and uploads it
 * (runtime/worker/llm_worker/ops/cache_ops.py:12-19) and the swap / push paths walk
 * protobuf BlockMapping entries on the host (runtime/worker/llm_worker/kv_worker.py:204-211,
 * 220-227,375-387).  The table is uploaded on `stream` into a per-device table buffer owned
 * by the library (cudaMalloc, grown on demand), then the same kernel runs.  These entry points
 * cannot be captured into a CUDA graph - a replay would upload from a host buffer the caller
 * has long reused - and return LMS_ERR_UNSUPPORTED when `stream` is capturing: upload the
 * table yourself and capture the device-table entry point.  Calls on different streams are ordered
 * against each other through an event so that the shared buffer is never overwritten while a
 * kernel still reads it.  `host_pairs` may be reused as soon as the call returns when it is
 * pageable memory; page-locked memory must stay valid until `stream` has passed the call.
 * All other arguments are those of the device-table entry points above.
 *
 * lms_swap_blocks_host can also run on the copy engines instead of the SMs
 * (LMS_TUNE_SWAP_ENGINE = 2): one cudaMemcpy2DAsync per block covering the layer range (one
 * copy per layer and block when the layer stride exceeds the 2D-copy pitch limit).  It is a
 * little slower on an idle GPU (2 MiB copies instead of one kernel) and needs one driver call
 * per block, but it leaves every SM to the kernels it overlaps with; with debug checks on, the
 * block ids are checked on the host and LMS_ERR_INDEX is returned before anything is copied.
 */
int lms_copy_blocks_host(void* kv, int64_t layer_stride, int64_t block_stride,
                         int64_t chunk_bytes, int32_t num_layers,
                         const int64_t* host_pairs, int64_t n_pairs,
                         int64_t num_blocks, void* stream);
int lms_swap_blocks_host(int direction, void* gpu, int64_t gpu_layer_stride,
                         int64_t gpu_block_stride, void* host,
                         int64_t host_block_stride, int64_t host_layer_stride,
                         int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                         const int64_t* host_pairs, int64_t n_pairs,
                         int64_t num_gpu_blocks, int64_t num_host_blocks,
                         void* stream);
/* The copy-engine form of lms_swap_blocks_host as an entry point of its own (what
 * LMS_TUNE_SWAP_ENGINE = 2 selects): no kernel is launched and no SM is used.  This is the
 * form to use when the swap overlaps the model's forward pass, as it does in LMServe
 * (runtime/worker/llm_worker/kv_worker.py:249-295): a resident copy kernel, however small,
 * keeps full-SM GEMM kernels from using the SMs it sits on.  Same arguments. */
int lms_swap_blocks_dma(int direction, void* gpu, int64_t gpu_layer_stride,
                        int64_t gpu_block_stride, void* host,
                        int64_t host_block_stride, int64_t host_layer_stride,
                        int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                        const int64_t* host_pairs, int64_t n_pairs,
                        int64_t num_gpu_blocks, int64_t num_host_blocks,
                        void* stream);
/* The swap through a contiguous device staging buffer (replaces the per-(layer, block)
 * cuMemcpy{HtoD,DtoH}Async loops of runtime/worker/llm_worker/kv_worker.py:206-211,222-227).
 * Swap-out: a gather kernel packs the scattered (layer, block) chunks of a group of blocks
 * into one half of `staging` ([block in group][layer][chunk], HBM to HBM), then the copy
 * engines move every host block - or every run of host blocks with adjacent ids, after the
 * pairs have been ordered by host block - in ONE transfer, on a copy stream owned by the
 * library; the two halves alternate so that the transfer of one group overlaps the gather of
 * the next.  Swap-in is the mirror image (large host-to-device transfers into a half, then a
 * scatter kernel).  The SMs are busy for about 2 % of the swap; the link carries the copy
 * engines' large packets instead of the 128-byte transactions SM-issued accesses become.
 * `staging`: device memory of the caller, 256-byte aligned, `staging_bytes` >= twice the bytes
 * of one block over the layer range (LMS_ERR_TOO_LARGE otherwise); two calls in the same
 * direction that may overlap need a staging buffer each.  `host` is the address of the
 * pinned pool; its layers of one block must be adjacent (host_layer_stride == chunk_bytes,
 * else LMS_ERR_UNSUPPORTED).  Block ids are always range-checked on the host (when the
 * bounds are > 0): the copy engines cannot skip a bad index, LMS_ERR_INDEX is returned
 * before anything moves.  Work is complete when `stream` has passed the call.  Not for use
 * inside stream capture.  Meant for whole-block swaps: with a one-layer range every
 * transfer is one chunk and the rate drops to what single 64 KiB copies reach. */
int lms_swap_blocks_staged(int direction, void* gpu, int64_t gpu_layer_stride,
                           int64_t gpu_block_stride, void* host,
                           int64_t host_block_stride, int64_t host_layer_stride,
                           int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                           const int64_t* host_pairs, int64_t n_pairs,
                           int64_t num_gpu_blocks, int64_t num_host_blocks,
                           void* staging, int64_t staging_bytes, void* stream);
int lms_transfer_blocks_host(const void* src, int64_t src_layer_stride,
                             int64_t src_block_stride, void* dst,
                             int64_t dst_layer_stride, int64_t dst_block_stride,
                             int64_t chunk_bytes, int32_t num_layers,
                             const int64_t* host_pairs, int64_t n_pairs,
                             int64_t num_src_blocks, int64_t num_dst_blocks,
                             void* stream);

/*
 * lms_copy_blocks_host for callers that must not allocate device memory.  (No counterpart in
 * the reference; it exists because of how LMServe is deployed.)  An LMServe worker hands
 * every byte the GPU has left to the KV cache when it starts (cache size = total * fraction -
 * peak, runtime/src/llm_engine/engine.rs:56-90), so a cudaMalloc made later, in the middle of
 * serving, can fail outright, and even when it succeeds it stalls every stream of the device
 * while the driver services it.  lms_copy_blocks_host makes such a call whenever its device
 * pair table has to be created or grown.  This variant never does: the uploaded (src, dst)
 * table lives in a fixed array that is part of the library image itself - 256 KiB of device
 * memory on every GPU that loads the library, held until the process exits - so it takes at
 * most LMS_STATIC_MAX_PAIRS pairs and returns LMS_ERR_TOO_LARGE beyond that.  It calls no
 * cudaMalloc / cudaFree, creates no event, and does not touch the per-device error record,
 * therefore the debug index checks are not available through it.
 *
 * The first call on a device looks the array's device address up (once per device, with that
 * device current); make that first call outside any stream capture.  All calls share the one
 * array, and the array keeps whatever the previous call uploaded: only the first n_pairs
 * entries are rewritten and only those are read, so stale entries are harmless, but two calls
 * whose work overlaps on the GPU (different streams without a dependency between them) race
 * on it - issue them on one stream or order them yourself.  `host_pairs` follows the rule of
 * lms_copy_blocks_host (pageable memory may be reused on return).
 */
#define LMS_STATIC_MAX_PAIRS 16384
int lms_copy_blocks_host_static(void* kv, int64_t layer_stride, int64_t block_stride,
                                int64_t chunk_bytes, int32_t num_layers,
                                const int64_t* host_pairs, int64_t n_pairs,
                                void* stream);

/* Enables peer access from the current device to `peer_device`
 * (LMS_ERR_PEER when the two GPUs cannot reach each other). */
int lms_peer_enable(int peer_device);

/*
 * Pinned host pool helpers — the role of pycuda.pagelocked_empty in
 *   runtime/worker/llm_worker/kv_worker.py:123-130.
 * lms_host_alloc returns page-locked, mapped, portable memory in *host_ptr and
 * its device-visible alias in *device_ptr; lms_host_register pins and maps an
 * existing allocation.  Free / unregister with the matching call.
 */
int lms_host_alloc(int64_t bytes, void** host_ptr, void** device_ptr);
int lms_host_free(void* host_ptr);
int lms_host_register(void* host_ptr, int64_t bytes, void** device_ptr);
int lms_host_unregister(void* host_ptr);

/*
 * Cross-process mapping of a peer's cache — the role of
 * UntypedStorage._share_cuda_ / _new_shared_cuda in
 *   runtime/worker/llm_worker/model_worker.py:284 and kv_worker.py:104-108.
 * lms_ipc_export fills a 64-byte handle for the allocation that contains
 * `device_ptr` and the byte offset of device_ptr inside it; lms_ipc_open maps
 * it in another process and returns base+offset; lms_ipc_close unmaps (pass the
 * pointer lms_ipc_open returned and the same offset).
 */
#define LMS_IPC_HANDLE_BYTES 64
int lms_ipc_export(void* device_ptr, void* handle64, int64_t* offset);
int lms_ipc_open(const void* handle64, int64_t offset, void** device_ptr);
int lms_ipc_close(void* device_ptr, int64_t offset);

/*
 * Asynchronous read of the device error record: enqueues, on `stream`, a copy of the 32-byte
 * record (the one lms_check_device_errors reads) into `host_dst32`, which must be page-locked
 * host memory that stays valid until `stream` has passed the call.  Nothing is synchronised
 * and the record is not cleared, so a pipelined caller can look at the record of step i while
 * step i + 1 is already running; word 0 of the copy is 0 when no kernel has reported anything.
 * No counterpart in the reference (its kernels do not check indices).
 */
int lms_error_record_async(void* host_dst32, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LMSERVE_KV_H_ */
