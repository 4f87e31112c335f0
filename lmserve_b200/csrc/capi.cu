// C ABI of the KV-cache data-movement library: argument validation, launch
// configuration, per-device state (SM count, error record) and the small
// host-memory / IPC helpers.  Declarations and the reference call sites each
// entry point replaces are in include/lmserve_kv.h.
#include <algorithm>
#include <atomic>
#include <mutex>
#include <new>
#include <vector>
#include <stdio.h>
#include <string.h>

#include "../../include/lmserve_kv.h"
#include "../../include/lmserve_kv_bench.h"
#include "kernels.cuh"

// A validated cache write (see lms_write_plan_create).
struct lms_write_plan {
  lms::WriteParams params;
  bool empty;
};

namespace {

using namespace lms;

constexpr int kMaxDevices = 64;

struct DeviceState {
  int sms = 0;
  // Device memory, allocated on first use.  Published with release order after `sms` is
  // set, read with acquire order, so a thread that sees the pointer sees the whole state.
  std::atomic<ErrRecord*> err{nullptr};
  // Device copy of the most recent host-side pair table (the *_host entry points).
  long long* table = nullptr;
  long long table_cap = 0;        // capacity in pairs
  cudaEvent_t table_free = nullptr;  // recorded after the kernel that last read `table`
  std::mutex table_mutex;
  // Staged swap (lms_swap_blocks_staged), one set per direction: the copy-engine stream the
  // large DMA transfers run on and the events that hand the two halves of the caller's
  // staging buffer back and forth between that stream and the caller's stream.
  struct Staged {
    cudaStream_t copy[2] = {nullptr, nullptr};  // transfers alternate between the two
    cudaEvent_t ready[2] = {nullptr, nullptr};  // half b holds data for the consumer
    cudaEvent_t freed[2] = {nullptr, nullptr};  // half b has been consumed
    cudaEvent_t start = nullptr;
    cudaEvent_t join = nullptr;                 // second copy stream has finished a group
    std::mutex mutex;
  } staged[2];
};

std::mutex g_mutex;
DeviceState g_dev[kMaxDevices];
std::atomic<int> g_checks{0};
std::atomic<long long> g_launches{0};
std::atomic<int> g_tuning[LMS_TUNE__COUNT];
thread_local char g_cuda_msg[256] = "";

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_msg, sizeof(g_cuda_msg), "%s: %s (%s)", what,
           cudaGetErrorName(e), cudaGetErrorString(e));
  // The runtime also remembers the error as the thread's "last error"; clear it so that the
  // cudaGetLastError() after a later, healthy kernel launch does not report this one again.
  cudaGetLastError();
  return LMS_ERR_CUDA;
}

#define LMS_CUDA(call)                                  \
  do {                                                  \
    cudaError_t e__ = (call);                           \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

// Per-device state of the current device; allocates the 32-byte error record
// the first time a device is seen.
int device_state(DeviceState** out) {
  int dev = 0;
  LMS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return LMS_ERR_RANGE;
  DeviceState& s = g_dev[dev];
  if (s.err.load(std::memory_order_acquire) == nullptr) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (s.err.load(std::memory_order_relaxed) == nullptr) {
      LMS_CUDA(cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev));
      ErrRecord* e = nullptr;
      LMS_CUDA(cudaMalloc(&e, sizeof(ErrRecord)));
      cudaError_t me = cudaMemset(e, 0, sizeof(ErrRecord));
      if (me != cudaSuccess) {
        cudaFree(e);
        return cuda_fail(me, "cudaMemset(error record)");
      }
      s.err.store(e, std::memory_order_release);
    }
  }
  *out = &s;
  return LMS_OK;
}

inline bool mult16(long long v) { return (v & 15) == 0; }
inline bool ptr16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

int tuned(int key, int fallback) {
  const int v = g_tuning[key].load(std::memory_order_relaxed);
  return v > 0 ? v : fallback;
}
int tuned_variant(int key, int fallback) {
  // variant numbers start at 0, so they are stored +1 and 0 means "not set"
  const int v = g_tuning[key].load(std::memory_order_relaxed);
  return v > 0 ? v - 1 : fallback;
}

// Page-table addressing of a write (all nullptr for direct slot addressing).
struct PagedIndex {
  const int32_t* batch_idx = nullptr;
  const int32_t* positions = nullptr;
  const int32_t* page_indices = nullptr;
  const int32_t* page_indptr = nullptr;
  int64_t num_requests = 0;  // entries of page_indptr minus one; 0 = not known
};

// Validates the arguments of a write and fills the kernel parameter block (everything but
// the per-launch fields: error record, checks flag).  LMS_OK with *empty = true means there
// is nothing to do.
int write_params(const void* key, const void* value, int64_t key_tok,
                 int64_t val_tok, int64_t key_layer, int64_t val_layer,
                 void* kcache, void* vcache, int64_t cache_layer,
                 int64_t block_stride, int64_t slot_stride,
                 const int64_t* slots, int64_t slot_layer, int64_t num_tokens,
                 int32_t num_layers, int64_t row_bytes, int32_t block_size,
                 int64_t num_slots, const PagedIndex* paged, WriteParams* out,
                 bool* empty) {
  *empty = false;
  if (num_tokens < 0 || num_layers < 0 || row_bytes <= 0 || block_size <= 0 ||
      num_tokens > 0x7fffffffll || row_bytes > (1 << 24) || slot_layer < 0 ||
      num_slots < 0)
    return LMS_ERR_RANGE;
  if (num_tokens == 0 || num_layers == 0) {
    *empty = true;
    return LMS_OK;
  }
  if (!key || !value || !kcache || !vcache) return LMS_ERR_NULL;
  if (paged == nullptr) {
    if (!slots) return LMS_ERR_NULL;
  } else {
    if (!paged->batch_idx || !paged->positions || !paged->page_indices || !paged->page_indptr)
      return LMS_ERR_NULL;
    if ((((uintptr_t)paged->batch_idx | (uintptr_t)paged->positions |
          (uintptr_t)paged->page_indices | (uintptr_t)paged->page_indptr) & 3u) != 0)
      return LMS_ERR_ALIGN;
  }
  if (!ptr16(key) || !ptr16(value) || !ptr16(kcache) || !ptr16(vcache) ||
      ((uintptr_t)slots & 7u) != 0 || !mult16(key_tok) || !mult16(val_tok) ||
      !mult16(key_layer) || !mult16(val_layer) || !mult16(cache_layer) ||
      !mult16(block_stride) || !mult16(slot_stride) || !mult16(row_bytes))
    return LMS_ERR_ALIGN;

  WriteParams p{};
  p.key = (const char*)key;
  p.value = (const char*)value;
  p.kcache = (char*)kcache;
  p.vcache = (char*)vcache;
  p.slots = paged ? nullptr : (const long long*)slots;
  if (paged) {
    p.batch_idx = paged->batch_idx;
    p.positions = paged->positions;
    p.page_indices = paged->page_indices;
    p.page_indptr = paged->page_indptr;
    if (paged->num_requests < 0 || paged->num_requests > 0x7fffffffll) return LMS_ERR_RANGE;
    p.num_requests = (int)paged->num_requests;
  }
  p.key_tok = key_tok;
  p.val_tok = val_tok;
  p.key_layer = key_layer;
  p.val_layer = val_layer;
  p.cache_layer = cache_layer;
  p.block_stride = block_stride;
  p.slot_stride = slot_stride;
  p.slot_layer = slot_layer;
  p.num_slots = num_slots;
  p.num_tokens = (int)num_tokens;
  p.num_layers = num_layers;
  p.block_size = block_size;
  p.row_bytes = (int)row_bytes;
  *out = p;
  return LMS_OK;
}

// Launches a validated write on the current device.
int write_launch(WriteParams p, void* stream) {
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  p.err = ds->err.load(std::memory_order_relaxed);
  p.checks = g_checks.load(std::memory_order_relaxed);
  const int variant = tuned_variant(LMS_TUNE_WRITE_VARIANT, -1);  // -1: launch_write chooses
  const int tile = tuned(LMS_TUNE_WRITE_TILE_BYTES, 0);
  const int vpt = tuned(LMS_TUNE_WRITE_VPT, 2);
  const bool pdl = tuned(LMS_TUNE_WRITE_PDL, 1) == 1;
  p.prefetch = tuned(LMS_TUNE_WRITE_PREFETCH, 1) == 1 ? 1 : 0;
  LMS_CUDA(launch_write(p, variant, tile, vpt, ds->sms, pdl, (cudaStream_t)stream));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return LMS_OK;
}

int write_layers(const void* key, const void* value, int64_t key_tok,
                 int64_t val_tok, int64_t key_layer, int64_t val_layer,
                 void* kcache, void* vcache, int64_t cache_layer,
                 int64_t block_stride, int64_t slot_stride,
                 const int64_t* slots, int64_t slot_layer, int64_t num_tokens,
                 int32_t num_layers, int64_t row_bytes, int32_t block_size,
                 int64_t num_slots, void* stream, const PagedIndex* paged = nullptr) {
  WriteParams p{};
  bool empty = false;
  if (int rc = write_params(key, value, key_tok, val_tok, key_layer, val_layer, kcache,
                            vcache, cache_layer, block_stride, slot_stride, slots,
                            slot_layer, num_tokens, num_layers, row_bytes, block_size,
                            num_slots, paged, &p, &empty))
    return rc;
  if (empty) return LMS_OK;
  return write_launch(p, stream);
}

// Shared validation + launch of the three chunk-copy entry points.
int chunk_copy(const void* src, int64_t src_layer, int64_t src_block, void* dst,
               int64_t dst_layer, int64_t dst_block, int64_t chunk_bytes,
               int32_t num_layers, const int64_t* pairs, int64_t n_pairs,
               int64_t num_src_blocks, int64_t num_dst_blocks, int layer_major,
               unsigned where, int variant, int policy, int ctas, void* stream) {
  if (n_pairs < 0 || num_layers < 0 || chunk_bytes <= 0 ||
      chunk_bytes > (1ll << 30) || num_src_blocks < 0 || num_dst_blocks < 0)
    return LMS_ERR_RANGE;
  if (n_pairs == 0 || num_layers == 0) return LMS_OK;
  if (!src || !dst || !pairs) return LMS_ERR_NULL;
  if (!ptr16(src) || !ptr16(dst) || !ptr16(pairs) || !mult16(src_layer) ||
      !mult16(src_block) || !mult16(dst_layer) || !mult16(dst_block) ||
      !mult16(chunk_bytes))
    return LMS_ERR_ALIGN;

  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;

  CopyParams p{};
  p.src = (const char*)src;
  p.dst = (char*)dst;
  p.src_layer = src_layer;
  p.src_block = src_block;
  p.dst_layer = dst_layer;
  p.dst_block = dst_block;
  p.pairs = (const long long*)pairs;
  p.n_pairs = n_pairs;
  p.num_src_blocks = num_src_blocks;
  p.num_dst_blocks = num_dst_blocks;
  p.num_layers = num_layers;
  p.layer_major = layer_major;
  p.chunk_bytes = (int)chunk_bytes;
  p.err = ds->err.load(std::memory_order_relaxed);
  p.where = where;
  p.checks = g_checks.load(std::memory_order_relaxed);
  p.pdl = tuned(LMS_TUNE_WRITE_PDL, 1) == 1 ? 1 : 0;

  if (ctas <= 0) ctas = ds->sms * 8;
  LMS_CUDA(launch_chunk_copy(p, variant, policy, ctas, (cudaStream_t)stream));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return LMS_OK;
}

// Uploads a host pair table into the device's table buffer on `stream` and returns the
// device pointer.  The caller launches its kernel on `stream` and then calls table_release.
int table_upload(DeviceState* ds, const int64_t* host_pairs, int64_t n_pairs,
                 cudaStream_t stream, const long long** out) {
  if (n_pairs > ds->table_cap) {
    if (ds->table != nullptr) {
      LMS_CUDA(cudaEventSynchronize(ds->table_free));
      LMS_CUDA(cudaFree(ds->table));
      ds->table = nullptr;
      ds->table_cap = 0;
    }
    long long cap = 4096;
    while (cap < n_pairs) cap *= 2;
    LMS_CUDA(cudaMalloc(&ds->table, (size_t)cap * 16));
    ds->table_cap = cap;
    if (ds->table_free == nullptr)
      LMS_CUDA(cudaEventCreateWithFlags(&ds->table_free, cudaEventDisableTiming));
  } else if (ds->table_free != nullptr) {
    LMS_CUDA(cudaStreamWaitEvent(stream, ds->table_free, 0));
  }
  LMS_CUDA(cudaMemcpyAsync(ds->table, host_pairs, (size_t)n_pairs * 16,
                           cudaMemcpyHostToDevice, stream));
  *out = ds->table;
  return LMS_OK;
}

int table_release(DeviceState* ds, cudaStream_t stream) {
  LMS_CUDA(cudaEventRecord(ds->table_free, stream));
  return LMS_OK;
}

// The entry points that upload a host-side table cannot be captured into a CUDA graph: the
// upload would be replayed from a host buffer the caller has long reused, and the shared
// table is guarded by an event recorded outside the capture.  They say so instead of failing
// somewhere inside the runtime.
int refuse_capture(cudaStream_t stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
    cudaGetLastError();
    return LMS_OK;  // let the real call report whatever is wrong with the stream
  }
  if (st == cudaStreamCaptureStatusNone) return LMS_OK;
  snprintf(g_cuda_msg, sizeof(g_cuda_msg),
           "a host-side pair table cannot be used while the stream is being captured; upload "
           "the table yourself and call the device-table entry point");
  return LMS_ERR_UNSUPPORTED;
}

// Runs `launch(device_pairs)` with the host table uploaded first.
template <class F>
int with_host_table(const int64_t* host_pairs, int64_t n_pairs, void* stream, F launch) {
  if (n_pairs < 0) return LMS_ERR_RANGE;
  if (n_pairs == 0) return launch((const int64_t*)nullptr);
  if (!host_pairs) return LMS_ERR_NULL;
  if (int rc = refuse_capture((cudaStream_t)stream)) return rc;
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  std::lock_guard<std::mutex> lock(ds->table_mutex);
  const long long* dev_pairs = nullptr;
  if (int rc = table_upload(ds, host_pairs, n_pairs, (cudaStream_t)stream, &dev_pairs)) return rc;
  const int rc = launch((const int64_t*)dev_pairs);
  const int rc2 = table_release(ds, (cudaStream_t)stream);
  return rc != LMS_OK ? rc : rc2;
}

// ---- fixed pair table of lms_copy_blocks_host_static -------------------------------------
// Part of the library image: every device that loads the library holds these 256 KiB until
// the process exits.  In host code the name below is only a handle for the runtime, not a
// device address; static_table() asks the runtime for the address, per device.
static __device__ __align__(256) long long g_static_pairs[2 * LMS_STATIC_MAX_PAIRS];

struct StaticTable {
  long long* table = nullptr;  // device address of g_static_pairs on this device
  int sms = 0;
};
StaticTable g_static[kMaxDevices];
std::mutex g_static_mutex;

// Once per device, with that device current.  No allocation.
int static_table(StaticTable** out) {
  int dev = 0;
  LMS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return LMS_ERR_RANGE;
  StaticTable& t = g_static[dev];
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (t.table == nullptr) {
    void* ptr = nullptr;
    LMS_CUDA(cudaGetSymbolAddress(&ptr, g_static_pairs));
    int sms = 0;
    LMS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    t.sms = sms;
    t.table = static_cast<long long*>(ptr);
  }
  *out = &t;
  return LMS_OK;
}

int sm_count() {
  DeviceState* ds = nullptr;
  if (device_state(&ds) != LMS_OK) return 148;
  return ds->sms;
}

}  // namespace

extern "C" {
#pragma GCC visibility push(default)

int lms_version(void) { return LMS_VERSION; }

const char* lms_strerror(int status) {
  switch (status) {
    case LMS_OK: return "ok";
    case LMS_ERR_NULL: return "a required pointer is NULL";
    case LMS_ERR_ALIGN: return "pointer, stride or size is not a multiple of 16 bytes";
    case LMS_ERR_RANGE: return "argument out of range";
    case LMS_ERR_CUDA: return "a CUDA call failed (see lms_last_cuda_error)";
    case LMS_ERR_INDEX: return "a kernel met an out-of-range slot or block index";
    case LMS_ERR_PEER: return "peer access between the devices is unavailable";
    case LMS_ERR_UNSUPPORTED: return "unsupported";
    case LMS_ERR_TOO_LARGE: return "more block pairs than the fixed-size table holds";
    default: return "unknown status";
  }
}

const char* lms_last_cuda_error(void) { return g_cuda_msg; }

int lms_init_device(void) {
  DeviceState* ds = nullptr;
  return device_state(&ds);
}

int lms_set_tuning(int key, int value) {
  if (key <= 0 || key >= LMS_TUNE__COUNT) return LMS_ERR_RANGE;
  const bool is_variant = key == LMS_TUNE_WRITE_VARIANT || key == LMS_TUNE_COPY_VARIANT ||
                          key == LMS_TUNE_XFER_VARIANT || key == LMS_TUNE_SWAP_VARIANT;
  if (is_variant) {
    if (value > (key == LMS_TUNE_WRITE_VARIANT ? 7 : 4)) return LMS_ERR_RANGE;
    g_tuning[key].store(value < 0 ? 0 : value + 1);
  } else {
    g_tuning[key].store(value < 0 ? 0 : value);
  }
  return LMS_OK;
}

int lms_get_tuning(int key) {
  if (key <= 0 || key >= LMS_TUNE__COUNT) return LMS_ERR_RANGE;
  const bool is_variant = key == LMS_TUNE_WRITE_VARIANT || key == LMS_TUNE_COPY_VARIANT ||
                          key == LMS_TUNE_XFER_VARIANT || key == LMS_TUNE_SWAP_VARIANT;
  const int v = g_tuning[key].load();
  return is_variant ? v - 1 : v;
}

int lms_set_debug_checks(int enable) {
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  g_checks.store(enable ? 1 : 0);
  return LMS_OK;
}

int lms_check_device_errors(void* stream, int64_t* index, int64_t* value) {
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  ErrRecord h{};
  LMS_CUDA(cudaMemcpyAsync(&h, ds->err.load(std::memory_order_relaxed), sizeof(h), cudaMemcpyDeviceToHost,
                           (cudaStream_t)stream));
  LMS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (h.code == kErrNone) return LMS_OK;
  LMS_CUDA(cudaMemsetAsync(ds->err.load(std::memory_order_relaxed), 0, sizeof(h), (cudaStream_t)stream));
  LMS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (index) *index = h.index;
  if (value) *value = h.value;
  if (h.code == kErrBadPosition && h.where == kWhereStepIndices) {
    snprintf(g_cuda_msg, sizeof(g_cuda_msg),
             "token %lld: position %lld has no page in its request's block table", h.index, h.value);
    return LMS_ERR_INDEX;
  }
  if (h.code == kErrBadPosition) {
    snprintf(g_cuda_msg, sizeof(g_cuda_msg), "position %lld of token %lld is outside the cos/sin cache",
             h.value, h.index);
    return LMS_ERR_INDEX;
  }
  if (h.code == kErrWaitTimeout) {
    snprintf(g_cuda_msg, sizeof(g_cuda_msg),
             "kernel %u gave up waiting for a bulk copy (task %lld)", h.where,
             h.index);
    return LMS_ERR_CUDA;
  }
  return LMS_ERR_INDEX;
}

int lms_error_record_async(void* host_dst32, void* stream) {
  if (!host_dst32) return LMS_ERR_NULL;
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  static_assert(sizeof(ErrRecord) == 32, "the error record is 32 bytes");
  LMS_CUDA(cudaMemcpyAsync(host_dst32, ds->err.load(std::memory_order_relaxed), sizeof(ErrRecord),
                           cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return LMS_OK;
}

const char* lms_write_kernel_name(int64_t row_bytes, int64_t total_bytes) {
  return write_kernel_name(tuned_variant(LMS_TUNE_WRITE_VARIANT, -1), row_bytes, total_bytes);
}

int lms_reshape_and_cache(const void* key, const void* value,
                          int64_t key_token_stride, int64_t value_token_stride,
                          void* key_cache, void* value_cache,
                          int64_t block_stride, int64_t slot_stride,
                          const int64_t* slot_mapping, int64_t num_tokens,
                          int64_t row_bytes, int32_t block_size,
                          int64_t num_slots, void* stream) {
  return write_layers(key, value, key_token_stride, value_token_stride, 0, 0,
                      key_cache, value_cache, 0, block_stride, slot_stride,
                      slot_mapping, 0, num_tokens, 1, row_bytes, block_size,
                      num_slots, stream);
}

int lms_reshape_and_cache_layers(const void* key, const void* value,
                                 int64_t key_token_stride, int64_t value_token_stride,
                                 int64_t key_layer_stride, int64_t value_layer_stride,
                                 void* key_cache, void* value_cache,
                                 int64_t cache_layer_stride,
                                 int64_t block_stride, int64_t slot_stride,
                                 const int64_t* slot_mapping, int64_t slot_layer_stride,
                                 int64_t num_tokens, int32_t num_layers,
                                 int64_t row_bytes, int32_t block_size,
                                 int64_t num_slots, void* stream) {
  return write_layers(key, value, key_token_stride, value_token_stride,
                      key_layer_stride, value_layer_stride, key_cache,
                      value_cache, cache_layer_stride, block_stride,
                      slot_stride, slot_mapping, slot_layer_stride, num_tokens,
                      num_layers, row_bytes, block_size, num_slots, stream);
}

int lms_write_plan_create(const void* key, const void* value,
                          int64_t key_token_stride, int64_t value_token_stride,
                          int64_t key_layer_stride, int64_t value_layer_stride,
                          void* key_cache, void* value_cache,
                          int64_t cache_layer_stride,
                          int64_t block_stride, int64_t slot_stride,
                          const int64_t* slot_mapping, int64_t slot_layer_stride,
                          int64_t num_tokens, int32_t num_layers,
                          int64_t row_bytes, int32_t block_size,
                          int64_t num_slots, lms_write_plan** plan) {
  if (!plan) return LMS_ERR_NULL;
  *plan = nullptr;
  WriteParams p{};
  bool empty = false;
  if (int rc = write_params(key, value, key_token_stride, value_token_stride,
                            key_layer_stride, value_layer_stride, key_cache, value_cache,
                            cache_layer_stride, block_stride, slot_stride, slot_mapping,
                            slot_layer_stride, num_tokens, num_layers, row_bytes,
                            block_size, num_slots, nullptr, &p, &empty))
    return rc;
  // Per-device set-up now, so that the first run may already sit inside a graph capture.
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  lms_write_plan* out = new (std::nothrow) lms_write_plan;
  if (!out) return LMS_ERR_UNSUPPORTED;
  out->params = p;
  out->empty = empty;
  *plan = out;
  return LMS_OK;
}

int lms_write_plan_run(const lms_write_plan* plan, void* stream) {
  if (!plan) return LMS_ERR_NULL;
  if (plan->empty) return LMS_OK;
  return write_launch(plan->params, stream);
}

int lms_write_plan_destroy(lms_write_plan* plan) {
  delete plan;
  return LMS_OK;
}

int lms_append_paged_kv_cache(const void* key, const void* value,
                              int64_t key_token_stride, int64_t value_token_stride,
                              int64_t key_layer_stride, int64_t value_layer_stride,
                              const int32_t* batch_indices, const int32_t* positions,
                              void* key_cache, void* value_cache,
                              int64_t cache_layer_stride, int64_t block_stride,
                              int64_t slot_stride, const int32_t* kv_indices,
                              const int32_t* kv_indptr, int64_t num_tokens,
                              int32_t num_layers, int64_t row_bytes,
                              int32_t block_size, int64_t num_blocks, void* stream) {
  if (num_blocks < 0 || num_blocks > (1ll << 40)) return LMS_ERR_RANGE;
  PagedIndex paged;
  paged.batch_idx = batch_indices;
  paged.positions = positions;
  paged.page_indices = kv_indices;
  paged.page_indptr = kv_indptr;
  return write_layers(key, value, key_token_stride, value_token_stride,
                      key_layer_stride, value_layer_stride, key_cache, value_cache,
                      cache_layer_stride, block_stride, slot_stride, nullptr, 0,
                      num_tokens, num_layers, row_bytes, block_size,
                      num_blocks * (int64_t)block_size, stream, &paged);
}

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
                                lms_write_plan** plan) {
  if (!plan) return LMS_ERR_NULL;
  *plan = nullptr;
  if (num_blocks < 0 || num_blocks > (1ll << 40)) return LMS_ERR_RANGE;
  PagedIndex paged;
  paged.batch_idx = batch_indices;
  paged.positions = positions;
  paged.page_indices = kv_indices;
  paged.page_indptr = kv_indptr;
  paged.num_requests = num_requests;
  WriteParams p{};
  bool empty = false;
  if (int rc = write_params(key, value, key_token_stride, value_token_stride,
                            key_layer_stride, value_layer_stride, key_cache, value_cache,
                            cache_layer_stride, block_stride, slot_stride, nullptr, 0,
                            num_tokens, num_layers, row_bytes, block_size,
                            num_blocks * (int64_t)block_size, &paged, &p, &empty))
    return rc;
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  lms_write_plan* out = new (std::nothrow) lms_write_plan;
  if (!out) return LMS_ERR_UNSUPPORTED;
  out->params = p;
  out->empty = empty;
  *plan = out;
  return LMS_OK;
}

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
                       int64_t num_slots, int64_t max_position, void* stream) {
  if (num_tokens < 0 || num_tokens > 0x7fffffffll || num_heads <= 0 || num_kv_heads <= 0 ||
      head_dim <= 0 || num_slots < 0 || max_position < 0 || (dtype != 0 && dtype != 1) ||
      (arithmetic != LMS_ROPE_CONTRACTED && arithmetic != LMS_ROPE_ROUND_EACH))
    return LMS_ERR_RANGE;
  if (head_dim % 16 != 0) return LMS_ERR_UNSUPPORTED;
  if (num_tokens == 0) return LMS_OK;
  const bool cached = key_cache != nullptr || value_cache != nullptr;
  if (!query || !key || !positions || !cos_sin_cache || !q_out) return LMS_ERR_NULL;
  if (cached && (!key_cache || !value_cache || !value || !slot_mapping)) return LMS_ERR_NULL;
  if (cached && block_size <= 0) return LMS_ERR_RANGE;
  if (!ptr16(query) || !ptr16(key) || !ptr16(cos_sin_cache) || !ptr16(q_out) || !ptr16(k_out) ||
      !mult16(query_token_stride) || !mult16(key_token_stride) ||
      !mult16(cos_sin_row_stride) || !mult16(q_out_token_stride) ||
      !mult16(k_out_token_stride) ||
      ((uintptr_t)positions & (positions_are_int64 ? 7u : 3u)) != 0)
    return LMS_ERR_ALIGN;
  if (cached && (!ptr16(value) || !ptr16(key_cache) || !ptr16(value_cache) ||
                 !mult16(value_token_stride) || !mult16(block_stride) ||
                 !mult16(slot_stride) || ((uintptr_t)slot_mapping & 7u) != 0))
    return LMS_ERR_ALIGN;

  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  RopeParams p{};
  p.q = (const char*)query;
  p.k = (const char*)key;
  p.v = (const char*)value;
  p.q_tok = query_token_stride;
  p.k_tok = key_token_stride;
  p.v_tok = value_token_stride;
  p.positions = positions;
  p.pos64 = positions_are_int64 ? 1 : 0;
  p.cos_sin = (const char*)cos_sin_cache;
  p.cs_row = cos_sin_row_stride;
  p.q_out = (char*)q_out;
  p.qo_tok = q_out_token_stride;
  p.k_out = (char*)k_out;
  p.ko_tok = k_out_token_stride;
  p.kcache = cached ? (char*)key_cache : nullptr;
  p.vcache = cached ? (char*)value_cache : nullptr;
  p.block_stride = block_stride;
  p.slot_stride = slot_stride;
  p.slots = (const long long*)slot_mapping;
  p.num_slots = num_slots;
  p.max_pos = max_position;
  p.num_tokens = (int)num_tokens;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.head_dim = head_dim;
  p.block_size = cached ? block_size : 1;
  p.is_bf16 = dtype;
  p.fused = arithmetic == LMS_ROPE_CONTRACTED ? 1 : 0;
  p.prefetch = tuned(LMS_TUNE_WRITE_PREFETCH, 1) == 1 ? 1 : 0;
  p.err = ds->err.load(std::memory_order_relaxed);
  p.checks = g_checks.load(std::memory_order_relaxed);
  LMS_CUDA(launch_rope_cache(p, tuned(LMS_TUNE_WRITE_PDL, 1) == 1, (cudaStream_t)stream));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return LMS_OK;
}

int lms_build_step_indices(const int32_t* input_len, const int32_t* filled_len,
                           const int32_t* context_len, const int32_t* num_blocks,
                           const int32_t* block_ids, const int32_t* token_ids,
                           int32_t batch, int64_t total_tokens, int64_t total_blocks,
                           int32_t block_size, int32_t* position_ids,
                           int32_t* cu_seqlens_q, int32_t* kv_block_indptrs,
                           int32_t* kv_block_indices, int32_t* kv_last_block_lens,
                           int32_t* batch_indices, int32_t* positions,
                           int64_t* slot_mapping, int64_t* input_ids, int32_t num_prefill,
                           int32_t num_decode, int32_t* decode_kv_block_indptrs, void* stream) {
  if (num_prefill < 0 || num_decode < 0 || (int64_t)num_prefill + num_decode > batch)
    return LMS_ERR_RANGE;
  if (batch < 0 || total_tokens < 0 || total_blocks < 0 || block_size <= 0 ||
      total_tokens > 0x7fffffffll || total_blocks > 0x7fffffffll)
    return LMS_ERR_RANGE;
  if (batch > LMS_STEP_MAX_BATCH) return LMS_ERR_TOO_LARGE;
  // An empty step still defines cu_seqlens_q[0] = kv_block_indptrs[0] = 0.
  if (batch == 0 && total_tokens == 0 && total_blocks == 0 && !cu_seqlens_q && !kv_block_indptrs &&
      !decode_kv_block_indptrs)
    return LMS_OK;
  if (batch > 0 && (!input_len || !filled_len || !context_len || !num_blocks)) return LMS_ERR_NULL;
  if (total_blocks > 0 && !block_ids) return LMS_ERR_NULL;
  if (input_ids && total_tokens > 0 && !token_ids) return LMS_ERR_NULL;
  const void* four[] = {input_len, filled_len, context_len, num_blocks, block_ids, token_ids,
                        position_ids, cu_seqlens_q, kv_block_indptrs, kv_block_indices,
                        kv_last_block_lens, batch_indices, positions, decode_kv_block_indptrs};
  for (const void* q : four)
    if (((uintptr_t)q & 3u) != 0) return LMS_ERR_ALIGN;
  if (((uintptr_t)slot_mapping & 7u) != 0 || ((uintptr_t)input_ids & 7u) != 0) return LMS_ERR_ALIGN;

  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  StepIndexParams p{};
  p.input_len = input_len;
  p.filled_len = filled_len;
  p.context_len = context_len;
  p.num_blocks = num_blocks;
  p.block_ids = block_ids;
  p.token_ids = token_ids;
  p.batch = batch;
  p.block_size = block_size;
  p.total_tokens = total_tokens;
  p.total_blocks = total_blocks;
  p.position_ids = position_ids;
  p.cu_seqlens_q = cu_seqlens_q;
  p.kv_block_indptrs = kv_block_indptrs;
  p.kv_block_indices = kv_block_indices;
  p.kv_last_block_lens = kv_last_block_lens;
  p.batch_indices = batch_indices;
  p.positions = positions;
  p.slot_mapping = (long long*)slot_mapping;
  p.input_ids = (long long*)input_ids;
  p.decode_kv_block_indptrs = decode_kv_block_indptrs;
  p.num_prefill = num_prefill;
  p.num_decode = num_decode;
  p.err = ds->err.load(std::memory_order_relaxed);
  p.checks = g_checks.load(std::memory_order_relaxed);
  LMS_CUDA(launch_step_indices(p, ds->sms, (cudaStream_t)stream));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return LMS_OK;
}

int lms_copy_blocks(void* kv, int64_t layer_stride, int64_t block_stride,
                    int64_t chunk_bytes, int32_t num_layers,
                    const int64_t* pairs, int64_t n_pairs, int64_t num_blocks,
                    void* stream) {
  // Layer-major unit order: CTAs running at the same time work on one layer,
  // so a source block that fans out to many destinations is re-read from L2.
  const int per_sm = tuned(LMS_TUNE_COPY_CTAS_PER_SM, 2);
  return chunk_copy(kv, layer_stride, block_stride, kv, layer_stride,
                    block_stride, chunk_bytes, num_layers, pairs, n_pairs,
                    num_blocks, num_blocks, /*layer_major=*/1, kWhereCopyBlocks,
                    tuned_variant(LMS_TUNE_COPY_VARIANT, 3), /*policy=*/1,
                    sm_count() * per_sm, stream);
}

int lms_swap_blocks(int direction, void* gpu, int64_t gpu_layer_stride,
                    int64_t gpu_block_stride, void* host,
                    int64_t host_block_stride, int64_t host_layer_stride,
                    int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                    const int64_t* pairs, int64_t n_pairs,
                    int64_t num_gpu_blocks, int64_t num_host_blocks,
                    void* stream) {
  if (direction != LMS_SWAP_OUT && direction != LMS_SWAP_IN) return LMS_ERR_RANGE;
  if (layer_begin < 0 || layer_end < layer_begin) return LMS_ERR_RANGE;
  if (!gpu || !host) return (n_pairs == 0 || layer_end == layer_begin) ? LMS_OK : LMS_ERR_NULL;
  const int nl = layer_end - layer_begin;
  char* g = (char*)gpu + (long long)layer_begin * gpu_layer_stride;
  char* h = (char*)host + (long long)layer_begin * host_layer_stride;
  // Pair-major unit order: consecutive units are the layers of one block,
  // which are adjacent in the block-major host pool.  Three CTAs of 1024 threads (64 KiB in
  // flight each): the link, not the GPU, is the limit (2 such CTAs already fill PCIe
  // outbound, 3 inbound; with 256-thread CTAs inbound needs 6), and a resident copy CTA takes
  // its SM away from the full-SM GEMM kernels of the forward pass the swap overlaps with:
  // measured against a stream of 8192^3 bf16 GEMMs, up to 3 copy CTAs cost them nothing,
  // 4 cost 20 %, 5 or more 85 % and upwards.
  constexpr int kSwapCtas = 3;
  if (direction == LMS_SWAP_OUT)
    return chunk_copy(g, gpu_layer_stride, gpu_block_stride, h,
                      host_layer_stride, host_block_stride, chunk_bytes, nl,
                      pairs, n_pairs, num_gpu_blocks, num_host_blocks,
                      /*layer_major=*/0, kWhereSwapOut,
                      tuned_variant(LMS_TUNE_SWAP_VARIANT, 4), 0,
                      tuned(LMS_TUNE_SWAP_OUT_CTAS, kSwapCtas), stream);
  return chunk_copy(h, host_layer_stride, host_block_stride, g,
                    gpu_layer_stride, gpu_block_stride, chunk_bytes, nl, pairs,
                    n_pairs, num_host_blocks, num_gpu_blocks,
                    /*layer_major=*/0, kWhereSwapIn,
                    tuned_variant(LMS_TUNE_SWAP_VARIANT, 4), 0,
                    tuned(LMS_TUNE_SWAP_IN_CTAS, kSwapCtas), stream);
}

int lms_transfer_blocks(const void* src, int64_t src_layer_stride,
                        int64_t src_block_stride, void* dst,
                        int64_t dst_layer_stride, int64_t dst_block_stride,
                        int64_t chunk_bytes, int32_t num_layers,
                        const int64_t* pairs, int64_t n_pairs,
                        int64_t num_src_blocks, int64_t num_dst_blocks,
                        void* stream) {
  const int per_sm = tuned(LMS_TUNE_XFER_CTAS_PER_SM, 4);
  return chunk_copy(src, src_layer_stride, src_block_stride, dst,
                    dst_layer_stride, dst_block_stride, chunk_bytes, num_layers,
                    pairs, n_pairs, num_src_blocks, num_dst_blocks,
                    /*layer_major=*/1, kWhereTransfer,
                    tuned_variant(LMS_TUNE_XFER_VARIANT, 3), 0,
                    sm_count() * per_sm, stream);
}

int lms_copy_blocks_host(void* kv, int64_t layer_stride, int64_t block_stride,
                         int64_t chunk_bytes, int32_t num_layers,
                         const int64_t* host_pairs, int64_t n_pairs,
                         int64_t num_blocks, void* stream) {
  return with_host_table(host_pairs, n_pairs, stream, [&](const int64_t* pairs) {
    return lms_copy_blocks(kv, layer_stride, block_stride, chunk_bytes, num_layers,
                           pairs, n_pairs, num_blocks, stream);
  });
}

int lms_copy_blocks_host_static(void* kv, int64_t layer_stride, int64_t block_stride,
                                int64_t chunk_bytes, int32_t num_layers,
                                const int64_t* host_pairs, int64_t n_pairs,
                                void* stream) {
  if (n_pairs < 0 || num_layers < 0 || chunk_bytes <= 0 || chunk_bytes > (1ll << 30))
    return LMS_ERR_RANGE;
  if (n_pairs > LMS_STATIC_MAX_PAIRS) return LMS_ERR_TOO_LARGE;
  if (n_pairs == 0 || num_layers == 0) return LMS_OK;
  if (!kv || !host_pairs) return LMS_ERR_NULL;
  if (!ptr16(kv) || !mult16(layer_stride) || !mult16(block_stride) || !mult16(chunk_bytes))
    return LMS_ERR_ALIGN;

  StaticTable* st = nullptr;
  if (int rc = static_table(&st)) return rc;
  // Upload into the fixed table, then the same kernel as lms_copy_blocks on the same stream.
  LMS_CUDA(cudaMemcpyAsync(st->table, host_pairs, (size_t)n_pairs * 16,
                           cudaMemcpyHostToDevice, (cudaStream_t)stream));
  CopyParams p{};
  p.src = (const char*)kv;
  p.dst = (char*)kv;
  p.src_layer = p.dst_layer = layer_stride;
  p.src_block = p.dst_block = block_stride;
  p.pairs = st->table;
  p.n_pairs = n_pairs;
  p.num_layers = num_layers;
  p.layer_major = 1;
  p.chunk_bytes = (int)chunk_bytes;
  p.err = nullptr;  // no error record on this path
  p.where = kWhereCopyBlocks;
  p.checks = 0;
  const int per_sm = tuned(LMS_TUNE_COPY_CTAS_PER_SM, 2);
  LMS_CUDA(launch_chunk_copy(p, tuned_variant(LMS_TUNE_COPY_VARIANT, 3), /*policy=*/1,
                             st->sms * per_sm, (cudaStream_t)stream));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return LMS_OK;
}

#pragma GCC visibility pop
}  // extern "C"

namespace {

// Swap on the copy engines: one strided DMA per block over the layer range.
int swap_blocks_dma(int direction, char* gpu, int64_t gpu_layer_stride,
                    int64_t gpu_block_stride, char* host, int64_t host_block_stride,
                    int64_t host_layer_stride, int64_t chunk_bytes, int32_t layer_begin,
                    int32_t layer_end, const int64_t* pairs, int64_t n_pairs,
                    int64_t num_gpu_blocks, int64_t num_host_blocks, cudaStream_t stream) {
  if (direction != LMS_SWAP_OUT && direction != LMS_SWAP_IN) return LMS_ERR_RANGE;
  if (layer_begin < 0 || layer_end < layer_begin || n_pairs < 0 || chunk_bytes <= 0)
    return LMS_ERR_RANGE;
  const int nl = layer_end - layer_begin;
  if (n_pairs == 0 || nl == 0) return LMS_OK;
  if (!gpu || !host || !pairs) return LMS_ERR_NULL;
  if (!mult16(gpu_layer_stride) || !mult16(gpu_block_stride) || !mult16(host_block_stride) ||
      !mult16(host_layer_stride) || !mult16(chunk_bytes) || !ptr16(gpu) || !ptr16(host))
    return LMS_ERR_ALIGN;
  const bool out = direction == LMS_SWAP_OUT;
  if (g_checks.load(std::memory_order_relaxed)) {
    for (int64_t i = 0; i < n_pairs; ++i) {
      const int64_t g = out ? pairs[2 * i] : pairs[2 * i + 1];
      const int64_t h = out ? pairs[2 * i + 1] : pairs[2 * i];
      if (g < 0 || h < 0 || (num_gpu_blocks > 0 && g >= num_gpu_blocks) ||
          (num_host_blocks > 0 && h >= num_host_blocks)) {
        snprintf(g_cuda_msg, sizeof(g_cuda_msg), "block pair %lld (%lld, %lld) is out of range",
                 (long long)i, (long long)pairs[2 * i], (long long)pairs[2 * i + 1]);
        return LMS_ERR_INDEX;
      }
    }
  }
  int dev = 0, max_pitch = 0;
  LMS_CUDA(cudaGetDevice(&dev));
  LMS_CUDA(cudaDeviceGetAttribute(&max_pitch, cudaDevAttrMaxPitch, dev));
  const bool strided = gpu_layer_stride <= max_pitch && host_layer_stride <= max_pitch;
  const cudaMemcpyKind kind = out ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice;
  for (int64_t i = 0; i < n_pairs; ++i) {
    const int64_t gb = out ? pairs[2 * i] : pairs[2 * i + 1];
    const int64_t hb = out ? pairs[2 * i + 1] : pairs[2 * i];
    char* g = gpu + (long long)layer_begin * gpu_layer_stride + gb * gpu_block_stride;
    char* h = host + hb * host_block_stride + (long long)layer_begin * host_layer_stride;
    if (strided) {
      if (out)
        LMS_CUDA(cudaMemcpy2DAsync(h, (size_t)host_layer_stride, g, (size_t)gpu_layer_stride,
                                   (size_t)chunk_bytes, (size_t)nl, kind, stream));
      else
        LMS_CUDA(cudaMemcpy2DAsync(g, (size_t)gpu_layer_stride, h, (size_t)host_layer_stride,
                                   (size_t)chunk_bytes, (size_t)nl, kind, stream));
    } else {
      for (int l = 0; l < nl; ++l) {
        char* gl = g + (long long)l * gpu_layer_stride;
        char* hl = h + (long long)l * host_layer_stride;
        LMS_CUDA(cudaMemcpyAsync(out ? hl : gl, out ? gl : hl, (size_t)chunk_bytes, kind, stream));
      }
    }
  }
  return LMS_OK;
}

// Swap through a contiguous device staging ring: the SMs only move HBM -> HBM (gather the
// scattered chunks of a group of blocks into one half of the staging buffer, or scatter them
// out of it) and the PCIe hop is done by the copy engines in transfers of whole host blocks -
// or of runs of adjacent host blocks - which use the link's large packets.  The two halves
// alternate, so the DMA of one group overlaps the gather / scatter of the next.
int staged_setup(DeviceState::Staged& st) {
  if (st.join != nullptr) return LMS_OK;
  for (int b = 0; b < 2; ++b) {
    LMS_CUDA(cudaStreamCreateWithFlags(&st.copy[b], cudaStreamNonBlocking));
    LMS_CUDA(cudaEventCreateWithFlags(&st.ready[b], cudaEventDisableTiming));
    LMS_CUDA(cudaEventCreateWithFlags(&st.freed[b], cudaEventDisableTiming));
  }
  LMS_CUDA(cudaEventCreateWithFlags(&st.start, cudaEventDisableTiming));
  LMS_CUDA(cudaEventCreateWithFlags(&st.join, cudaEventDisableTiming));
  return LMS_OK;
}

int swap_blocks_staged(int direction, char* gpu, int64_t gpu_layer_stride,
                       int64_t gpu_block_stride, char* host, int64_t host_block_stride,
                       int64_t host_layer_stride, int64_t chunk_bytes, int32_t layer_begin,
                       int32_t layer_end, const int64_t* pairs, int64_t n_pairs,
                       int64_t num_gpu_blocks, int64_t num_host_blocks, char* staging,
                       int64_t staging_bytes, cudaStream_t stream) {
  if (direction != LMS_SWAP_OUT && direction != LMS_SWAP_IN) return LMS_ERR_RANGE;
  if (layer_begin < 0 || layer_end < layer_begin || n_pairs < 0 || chunk_bytes <= 0 ||
      chunk_bytes > (1ll << 30) || staging_bytes < 0)
    return LMS_ERR_RANGE;
  const int nl = layer_end - layer_begin;
  if (n_pairs == 0 || nl == 0) return LMS_OK;
  if (!gpu || !host || !pairs || !staging) return LMS_ERR_NULL;
  if (!mult16(gpu_layer_stride) || !mult16(gpu_block_stride) || !mult16(host_block_stride) ||
      !mult16(host_layer_stride) || !mult16(chunk_bytes) || !ptr16(gpu) || !ptr16(host) ||
      ((uintptr_t)staging & 255u) != 0)
    return LMS_ERR_ALIGN;
  // The layers of one host block must be adjacent, or a block is not one DMA transfer.
  if (host_layer_stride != chunk_bytes) return LMS_ERR_UNSUPPORTED;
  const bool out = direction == LMS_SWAP_OUT;
  const int64_t per_block = (int64_t)nl * chunk_bytes;
  const int64_t half = (staging_bytes / 2) & ~(int64_t)255;
  const int64_t group = half / per_block;  // blocks per half
  if (group < 1) return LMS_ERR_TOO_LARGE;

  // (host block, gpu block), ordered by host block so that adjacent host blocks form runs.
  std::vector<std::pair<int64_t, int64_t>> order((size_t)n_pairs);
  for (int64_t i = 0; i < n_pairs; ++i) {
    const int64_t g = out ? pairs[2 * i] : pairs[2 * i + 1];
    const int64_t h = out ? pairs[2 * i + 1] : pairs[2 * i];
    if (g < 0 || h < 0 || (num_gpu_blocks > 0 && g >= num_gpu_blocks) ||
        (num_host_blocks > 0 && h >= num_host_blocks)) {
      // unlike the kernels, the copy engines cannot skip a bad index: it is always refused
      snprintf(g_cuda_msg, sizeof(g_cuda_msg), "block pair %lld (%lld, %lld) is out of range",
               (long long)i, (long long)pairs[2 * i], (long long)pairs[2 * i + 1]);
      return LMS_ERR_INDEX;
    }
    order[(size_t)i] = {h, g};
  }
  std::sort(order.begin(), order.end());
  // Kernel table: (gpu block, position inside its group's half of the staging buffer).
  std::vector<int64_t> table((size_t)n_pairs * 2);
  for (int64_t i = 0; i < n_pairs; ++i) {
    table[(size_t)(2 * i + (out ? 0 : 1))] = order[(size_t)i].second;
    table[(size_t)(2 * i + (out ? 1 : 0))] = i % group;
  }

  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  DeviceState::Staged& st = ds->staged[out ? 0 : 1];
  std::lock_guard<std::mutex> lock(st.mutex);
  if (int rc = staged_setup(st)) return rc;
  // A whole run of adjacent host blocks is one transfer only if consecutive blocks touch.
  const bool runs = host_block_stride == per_block;
  char* gbase = gpu + (long long)layer_begin * gpu_layer_stride;
  char* hbase = host + (long long)layer_begin * host_layer_stride;
  const int64_t n_groups = (n_pairs + group - 1) / group;
  const int ctas = ds->sms * 2;

  // The transfers can alternate between two copy streams (LMS_TUNE_STAGED_STREAMS = 2).
  // Measured, it changes nothing: what a 2 MiB transfer loses against one large copy (about
  // 3 us each) is spent inside the copy engine, not between transfers.
  const int n_copy = tuned(LMS_TUNE_STAGED_STREAMS, 1) >= 2 ? 2 : 1;
  cudaStream_t c0 = st.copy[0], c1 = st.copy[n_copy - 1];

  return with_host_table(table.data(), n_pairs, stream, [&](const int64_t* dev_table) {
    if (!out) {
      // the DMA reads host memory that earlier work of the caller's stream may still write
      LMS_CUDA(cudaEventRecord(st.start, stream));
      LMS_CUDA(cudaStreamWaitEvent(c0, st.start, 0));
      if (n_copy == 2) LMS_CUDA(cudaStreamWaitEvent(c1, st.start, 0));
    }
    for (int64_t g = 0; g < n_groups; ++g) {
      const int b = (int)(g & 1);
      const int64_t first = g * group;
      const int64_t count = std::min(group, n_pairs - first);
      char* buf = staging + (int64_t)b * half;
      // the transfers of one group, spread over the copy streams; c0 ends up behind both
      auto dma = [&]() -> int {
        int turn = 0;
        for (int64_t k = 0; k < count;) {
          int64_t len = 1;
          if (runs)
            while (k + len < count &&
                   order[(size_t)(first + k + len)].first == order[(size_t)(first + k)].first + len)
              ++len;
          char* h = hbase + order[(size_t)(first + k)].first * host_block_stride;
          char* d = buf + k * per_block;
          cudaStream_t cs = (turn++ & 1) ? c1 : c0;
          if (out)
            LMS_CUDA(cudaMemcpyAsync(h, d, (size_t)(len * per_block), cudaMemcpyDeviceToHost, cs));
          else
            LMS_CUDA(cudaMemcpyAsync(d, h, (size_t)(len * per_block), cudaMemcpyHostToDevice, cs));
          k += len;
        }
        if (n_copy == 2) {
          LMS_CUDA(cudaEventRecord(st.join, c1));
          LMS_CUDA(cudaStreamWaitEvent(c0, st.join, 0));
        }
        return LMS_OK;
      };
      auto kernel = [&]() -> int {
        if (out)
          return chunk_copy(gbase, gpu_layer_stride, gpu_block_stride, buf, chunk_bytes,
                            per_block, chunk_bytes, nl, dev_table + 2 * first, count,
                            num_gpu_blocks, group, /*layer_major=*/0, kWhereSwapOut,
                            tuned_variant(LMS_TUNE_COPY_VARIANT, 3), 0, ctas, stream);
        return chunk_copy(buf, chunk_bytes, per_block, gbase, gpu_layer_stride,
                          gpu_block_stride, chunk_bytes, nl, dev_table + 2 * first, count, group,
                          num_gpu_blocks, /*layer_major=*/0, kWhereSwapIn,
                          tuned_variant(LMS_TUNE_COPY_VARIANT, 3), 0, ctas, stream);
      };
      if (out) {
        if (g >= 2) LMS_CUDA(cudaStreamWaitEvent(stream, st.freed[b], 0));
        if (int rc = kernel()) return rc;
        LMS_CUDA(cudaEventRecord(st.ready[b], stream));
        LMS_CUDA(cudaStreamWaitEvent(c0, st.ready[b], 0));
        if (n_copy == 2) LMS_CUDA(cudaStreamWaitEvent(c1, st.ready[b], 0));
        if (int rc = dma()) return rc;
        LMS_CUDA(cudaEventRecord(st.freed[b], c0));
      } else {
        if (g >= 2) {
          LMS_CUDA(cudaStreamWaitEvent(c0, st.freed[b], 0));
          if (n_copy == 2) LMS_CUDA(cudaStreamWaitEvent(c1, st.freed[b], 0));
        }
        if (int rc = dma()) return rc;
        LMS_CUDA(cudaEventRecord(st.ready[b], c0));
        LMS_CUDA(cudaStreamWaitEvent(stream, st.ready[b], 0));
        if (int rc = kernel()) return rc;
        LMS_CUDA(cudaEventRecord(st.freed[b], stream));
      }
    }
    if (out) {
      // the caller's stream completes when the last transfers have landed in host memory
      LMS_CUDA(cudaStreamWaitEvent(stream, st.freed[(n_groups - 1) & 1], 0));
      if (n_groups >= 2) LMS_CUDA(cudaStreamWaitEvent(stream, st.freed[n_groups & 1], 0));
    }
    return (int)LMS_OK;
  });
}

}  // namespace

extern "C" {
#pragma GCC visibility push(default)

int lms_swap_blocks_dma(int direction, void* gpu, int64_t gpu_layer_stride,
                        int64_t gpu_block_stride, void* host,
                        int64_t host_block_stride, int64_t host_layer_stride,
                        int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                        const int64_t* host_pairs, int64_t n_pairs,
                        int64_t num_gpu_blocks, int64_t num_host_blocks,
                        void* stream) {
  return swap_blocks_dma(direction, (char*)gpu, gpu_layer_stride, gpu_block_stride,
                         (char*)host, host_block_stride, host_layer_stride, chunk_bytes,
                         layer_begin, layer_end, host_pairs, n_pairs, num_gpu_blocks,
                         num_host_blocks, (cudaStream_t)stream);
}

int lms_swap_blocks_staged(int direction, void* gpu, int64_t gpu_layer_stride,
                           int64_t gpu_block_stride, void* host,
                           int64_t host_block_stride, int64_t host_layer_stride,
                           int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                           const int64_t* host_pairs, int64_t n_pairs,
                           int64_t num_gpu_blocks, int64_t num_host_blocks,
                           void* staging, int64_t staging_bytes, void* stream) {
  return swap_blocks_staged(direction, (char*)gpu, gpu_layer_stride, gpu_block_stride,
                            (char*)host, host_block_stride, host_layer_stride, chunk_bytes,
                            layer_begin, layer_end, host_pairs, n_pairs, num_gpu_blocks,
                            num_host_blocks, (char*)staging, staging_bytes,
                            (cudaStream_t)stream);
}

int lms_swap_blocks_host(int direction, void* gpu, int64_t gpu_layer_stride,
                         int64_t gpu_block_stride, void* host,
                         int64_t host_block_stride, int64_t host_layer_stride,
                         int64_t chunk_bytes, int32_t layer_begin, int32_t layer_end,
                         const int64_t* host_pairs, int64_t n_pairs,
                         int64_t num_gpu_blocks, int64_t num_host_blocks,
                         void* stream) {
  if (tuned(LMS_TUNE_SWAP_ENGINE, 1) == 2)
    return swap_blocks_dma(direction, (char*)gpu, gpu_layer_stride, gpu_block_stride,
                           (char*)host, host_block_stride, host_layer_stride, chunk_bytes,
                           layer_begin, layer_end, host_pairs, n_pairs, num_gpu_blocks,
                           num_host_blocks, (cudaStream_t)stream);
  return with_host_table(host_pairs, n_pairs, stream, [&](const int64_t* pairs) {
    return lms_swap_blocks(direction, gpu, gpu_layer_stride, gpu_block_stride, host,
                           host_block_stride, host_layer_stride, chunk_bytes,
                           layer_begin, layer_end, pairs, n_pairs, num_gpu_blocks,
                           num_host_blocks, stream);
  });
}

int lms_transfer_blocks_host(const void* src, int64_t src_layer_stride,
                             int64_t src_block_stride, void* dst,
                             int64_t dst_layer_stride, int64_t dst_block_stride,
                             int64_t chunk_bytes, int32_t num_layers,
                             const int64_t* host_pairs, int64_t n_pairs,
                             int64_t num_src_blocks, int64_t num_dst_blocks,
                             void* stream) {
  return with_host_table(host_pairs, n_pairs, stream, [&](const int64_t* pairs) {
    return lms_transfer_blocks(src, src_layer_stride, src_block_stride, dst,
                               dst_layer_stride, dst_block_stride, chunk_bytes,
                               num_layers, pairs, n_pairs, num_src_blocks,
                               num_dst_blocks, stream);
  });
}

int lms_peer_enable(int peer_device) {
  int dev = 0;
  LMS_CUDA(cudaGetDevice(&dev));
  if (peer_device == dev) return LMS_OK;
  int can = 0;
  LMS_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return LMS_ERR_PEER;
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return LMS_OK;
  }
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
  return LMS_OK;
}

int lms_host_alloc(int64_t bytes, void** host_ptr, void** device_ptr) {
  if (!host_ptr || !device_ptr) return LMS_ERR_NULL;
  if (bytes <= 0) return LMS_ERR_RANGE;
  void* h = nullptr;
  LMS_CUDA(cudaHostAlloc(&h, (size_t)bytes, cudaHostAllocMapped | cudaHostAllocPortable));
  void* d = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&d, h, 0);
  if (e != cudaSuccess) {
    cudaFreeHost(h);
    return cuda_fail(e, "cudaHostGetDevicePointer");
  }
  *host_ptr = h;
  *device_ptr = d;
  return LMS_OK;
}

int lms_host_free(void* host_ptr) {
  if (!host_ptr) return LMS_OK;
  LMS_CUDA(cudaFreeHost(host_ptr));
  return LMS_OK;
}

int lms_host_register(void* host_ptr, int64_t bytes, void** device_ptr) {
  if (!host_ptr || !device_ptr) return LMS_ERR_NULL;
  if (bytes <= 0) return LMS_ERR_RANGE;
  LMS_CUDA(cudaHostRegister(host_ptr, (size_t)bytes,
                            cudaHostRegisterMapped | cudaHostRegisterPortable));
  void* d = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&d, host_ptr, 0);
  if (e != cudaSuccess) {
    cudaHostUnregister(host_ptr);
    return cuda_fail(e, "cudaHostGetDevicePointer");
  }
  *device_ptr = d;
  return LMS_OK;
}

int lms_host_unregister(void* host_ptr) {
  if (!host_ptr) return LMS_OK;
  LMS_CUDA(cudaHostUnregister(host_ptr));
  return LMS_OK;
}

int lms_ipc_export(void* device_ptr, void* handle64, int64_t* offset) {
  if (!device_ptr || !handle64 || !offset) return LMS_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == LMS_IPC_HANDLE_BYTES, "handle size");
  // The handle names the whole allocation; find its base through the driver.
  typedef int (*GetRangeFn)(unsigned long long*, size_t*, unsigned long long);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qr;
  LMS_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr));
  if (!fn || qr != cudaDriverEntryPointSuccess) return LMS_ERR_UNSUPPORTED;
  unsigned long long base = 0;
  size_t size = 0;
  if (((GetRangeFn)fn)(&base, &size, (unsigned long long)(uintptr_t)device_ptr) != 0)
    return LMS_ERR_RANGE;
  cudaIpcMemHandle_t h;
  LMS_CUDA(cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base));
  memcpy(handle64, &h, sizeof(h));
  *offset = (int64_t)((unsigned long long)(uintptr_t)device_ptr - base);
  return LMS_OK;
}

int lms_ipc_open(const void* handle64, int64_t offset, void** device_ptr) {
  if (!handle64 || !device_ptr) return LMS_ERR_NULL;
  if (offset < 0) return LMS_ERR_RANGE;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* base = nullptr;
  LMS_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *device_ptr = (char*)base + offset;
  return LMS_OK;
}

int lms_ipc_close(void* device_ptr, int64_t offset) {
  if (!device_ptr) return LMS_OK;
  LMS_CUDA(cudaIpcCloseMemHandle((char*)device_ptr - offset));
  return LMS_OK;
}

int lms_selftest_bounded_wait(int64_t limit_us, void* stream) {
  DeviceState* ds = nullptr;
  if (int rc = device_state(&ds)) return rc;
  if (limit_us < 1) limit_us = 1;
  if (limit_us > 1000000) limit_us = 1000000;
  LMS_CUDA(launch_wait_selftest(ds->err.load(std::memory_order_relaxed),
                                (unsigned long long)limit_us * 1000ull, (cudaStream_t)stream));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return LMS_OK;
}

int lms_memcpy_async(void* dst, const void* src, int64_t bytes, void* stream) {
  if (!dst || !src) return bytes == 0 ? LMS_OK : LMS_ERR_NULL;
  if (bytes < 0) return LMS_ERR_RANGE;
  if (bytes == 0) return LMS_OK;
  LMS_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
  return LMS_OK;
}

int64_t lms_launch_count(void) { return g_launches.load(); }

#pragma GCC visibility pop
}  // extern "C"
