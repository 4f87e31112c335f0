// Parameter blocks and host-side launchers of the data-movement kernels.
// The C ABI (capi.cu) validates arguments, fills these structs and calls the
// launchers; the kernels themselves live in write_rows.cu, chunk_copy.cu, rope_cache.cu and
// step_indices.cu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "kv_common.cuh"

namespace lms {

// Kernel ids written into ErrRecord::where.
enum : unsigned int {
  kWhereWrite = 1,
  kWhereCopyBlocks = 2,
  kWhereSwapOut = 3,
  kWhereSwapIn = 4,
  kWhereTransfer = 5,
  kWhereRope = 6,
  kWhereSelfTest = 7,
  kWhereStepIndices = 8,
};

// ------------------------------------------------------------ paged cache write
struct WriteParams {
  const char* key;
  const char* value;
  char* kcache;
  char* vcache;
  const long long* slots;          // direct addressing: slot per token (nullptr in paged mode)
  // Paged addressing (slots == nullptr): token t belongs to request batch_idx[t] at position
  // positions[t]; its slot is page_indices[page_indptr[b] + pos / BS] * BS + pos % BS.
  const int* batch_idx;
  const int* positions;
  const int* page_indices;
  const int* page_indptr;
  int num_requests;                // paged: entries of page_indptr minus one, 0 = not known
  long long key_tok, val_tok;      // bytes between consecutive tokens
  long long key_layer, val_layer;  // bytes between consecutive layers (inputs)
  long long cache_layer;           // bytes between consecutive layers (cache)
  long long block_stride;          // bytes between consecutive cache blocks
  long long slot_stride;           // bytes between consecutive slots in a block
  long long slot_layer;            // elements between per-layer slot tables (0 = shared)
  long long num_slots;             // bound for the debug checks (0 = unchecked)
  int num_tokens;
  int num_layers;
  int block_size;
  int block_shift;      // log2(block_size) or -1
  int row_bytes;
  int tok_tile;         // tokens per CTA (vector kernels)
  int tiles_per_layer;
  int piece_bytes;      // bulk kernel: bytes moved per lane
  int pieces_per_row;
  ErrRecord* err;
  int checks;
  int prefetch;         // untiled kernels: prefetch the source lines into L2 before the launch wait
};

// variant: 0 = 16-byte vectors, 1 = 32-byte vectors, 2 = bulk copies;
// vpt: vectors per thread per pipeline batch (2, 4 or 8);
// pdl: launch the untiled kernel with programmatic stream serialization
cudaError_t launch_write(const WriteParams& p, int variant, int tile_bytes,
                         int vpt, int sms, bool pdl, cudaStream_t stream);
// Name of the kernel launch_write would run for this geometry under `variant` (-1 = built-in).
const char* write_kernel_name(int variant, long long row_bytes, long long total_bytes);

// ------------------------------------------------------------ chunk copies
// One kernel family serves copy_blocks, swap-out, swap-in and transfer: every
// unit of work copies (a slice of) the chunk of one (layer, pair).
struct CopyParams {
  const char* src;
  char* dst;
  long long src_layer, src_block;  // byte strides on the source side
  long long dst_layer, dst_block;  // byte strides on the destination side
  const long long* pairs;          // [n_pairs][2] = (src block, dst block)
  long long n_pairs;
  long long num_src_blocks, num_dst_blocks;  // debug-check bounds (0 = unchecked)
  long long units;                 // num_layers * n_pairs * slices
  int num_layers;
  int layer_major;   // 1: consecutive units walk pairs of one layer; 0: layers of one pair
  int chunk_bytes;
  int slice_bytes;   // bytes one CTA iteration (vector) / one lane (bulk) moves
  int slices;        // slices per chunk
  ErrRecord* err;
  unsigned int where;
  int checks;
  int pdl;           // untiled kernel: launch with programmatic stream serialization
};

// variant as above; policy: 0 = default caching, 1 = sources kept in L2 and
// destinations streamed (fan-out copies).
cudaError_t launch_chunk_copy(const CopyParams& p, int variant, int policy,
                              int grid_ctas, cudaStream_t stream);

// ------------------------------------------------------------ rotary embedding + cache write
struct RopeParams {
  const char* q;
  const char* k;
  const char* v;          // unused when there is no cache
  long long q_tok, k_tok, v_tok;  // bytes between consecutive tokens
  const void* positions;  // int32 or int64 [T]
  int pos64;
  const char* cos_sin;    // [max_pos, 2 * head_dim] elements: cos row then sin row
  long long cs_row;       // bytes between consecutive positions
  char* q_out;
  long long qo_tok;
  char* k_out;            // optional rotated-K output, nullptr to skip
  long long ko_tok;
  char* kcache;           // nullptr (with vcache) = rotary embedding only
  char* vcache;
  long long block_stride, slot_stride;
  const long long* slots;
  long long num_slots, max_pos;  // debug-check bounds (0 = unchecked)
  int num_tokens, num_heads, num_kv_heads, head_dim;
  int block_size, block_shift;
  int is_bf16;
  int fused;  // 1: contracted as the Triton compiler emits it, 0: every operation rounded
  int prefetch;  // prefetch the payload lines into L2 before the launch wait
  ErrRecord* err;
  int checks;
};

cudaError_t launch_rope_cache(const RopeParams& p, bool pdl, cudaStream_t stream);

// ------------------------------------------------------------ per-step index preparation
struct StepIndexParams {
  const int* input_len;    // [batch] new tokens of each request
  const int* filled_len;   // [batch] tokens already in the cache
  const int* context_len;  // [batch] tokens in the cache after this step
  const int* num_blocks;   // [batch] entries of each request's block table
  const int* block_ids;    // [total_blocks] the block tables, concatenated
  const int* token_ids;    // [total_tokens], read only when input_ids is set
  int batch;
  int block_size;
  long long total_tokens, total_blocks;
  int* position_ids;        // [total_tokens]      every output may be nullptr
  int* cu_seqlens_q;        // [batch + 1]
  int* kv_block_indptrs;    // [batch + 1]
  int* kv_block_indices;    // [total_blocks]
  int* kv_last_block_lens;  // [batch]
  int* batch_indices;       // [total_tokens]
  int* positions;           // [total_tokens]
  long long* slot_mapping;  // [total_tokens]
  long long* input_ids;     // [total_tokens]
  // Page-table offsets of the decode requests alone (requests [num_prefill, num_prefill +
  // num_decode) of the sorted batch), rebased to start at 0: [num_decode + 1]
  int* decode_kv_block_indptrs;
  int num_prefill, num_decode;
  ErrRecord* err;
  int checks;
};

cudaError_t launch_step_indices(const StepIndexParams& p, int sms, cudaStream_t stream);

// One warp waits (bounded) on an mbarrier that is never completed; see lms_selftest_bounded_wait.
cudaError_t launch_wait_selftest(ErrRecord* err, unsigned long long limit_ns, cudaStream_t stream);

}  // namespace lms
