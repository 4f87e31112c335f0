// Per-step index preparation on the device, for sm_100a.
//
// LMServe's model worker rebuilds, on the host and for every step, about ten small tensors from
// the scheduler's request list and uploads each one by itself
// (runtime/worker/llm_worker/model_worker.py:310-433): flattened token ids, position ids,
// cu_seqlens_q, the page table (indptr / indices / last-page lengths) and, through
// flashinfer.get_seq_lens + get_batch_indices_positions, the (batch index, position) pair of
// every new token.  Here the host uploads ONE packed int32 buffer (four numbers per request,
// the concatenated block ids, the token ids) and one launch derives everything, plus the slot
// mapping the cache-write kernels take:
//
//   cu_seqlens_q[b]        = sum of input_len[0..b)
//   kv_block_indptrs[b]    = sum of num_blocks[0..b)
//   kv_last_block_lens[b]  = (context_len[b] - 1) mod block_size + 1        (floor modulo)
//   seq_len[b]             = max(num_blocks[b] - 1, 0) * block_size + kv_last_block_lens[b]
//   for token i of request b, off = i - cu_seqlens_q[b]:
//     position_ids[i]      = filled_len[b] + off
//     batch_indices[i]     = b
//     positions[i]         = seq_len[b] - input_len[b] + off
//     slot_mapping[i]      = block_ids[kv_block_indptrs[b] + positions[i] / block_size] * block_size
//                            + positions[i] % block_size        (-1 if the page is not in the table)
//   kv_block_indices[j]    = block_ids[j];  input_ids[i] = (int64) token_ids[i]
//   decode_kv_block_indptrs[d] = kv_block_indptrs[num_prefill + d] - kv_block_indptrs[num_prefill]
//                            (the page table of the decode requests alone, for their attention plan)
//
// Every CTA scans the (small) per-request arrays into shared memory by itself, so there is no
// grid-wide dependency; CTA 0 also writes the per-request outputs.  Tokens find their request
// by binary search in the shared cu_seqlens_q.
#include "kernels.cuh"

namespace lms {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ int warp_inclusive_scan(int v) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, v, d);
    if ((threadIdx.x & 31) >= d) v += n;
  }
  return v;
}

// out[0] = 0, out[b + 1] = in[0] + ... + in[b]; all threads of the CTA take part.
__device__ void cta_exclusive_scan(const int* __restrict__ in, int n, int* out, int* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int carry = 0;
  if (threadIdx.x == 0) out[0] = 0;
  for (int base = 0; base < n; base += kThreads) {
    const int i = base + threadIdx.x;
    int v = i < n ? in[i] : 0;
    v = warp_inclusive_scan(v);
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
      int s = lane < kThreads / 32 ? warp_sums[lane] : 0;
      s = warp_inclusive_scan(s);
      if (lane < kThreads / 32) warp_sums[lane] = s;
    }
    __syncthreads();
    const int before = warp > 0 ? warp_sums[warp - 1] : 0;
    if (i < n) out[i + 1] = carry + before + v;
    carry += warp_sums[kThreads / 32 - 1];
    __syncthreads();
  }
}

__device__ __forceinline__ int floor_mod(int a, int m) {
  const int r = a % m;
  return r < 0 ? r + m : r;
}

__global__ void __launch_bounds__(kThreads) step_indices_kernel(const StepIndexParams p) {
  extern __shared__ int smem[];
  int* cu_q = smem;                    // [batch + 1]
  int* indptr = smem + p.batch + 1;    // [batch + 1]
  __shared__ int warp_sums[kThreads / 32];

  cta_exclusive_scan(p.input_len, p.batch, cu_q, warp_sums);
  cta_exclusive_scan(p.num_blocks, p.batch, indptr, warp_sums);
  __syncthreads();

  if (blockIdx.x == 0) {
    for (int b = threadIdx.x; b <= p.batch; b += kThreads) {
      if (p.cu_seqlens_q) p.cu_seqlens_q[b] = cu_q[b];
      if (p.kv_block_indptrs) p.kv_block_indptrs[b] = indptr[b];
      if (b < p.batch && p.kv_last_block_lens)
        p.kv_last_block_lens[b] = floor_mod(p.context_len[b] - 1, p.block_size) + 1;
      if (p.decode_kv_block_indptrs && b >= p.num_prefill && b <= p.num_prefill + p.num_decode)
        p.decode_kv_block_indptrs[b - p.num_prefill] = indptr[b] - indptr[p.num_prefill];
    }
  }

  const long long total = p.total_tokens + p.total_blocks;
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < total;
       i += (long long)gridDim.x * kThreads) {
    if (i >= p.total_tokens) {
      const long long j = i - p.total_tokens;
      if (p.kv_block_indices) p.kv_block_indices[j] = p.block_ids[j];
      continue;
    }
    // Tokens beyond what the requests account for (a caller-side inconsistency) get no request.
    if (i >= cu_q[p.batch]) {
      if (p.batch_indices) p.batch_indices[i] = -1;
      if (p.positions) p.positions[i] = 0;
      if (p.position_ids) p.position_ids[i] = 0;
      if (p.slot_mapping) p.slot_mapping[i] = -1;
      if (p.input_ids) p.input_ids[i] = p.token_ids[i];
      if (p.checks) report(p.err, kErrBadPosition, kWhereStepIndices, i, cu_q[p.batch]);
      continue;
    }
    // Largest b with cu_q[b] <= i (requests without new tokens are stepped over).
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (cu_q[mid] <= (int)i) lo = mid; else hi = mid;
    }
    const int b = lo;
    const int off = (int)i - cu_q[b];
    const int nb = indptr[b + 1] - indptr[b];
    const int last = floor_mod(p.context_len[b] - 1, p.block_size) + 1;
    const int seq_len = (nb > 1 ? nb - 1 : 0) * p.block_size + last;
    const int pos = seq_len - p.input_len[b] + off;
    if (p.position_ids) p.position_ids[i] = p.filled_len[b] + off;
    if (p.batch_indices) p.batch_indices[i] = b;
    if (p.positions) p.positions[i] = pos;
    if (p.input_ids) p.input_ids[i] = p.token_ids[i];
    if (p.slot_mapping) {
      long long slot = -1;
      const int page = pos >= 0 ? pos / p.block_size : -1;
      if (page >= 0 && page < nb) {
        slot = (long long)p.block_ids[indptr[b] + page] * p.block_size + (pos - page * p.block_size);
      } else if (p.checks) {
        report(p.err, kErrBadPosition, kWhereStepIndices, i, pos);
      }
      p.slot_mapping[i] = slot;
    }
  }
}

}  // namespace

cudaError_t launch_step_indices(const StepIndexParams& p, int sms, cudaStream_t stream) {
  const long long total = p.total_tokens + p.total_blocks;
  long long ctas = (total + kThreads - 1) / kThreads;
  if (ctas < 1) ctas = 1;  // the per-request outputs are written even without tokens
  const long long cap = 4ll * (sms > 0 ? sms : 148);
  if (ctas > cap) ctas = cap;
  const size_t smem = 2 * sizeof(int) * (size_t)(p.batch + 1);
  step_indices_kernel<<<(unsigned)ctas, kThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace lms
