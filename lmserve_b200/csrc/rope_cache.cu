// Rotary position embedding fused with the paged cache write, for sm_100a.
//
// In LMServe's attention layer the rotary kernel runs immediately before the cache write
// (models/llama.py:156-167 -> models/layers/attention.py:76-85): K is read, rotated, written
// to a temporary, then read again and scattered into the paged cache.  Here one launch
// rotates Q into its output buffer, rotates K straight into the cache row its slot selects
// (and into a K output buffer if the caller wants one), and copies V into the cache.
//
// Arithmetic follows LMServe's Triton kernel (ops/triton/rotary_embedding.py:5-66), element
// type in, element type out:
//   x = head[0 : D/2], y = head[D/2 : D]          (rotate-half pairing)
//   out_x = x * cos[i]       - y * sin[i]
//   out_y = y * cos[D/2 + i] + x * sin[D/2 + i]
// with cos = cos_sin_cache[pos, 0:D], sin = cos_sin_cache[pos, D:2D].  Two evaluations of that
// expression exist and both are offered:
//   * contracted (FUSED): what the Triton compiler emits for a GPU - the first product of each
//     line is fused into the sum, the second product is rounded on its own:
//       out_x = fma(x, cos[i], -rn(y * sin[i])),  out_y = fma(y, cos[D/2+i], rn(x * sin[D/2+i]))
//     (measured on B200 against a compiled Triton kernel of the same two lines: identical);
//   * every product and every sum rounded to the element type, which is the Triton language
//     semantics and what the Triton interpreter computes.  The *_rn intrinsics keep the
//     compiler from contracting, so the result is bit-identical to one rounded operation at a
//     time.
// The two differ by one unit in the last place in about a quarter of the elements.
//
// One thread owns 8 consecutive x elements and the 8 matching y elements of one head of one
// token (two 16-byte loads from the head, four from the cos/sin row, two 16-byte stores).
// Heads are numbered [0, NH) = Q, [NH, NH+NKV) = K, [NH+NKV, NH+2*NKV) = V (copied).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.cuh"

namespace lms {

namespace {

template <class T2>
struct __align__(16) Pack8 {
  T2 v[4];  // 8 elements = 16 bytes, moved as one 16-byte access
};

__device__ __forceinline__ void ld16(void* dst, const char* p) {
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ void st16(char* p, const void* src) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(src);
}

__device__ __forceinline__ __half2 mul_rn(__half2 a, __half2 b) { return __hmul2_rn(a, b); }
__device__ __forceinline__ __half2 add_rn(__half2 a, __half2 b) { return __hadd2_rn(a, b); }
__device__ __forceinline__ __half2 sub_rn(__half2 a, __half2 b) { return __hsub2_rn(a, b); }
__device__ __forceinline__ __nv_bfloat162 mul_rn(__nv_bfloat162 a, __nv_bfloat162 b) { return __hmul2_rn(a, b); }
__device__ __forceinline__ __nv_bfloat162 add_rn(__nv_bfloat162 a, __nv_bfloat162 b) { return __hadd2_rn(a, b); }
__device__ __forceinline__ __nv_bfloat162 sub_rn(__nv_bfloat162 a, __nv_bfloat162 b) { return __hsub2_rn(a, b); }

__device__ __forceinline__ __half2 fma_rn(__half2 a, __half2 b, __half2 c) { return __hfma2(a, b, c); }
__device__ __forceinline__ __nv_bfloat162 fma_rn(__nv_bfloat162 a, __nv_bfloat162 b, __nv_bfloat162 c) { return __hfma2(a, b, c); }
__device__ __forceinline__ __half2 neg(__half2 a) { return __hneg2(a); }
__device__ __forceinline__ __nv_bfloat162 neg(__nv_bfloat162 a) { return __hneg2(a); }

template <class T2, int THREADS, bool FUSED>
__global__ void __launch_bounds__(THREADS)
rope_cache_kernel(const RopeParams p, const int items_per_head, const int heads_total,
                  const long long n_items) {
  // item = (t * heads_total + h) * items_per_head + j; the arithmetic needs no memory and is
  // done before the programmatic-launch wait (32-bit division where the launch allows it)
  const long long item = (long long)blockIdx.x * THREADS + threadIdx.x;
  int j, h, t;
  if (n_items <= 0x7fffffffll) {
    const unsigned it = (unsigned)item;
    const unsigned q = it / (unsigned)items_per_head;
    j = (int)(it - q * (unsigned)items_per_head);
    t = (int)(q / (unsigned)heads_total);
    h = (int)(q - (unsigned)t * (unsigned)heads_total);
  } else {
    j = (int)(item % items_per_head);
    const long long q = item / items_per_head;
    h = (int)(q % heads_total);
    t = (int)(q / heads_total);
  }
  const int half_bytes = p.head_dim;          // D/2 elements * 2 bytes
  const int head_bytes = 2 * p.head_dim;
  const int vec = j * 16;                     // byte offset of this thread's x vector in the head
  const bool is_q = h < p.num_heads;
  const bool is_k = !is_q && h < p.num_heads + p.num_kv_heads;
  const int kvh = is_q ? 0 : (is_k ? h - p.num_heads : h - p.num_heads - p.num_kv_heads);
  const char* src = is_q ? p.q + (long long)t * p.q_tok + (long long)h * head_bytes
                  : is_k ? p.k + (long long)t * p.k_tok + (long long)kvh * head_bytes
                         : p.v + (long long)t * p.v_tok + (long long)kvh * head_bytes;
  // Hints only (a prefetch returns nothing and L2 is the point of coherence): the payload
  // lines start their way into L2 while the previous kernel of the stream is still draining.
  if (p.prefetch && item < n_items && (vec & 127) == 0) {
    prefetch_l2(src + vec);
    prefetch_l2(src + half_bytes + vec);
  }
  // Programmatic dependent launch, as in the cache-write kernel: resident early, but nothing
  // is read or written before the previous kernel of the stream has completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (item >= n_items) return;

  // Independent loads first: position, slot, payload.
  long long pos = p.pos64 ? reinterpret_cast<const long long*>(p.positions)[t]
                          : (long long)reinterpret_cast<const int*>(p.positions)[t];
  const bool to_cache = !is_q && p.kcache != nullptr;
  long long slot = -1;
  if (to_cache) slot = p.slots[t];

  Pack8<T2> x, y;
  ld16(&x, src + vec);
  ld16(&y, src + half_bytes + vec);

  // Destination row in the cache (K and V heads).
  long long cache_off = -1;
  if (to_cache && slot >= 0) {
    if (p.checks && p.num_slots > 0 && slot >= p.num_slots) {
      if (j == 0 && kvh == 0) report(p.err, kErrBadSlot, kWhereRope, t, slot);
    } else {
      long long blk, in;
      if (p.block_shift >= 0) {
        blk = slot >> p.block_shift;
        in = slot & ((1ll << p.block_shift) - 1);
      } else {
        blk = slot / p.block_size;
        in = slot - blk * p.block_size;
      }
      cache_off = blk * p.block_stride + in * p.slot_stride + (long long)kvh * head_bytes;
    }
  }

  if (!is_q && !is_k) {  // V: plain copy into the cache
    if (cache_off >= 0) {
      st16(p.vcache + cache_off + vec, &x);
      st16(p.vcache + cache_off + half_bytes + vec, &y);
    }
    return;
  }

  if (p.checks && (pos < 0 || (p.max_pos > 0 && pos >= p.max_pos))) {
    if (j == 0 && h == 0) report(p.err, kErrBadPosition, kWhereRope, t, pos);
    return;
  }
  const char* cs = p.cos_sin + pos * p.cs_row;
  Pack8<T2> cx, cy, sx, sy;
  ld16(&cx, cs + vec);
  ld16(&cy, cs + half_bytes + vec);
  ld16(&sx, cs + head_bytes + vec);
  ld16(&sy, cs + head_bytes + half_bytes + vec);

  Pack8<T2> ox, oy;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (FUSED) {
      ox.v[i] = fma_rn(x.v[i], cx.v[i], neg(mul_rn(y.v[i], sx.v[i])));
      oy.v[i] = fma_rn(y.v[i], cy.v[i], mul_rn(x.v[i], sy.v[i]));
    } else {
      ox.v[i] = sub_rn(mul_rn(x.v[i], cx.v[i]), mul_rn(y.v[i], sx.v[i]));
      oy.v[i] = add_rn(mul_rn(y.v[i], cy.v[i]), mul_rn(x.v[i], sy.v[i]));
    }
  }

  if (is_q) {
    char* d = p.q_out + (long long)t * p.qo_tok + (long long)h * head_bytes;
    st16(d + vec, &ox);
    st16(d + half_bytes + vec, &oy);
    return;
  }
  if (p.k_out != nullptr) {
    char* d = p.k_out + (long long)t * p.ko_tok + (long long)kvh * head_bytes;
    st16(d + vec, &ox);
    st16(d + half_bytes + vec, &oy);
  }
  if (cache_off >= 0) {
    st16(p.kcache + cache_off + vec, &ox);
    st16(p.kcache + cache_off + half_bytes + vec, &oy);
  }
}

}  // namespace

cudaError_t launch_rope_cache(const RopeParams& p_in, bool pdl, cudaStream_t stream) {
  RopeParams p = p_in;
  p.block_shift = -1;
  if (p.block_size > 0 && (p.block_size & (p.block_size - 1)) == 0) {
    p.block_shift = 0;
    while ((1 << p.block_shift) < p.block_size) ++p.block_shift;
  }
  constexpr int THREADS = 256;
  const int items_per_head = p.head_dim / 16;  // 8 x-elements per thread, D/2 x-elements per head
  // V heads only take part when there is a cache to copy them into.
  const int heads_total = p.num_heads + p.num_kv_heads + (p.kcache != nullptr ? p.num_kv_heads : 0);
  const long long n_items = (long long)p.num_tokens * heads_total * items_per_head;
  if (n_items <= 0) return cudaSuccess;
  const long long ctas = (n_items + THREADS - 1) / THREADS;
  if (ctas > 0x7fffffffll) return cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3(THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  if (p.is_bf16)
    return p.fused ? cudaLaunchKernelEx(&cfg, rope_cache_kernel<__nv_bfloat162, THREADS, true>, p,
                                        items_per_head, heads_total, n_items)
                   : cudaLaunchKernelEx(&cfg, rope_cache_kernel<__nv_bfloat162, THREADS, false>, p,
                                        items_per_head, heads_total, n_items);
  return p.fused ? cudaLaunchKernelEx(&cfg, rope_cache_kernel<__half2, THREADS, true>, p,
                                      items_per_head, heads_total, n_items)
                 : cudaLaunchKernelEx(&cfg, rope_cache_kernel<__half2, THREADS, false>, p,
                                      items_per_head, heads_total, n_items);
}

}  // namespace lms
