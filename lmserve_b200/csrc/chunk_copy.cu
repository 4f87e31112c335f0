// Whole-chunk copies for sm_100a: copy-on-write block copy, GPU<->host swap and
// prefill->decode transfer are the same movement with different address maps:
//   dst_base + l*dst_layer + dst_p*dst_block  <-  src_base + l*src_layer + src_p*src_block
// for every (src_p, dst_p) pair and every layer l, chunk_bytes each.
//
// A chunk is cut into slices; the flattened (layer, pair, slice) space is the
// unit list, walked by a persistent grid.  Each CTA first turns its next batch
// of units into (source offset, destination offset) couples in shared memory -
// one thread per unit does the index-table load, the bounds check and the
// divisions - and then streams the slices with no dependent global load and
// no division in the copy loop.
//
// Bound: HBM for copy_blocks (chunk_bytes written per pair per layer, sources
// re-read from L2 when one block fans out to many), PCIe for swap, NVLink for
// transfer; the kernel is identical, only grid size and cache policy differ.
#include "kernels.cuh"

namespace lms {

namespace {

constexpr int kStage = 128;  // units staged per CTA per round

struct UnitAddr {
  long long src;  // byte offset from p.src, or -1 for a unit to skip
  long long dst;  // byte offset from p.dst
  int bytes;      // length of this slice (only a chunk's last slice is short)
};

// Decodes unit u and looks its pair up.  Runs once per unit (not per thread).
__device__ __forceinline__ UnitAddr decode_unit(const CopyParams& p, long long u) {
  UnitAddr a;
  const long long q = u / p.slices;
  const int slice = (int)(u - q * p.slices);
  long long pair, layer;
  if (p.layer_major) {
    layer = q / p.n_pairs;
    pair = q - layer * p.n_pairs;
  } else {
    pair = q / p.num_layers;
    layer = q - pair * p.num_layers;
  }
  const longlong2 sd = reinterpret_cast<const longlong2*>(p.pairs)[pair];
  a.src = -1;
  a.dst = 0;
  a.bytes = (slice == p.slices - 1)
                ? p.chunk_bytes - (p.slices - 1) * p.slice_bytes
                : p.slice_bytes;
  if (p.checks) {
    if (sd.x < 0 || (p.num_src_blocks > 0 && sd.x >= p.num_src_blocks)) {
      report(p.err, kErrBadSrcBlock, p.where, pair, sd.x);
      return a;
    }
    if (sd.y < 0 || (p.num_dst_blocks > 0 && sd.y >= p.num_dst_blocks)) {
      report(p.err, kErrBadDstBlock, p.where, pair, sd.y);
      return a;
    }
  }
  const long long so = (long long)slice * p.slice_bytes;
  a.src = layer * p.src_layer + sd.x * p.src_block + so;
  a.dst = layer * p.dst_layer + sd.y * p.dst_block + so;
  return a;
}

template <class Vec, int THREADS, int VPT, int POLICY>
__global__ void __launch_bounds__(THREADS)
chunk_copy_vec(const CopyParams p) {
  __shared__ UnitAddr s_unit[kStage];

  uint64_t pol_src = 0, pol_dst = 0;
  if (POLICY == 1) {
    pol_src = policy_evict_last();
    pol_dst = policy_evict_first();
  }
  const long long stride = gridDim.x;

  for (long long u0 = blockIdx.x; u0 < p.units; u0 += stride * kStage) {
    for (int j = threadIdx.x; j < kStage; j += THREADS) {
      const long long u = u0 + j * stride;
      if (u < p.units) s_unit[j] = decode_unit(p, u);
    }
    __syncthreads();

    for (int j = 0; j < kStage; ++j) {
      const long long u = u0 + j * stride;
      if (u >= p.units) break;
      const UnitAddr a = s_unit[j];
      if (a.src < 0) continue;
      const int n_vec = a.bytes / Vec::kBytes;
      const char* s = p.src + a.src;
      char* d = p.dst + a.dst;
      for (int base = 0; base < n_vec; base += THREADS * VPT) {
        Vec r[VPT];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = base + k * THREADS + threadIdx.x;
          if (v < n_vec) {
            if (POLICY == 1) ld_hint(r[k], s + (long long)v * Vec::kBytes, pol_src);
            else ld(r[k], s + (long long)v * Vec::kBytes);
          }
        }
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = base + k * THREADS + threadIdx.x;
          if (v < n_vec) {
            if (POLICY == 1) st_hint(d + (long long)v * Vec::kBytes, r[k], pol_dst);
            else st(d + (long long)v * Vec::kBytes, r[k]);
          }
        }
      }
    }
    __syncthreads();
  }
}

// Untiled form: thread i owns vector i of the flattened (layer | pair, vector-in-chunk)
// space.  No persistent loop, no shared memory; the pair entry is a broadcast load.
template <class Vec, int THREADS, int POLICY>
__global__ void __launch_bounds__(THREADS)
chunk_copy_direct(const CopyParams p, const int chunk_vecs, const int chunk_shift,
                  const long long n_vec_total) {
  const long long v = (long long)blockIdx.x * THREADS + threadIdx.x;
  long long q;
  int c;
  if (chunk_shift >= 0) {
    q = v >> chunk_shift;
    c = (int)(v & (chunk_vecs - 1));
  } else {
    q = v / chunk_vecs;
    c = (int)(v - q * chunk_vecs);
  }
  long long pair, layer;
  if (p.layer_major) {
    layer = q / p.n_pairs;
    pair = q - layer * p.n_pairs;
  } else {
    pair = q / p.num_layers;
    layer = q - pair * p.num_layers;
  }
  // Programmatic dependent launch (a no-op when the launch does not ask for it): the grid may
  // be resident while the previous kernel of the stream drains; nothing is read or written
  // before that kernel has completed, so stream order is unchanged.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (v >= n_vec_total) return;
  const longlong2 sd = reinterpret_cast<const longlong2*>(p.pairs)[pair];
  if (p.checks) {
    if (sd.x < 0 || (p.num_src_blocks > 0 && sd.x >= p.num_src_blocks)) {
      if (c == 0) report(p.err, kErrBadSrcBlock, p.where, pair, sd.x);
      return;
    }
    if (sd.y < 0 || (p.num_dst_blocks > 0 && sd.y >= p.num_dst_blocks)) {
      if (c == 0) report(p.err, kErrBadDstBlock, p.where, pair, sd.y);
      return;
    }
  }
  const char* s = p.src + layer * p.src_layer + sd.x * p.src_block + (long long)c * Vec::kBytes;
  char* d = p.dst + layer * p.dst_layer + sd.y * p.dst_block + (long long)c * Vec::kBytes;
  Vec r;
  if (POLICY == 1) {
    ld_hint(r, s, policy_evict_last());
    st_hint(d, r, policy_evict_first());
  } else {
    ld(r, s);
    st(d, r);
  }
}

// Bulk (TMA) form: a slice is what ONE lane moves; 32 consecutive units are a
// warp-task.  Every lane issues one bulk load into its own shared-memory
// buffer, the warp waits on one mbarrier, every lane issues one bulk store.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
chunk_copy_bulk(const CopyParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t bars[WARPS];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint64_t* bar = &bars[warp];
  unsigned char* buf = smem + ((size_t)warp * 32 + lane) * p.slice_bytes;

  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();

  const long long n_tasks = (p.units + 31) / 32;
  const long long warp_stride = (long long)gridDim.x * WARPS;
  unsigned parity = 0;

  for (long long task = (long long)blockIdx.x * WARPS + warp; task < n_tasks;
       task += warp_stride) {
    const long long u = task * 32 + lane;
    const char* src = nullptr;
    char* dst = nullptr;
    unsigned bytes = 0;
    if (u < p.units) {
      const UnitAddr a = decode_unit(p, u);
      if (a.src >= 0) {
        src = p.src + a.src;
        dst = p.dst + a.dst;
        bytes = (unsigned)a.bytes;
      }
    }
    const unsigned total = __reduce_add_sync(0xffffffffu, bytes);
    if (total == 0) continue;
    if (lane == 0) mbar_expect_tx(bar, total);
    __syncwarp();
    if (bytes) bulk_g2s(buf, src, bytes, bar);
    const unsigned phase = parity;
    parity ^= 1u;
    const bool ok = mbar_wait_bounded(bar, phase);
    if (__any_sync(0xffffffffu, !ok)) {
      if (lane == 0) report(p.err, kErrWaitTimeout, p.where, task, 0);
      mbar_wait_bounded(bar, phase, 100000000ull);
      break;
    }
    if (bytes) {
      bulk_s2g(dst, buf, bytes);
      bulk_commit();
      bulk_wait_read_all();
    }
    __syncwarp();
  }
  bulk_wait_all();
}

// The wait of the bulk kernels, exercised on a barrier nobody completes.
__global__ void __launch_bounds__(32) wait_selftest_kernel(ErrRecord* err,
                                                          unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const bool ok = mbar_wait_bounded(&bar, 0, limit_ns);
  if (__any_sync(0xffffffffu, !ok) && threadIdx.x == 0)
    report(err, kErrWaitTimeout, kWhereSelfTest, 0, (long long)limit_ns);
}

template <class Vec, int POLICY, int THREADS = 256, int VPT = 8>
cudaError_t launch_vec(CopyParams p, int grid_ctas, cudaStream_t stream) {
  constexpr int kSlice = THREADS * VPT * Vec::kBytes;  // bytes per CTA iteration
  p.slice_bytes = p.chunk_bytes < kSlice ? p.chunk_bytes : kSlice;
  p.slices = (p.chunk_bytes + p.slice_bytes - 1) / p.slice_bytes;
  p.units = (long long)p.num_layers * p.n_pairs * p.slices;
  long long ctas = grid_ctas;
  if (ctas > p.units) ctas = p.units;
  if (ctas < 1) ctas = 1;
  chunk_copy_vec<Vec, THREADS, VPT, POLICY><<<(unsigned)ctas, THREADS, 0, stream>>>(p);
  return cudaGetLastError();
}

template <class Vec, int POLICY>
cudaError_t launch_direct(const CopyParams& p, cudaStream_t stream) {
  constexpr int THREADS = 256;
  const int chunk_vecs = p.chunk_bytes / Vec::kBytes;
  int shift = -1;
  if ((chunk_vecs & (chunk_vecs - 1)) == 0) {
    shift = 0;
    while ((1 << shift) < chunk_vecs) ++shift;
  }
  const long long n_vec = (long long)p.num_layers * p.n_pairs * chunk_vecs;
  const long long ctas = (n_vec + THREADS - 1) / THREADS;
  if (ctas > 0x7fffffffll) return cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3(THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (p.pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, chunk_copy_direct<Vec, THREADS, POLICY>, p, chunk_vecs, shift, n_vec);
}

}  // namespace

cudaError_t launch_wait_selftest(ErrRecord* err, unsigned long long limit_ns,
                                 cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(err, limit_ns);
  return cudaGetLastError();
}

cudaError_t launch_chunk_copy(const CopyParams& p_in, int variant, int policy,
                              int grid_ctas, cudaStream_t stream) {
  CopyParams p = p_in;
  if (p.n_pairs <= 0 || p.num_layers <= 0) return cudaSuccess;

  const uintptr_t a32 = (uintptr_t)p.src | (uintptr_t)p.dst |
                        (uintptr_t)(p.src_layer | p.src_block | p.dst_layer |
                                    p.dst_block | (long long)p.chunk_bytes);
  if (variant == 1 && (a32 & 31u) != 0) variant = 0;
  if (variant == 3) {
    if ((a32 & 31u) != 0)
      return policy == 1 ? launch_direct<V16, 1>(p, stream) : launch_direct<V16, 0>(p, stream);
    return policy == 1 ? launch_direct<V32, 1>(p, stream) : launch_direct<V32, 0>(p, stream);
  }

  if (variant == 2) {
    constexpr int WARPS = 2;
    constexpr int kLaneBytes = 1024;
    p.slice_bytes = p.chunk_bytes < kLaneBytes ? p.chunk_bytes : kLaneBytes;
    p.slices = (p.chunk_bytes + p.slice_bytes - 1) / p.slice_bytes;
    p.units = (long long)p.num_layers * p.n_pairs * p.slices;
    const size_t smem = (size_t)WARPS * 32 * p.slice_bytes;
    int dev = 0;
    cudaGetDevice(&dev);
    static bool attr_set[64] = {};
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(chunk_copy_bulk<WARPS>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           WARPS * 32 * kLaneBytes);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const long long tasks = (p.units + 31) / 32;
    long long ctas = (tasks + WARPS - 1) / WARPS;
    if (ctas > grid_ctas) ctas = grid_ctas;
    if (ctas < 1) ctas = 1;
    chunk_copy_bulk<WARPS><<<(unsigned)ctas, WARPS * 32, smem, stream>>>(p);
    return cudaGetLastError();
  }
  // Wide CTAs for grids of a few CTAs (the swap): 1024 threads keep 128 KiB in flight per CTA,
  // which a read over PCIe needs to hide its latency without occupying more SMs.
  if (variant == 4) return launch_vec<V16, 0, 1024, 8>(p, grid_ctas, stream);
  if (variant == 1)
    return policy == 1 ? launch_vec<V32, 1>(p, grid_ctas, stream)
                       : launch_vec<V32, 0>(p, grid_ctas, stream);
  return policy == 1 ? launch_vec<V16, 1>(p, grid_ctas, stream)
                     : launch_vec<V16, 0>(p, grid_ctas, stream);
}

}  // namespace lms
