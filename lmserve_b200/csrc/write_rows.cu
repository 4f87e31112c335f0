// Paged KV-cache write ("reshape_and_cache") for sm_100a.
//
// Work: for every (layer, token, K|V) copy one row of row_bytes from the
// projection output into the paged cache at the address the token's slot
// selects; slot < 0 is padding and is skipped.  Pure byte movement, bound by
// HBM bandwidth: 2 * row_bytes read and 2 * row_bytes written per live token
// per layer.
//
// Several implementations share one parameter block.  write_rows_direct is the one the library
// launches by itself; the others were built to be measured against it (they are parity-tested
// and can be selected through the launch tunables) and lost:
//   * write_rows_direct - no tile and no shared memory: thread i owns vector i of the whole
//     launch.  Index arithmetic and an L2 prefetch of its source line come before the
//     programmatic-launch wait, then it issues its index loads and payload load together and
//     stores.
//   * write_rows_pair / write_rows_multi - the same idea with 2 ... 8 vectors per thread in a
//     grid of at most one wave (a thread moves the K and the V vector of 1, 2 or 4 tokens, or
//     2 / 4 independent vectors); write_rows_pair_persistent walks the same tiles with a
//     persistent grid and a two-deep register pipeline.
//   * write_rows_vec  - a CTA owns a tile of tokens of one layer.  Slot loads and the first
//     batch of payload loads are issued together; the slots are then turned into destination
//     byte offsets once, in shared memory, and the tile is streamed as a two-stage software
//     pipeline of 16- or 32-byte vectors (loads of batch b+1 in flight while batch b is stored).
//   * write_rows_bulk - every lane of a warp owns one piece of a row and moves it with a bulk
//     (TMA) copy global -> shared -> global; the warp shares one mbarrier with a bounded wait.
#include "kernels.cuh"

namespace lms {

namespace {

constexpr int kMaxTokTile = 512;

// slot -> byte offset of the row inside one layer's K (or V) plane, or -1.
__device__ __forceinline__ long long slot_offset(const WriteParams& p,
                                                 long long slot, long long index) {
  if (slot < 0) return -1;
  if (p.checks && p.num_slots > 0 && slot >= p.num_slots) {
    report(p.err, kErrBadSlot, kWhereWrite, index, slot);
    return -1;
  }
  long long blk, in;
  if (p.block_shift >= 0) {
    blk = slot >> p.block_shift;
    in = slot & ((1ll << p.block_shift) - 1);
  } else {
    blk = slot / p.block_size;
    in = slot - blk * p.block_size;
  }
  return blk * p.block_stride + in * p.slot_stride;
}

// Splits vector index v of a tile into (token in tile, K|V, vector in row).
template <bool POW2>
__device__ __forceinline__ void split_vec(int v, int row_vecs, int row_shift,
                                          int& ti, int& kv, int& c) {
  if (POW2) {
    ti = v >> (row_shift + 1);
    kv = (v >> row_shift) & 1;
    c = v & (row_vecs - 1);
  } else {
    const int vecs_per_tok = 2 * row_vecs;
    ti = v / vecs_per_tok;
    const int rem = v - ti * vecs_per_tok;
    kv = rem >= row_vecs;
    c = rem - kv * row_vecs;
  }
}

// Slot of token t (index into the call's token list) of `layer`, fetched in two steps so
// that the independent loads of step one can be issued before the payload loads and the
// dependent page-table walk of step two after them.
struct SlotRaw {
  long long a;  // direct: the slot;  paged: batch index
  int b;        // paged: position
  int ip;       // paged: page_indptr[min(t, num_requests)], read on the guess batch_idx[t] == t
};
__device__ __forceinline__ SlotRaw slot_fetch_begin(const WriteParams& p, int layer, int t) {
  SlotRaw r;
  r.b = 0;
  r.ip = 0;
  if (p.slots != nullptr) {
    r.a = p.slots[(long long)layer * p.slot_layer + t];
  } else {
    r.a = p.batch_idx[t];
    r.b = p.positions[t];
    // A decode step appends one token per request, so token t belongs to request t.  When the
    // caller said how many requests the page table has, the request's page-table offset is
    // fetched on that guess together with the two loads above; a right guess leaves one
    // dependent load (the page id) where the plain walk has two.
    if (p.num_requests > 0) r.ip = p.page_indptr[t < p.num_requests ? t : p.num_requests];
  }
  return r;
}
__device__ __forceinline__ long long slot_fetch_end(const WriteParams& p, const SlotRaw& r,
                                                    int t) {
  if (p.slots != nullptr) return r.a;
  if (r.a < 0 || r.b < 0) return -1;  // padding: negative batch index or position
  int pg, in;
  if (p.block_shift >= 0) {
    pg = r.b >> p.block_shift;
    in = r.b & ((1 << p.block_shift) - 1);
  } else {
    pg = r.b / p.block_size;
    in = r.b - pg * p.block_size;
  }
  const int first = (p.num_requests > 0 && r.a == t) ? r.ip : p.page_indptr[r.a];
  const long long page = p.page_indices[first + pg];
  return page * p.block_size + in;
}

template <class Vec, int THREADS, int VPT, bool POW2>
__global__ void __launch_bounds__(THREADS)
write_rows_vec(const WriteParams p, const int row_vecs, const int row_shift) {
  __shared__ long long s_off[kMaxTokTile];

  const int tile = blockIdx.x % p.tiles_per_layer;
  const int layer = blockIdx.x / p.tiles_per_layer;
  const int t0 = tile * p.tok_tile;
  const int nt = min(p.tok_tile, p.num_tokens - t0);

  const char* kin = p.key + (long long)layer * p.key_layer + (long long)t0 * p.key_tok;
  const char* vin = p.value + (long long)layer * p.val_layer + (long long)t0 * p.val_tok;
  char* kout = p.kcache + (long long)layer * p.cache_layer;
  char* vout = p.vcache + (long long)layer * p.cache_layer;
  const int n_vec = nt * 2 * row_vecs;
  constexpr int kBatch = THREADS * VPT;
  const int n_batches = (n_vec + kBatch - 1) / kBatch;

  // Batch b of the tile: VPT vectors per thread, consecutive threads on consecutive vectors.
  auto load_batch = [&](int b, Vec (&r)[VPT]) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = b * kBatch + k * THREADS + threadIdx.x;
      if (v < n_vec) {
        int ti, kv, c;
        split_vec<POW2>(v, row_vecs, row_shift, ti, kv, c);
        const char* s = kv ? vin + (long long)ti * p.val_tok : kin + (long long)ti * p.key_tok;
        ld(r[k], s + (long long)c * Vec::kBytes);
      }
    }
  };
  auto store_batch = [&](int b, const Vec (&r)[VPT]) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = b * kBatch + k * THREADS + threadIdx.x;
      if (v < n_vec) {
        int ti, kv, c;
        split_vec<POW2>(v, row_vecs, row_shift, ti, kv, c);
        const long long off = s_off[ti];
        if (off >= 0) st((kv ? vout : kout) + off + (long long)c * Vec::kBytes, r[k]);
      }
    }
  };

  // The source address of a row depends on the token only, the destination on its slot.
  // So the slot loads and the first batch of payload loads are issued together, before any
  // slot is known: one memory round trip instead of two in series.  Rows of padded tokens
  // are read and dropped.
  constexpr int kSlotsPerThread = (kMaxTokTile + THREADS - 1) / THREADS;
  SlotRaw my_slot[kSlotsPerThread];
#pragma unroll
  for (int k = 0; k < kSlotsPerThread; ++k) {
    const int i = k * THREADS + threadIdx.x;
    if (i < nt) my_slot[k] = slot_fetch_begin(p, layer, t0 + i);
  }

  Vec ra[VPT], rb[VPT];
  load_batch(0, ra);

#pragma unroll
  for (int k = 0; k < kSlotsPerThread; ++k) {
    const int i = k * THREADS + threadIdx.x;
    if (i < nt)
      s_off[i] = slot_offset(p, slot_fetch_end(p, my_slot[k], t0 + i),
                             (long long)layer * p.slot_layer + t0 + i);
  }
  __syncthreads();

  // Software pipeline over the tile: the loads of batch b+1 are in flight while batch b is
  // stored, so the memory system always has requests queued from this CTA.
  for (int b = 0; b < n_batches; b += 2) {
    if (b + 1 < n_batches) load_batch(b + 1, rb);
    store_batch(b, ra);
    if (b + 2 < n_batches) load_batch(b + 2, ra);
    if (b + 1 < n_batches) store_batch(b + 1, rb);
  }
}

// Small launches (one layer of a decode step is 2 MiB): no tile, no shared memory, no
// barrier.  Thread i owns vector i of the flattened (layer, token, K|V, vector-in-row) space;
// it issues its index loads and its payload load together, walks the page table if there is
// one, and stores.  Lanes of a warp that share a token read the same index words (one
// broadcast transaction).  Launch + one memory round trip + the store is all that is left.
template <class Vec, int THREADS, bool POW2>
__global__ void __launch_bounds__(THREADS)
write_rows_direct(const WriteParams p, const int row_vecs, const int row_shift,
                  const long long n_vec_total) {
  // Programmatic dependent launch (a no-op when the launch does not ask for it): this grid
  // may have been made resident while the previous kernel of the stream was still running.
  // Nothing is read or written before that kernel has completed and its writes are visible,
  // so stream order is exactly what it would be without the attribute; only the launch
  // latency is hidden.  The kernel that follows this one is allowed to do the same.
  const long long v = (long long)blockIdx.x * THREADS + threadIdx.x;
  // v = ((layer * T + t) * 2 + kv) * row_vecs + c; the arithmetic needs no memory, so it is
  // done before the wait
  long long q;
  int c;
  if (POW2) {
    c = (int)(v & (row_vecs - 1));
    q = v >> row_shift;
  } else {
    q = v / row_vecs;
    c = (int)(v - q * row_vecs);
  }
  const int kv = (int)(q & 1);
  q >>= 1;
  int layer, t;
  if (n_vec_total <= 0x7fffffffll) {  // 32-bit division where the launch allows it
    layer = (int)((unsigned)q / (unsigned)p.num_tokens);
    t = (int)((unsigned)q - (unsigned)layer * (unsigned)p.num_tokens);
  } else {
    layer = (int)(q / p.num_tokens);
    t = (int)(q - (long long)layer * p.num_tokens);
  }
  const char* src = (kv ? p.value + (long long)layer * p.val_layer + (long long)t * p.val_tok
                        : p.key + (long long)layer * p.key_layer + (long long)t * p.key_tok) +
                    (long long)c * Vec::kBytes;
  // Hints only (see prefetch_l2): the source line and the slot line start their way from DRAM
  // while the previous kernel of the stream is still draining.
  if (p.prefetch && v < n_vec_total) {
    if ((c & (128 / Vec::kBytes - 1)) == 0) prefetch_l2(src);
    if (c == 0 && kv == 0 && (t & 15) == 0 && p.slots != nullptr)
      prefetch_l2(p.slots + (long long)layer * p.slot_layer + t);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (v >= n_vec_total) return;

  const SlotRaw raw = slot_fetch_begin(p, layer, t);
  Vec r;
  ld(r, src);
  const long long off =
      slot_offset(p, slot_fetch_end(p, raw, t), (long long)layer * p.slot_layer + t);
  if (off >= 0)
    st((kv ? p.vcache : p.kcache) + (long long)layer * p.cache_layer + off +
           (long long)c * Vec::kBytes,
       r);
}

// A decode step in at most one wave.  Unit u of a layer is (token t, vector c of the row): the
// thread that owns it moves vector c of the K row AND of the V row of token t, so one slot
// resolution serves two payload vectors, and a thread owns TOK units THREADS apart (the
// accesses of a warp stay contiguous).  The layer is blockIdx.y, which removes the division by
// the token count; all index arithmetic is done before the programmatic-launch wait, all
// 2 * TOK payload loads and the TOK index loads are in flight together, then the stores.
// With TOK = 2 the 40 MiB step of a 70B TP8 shard is 640 CTAs (0.54 of a wave at 8 CTAs per
// SM), so the whole grid is resident - and waiting in griddepcontrol.wait - before the
// previous kernel of the stream has finished.
template <class Vec, int THREADS, int TOK, bool POW2>
__global__ void __launch_bounds__(THREADS)
write_rows_pair(const WriteParams p, const int row_vecs, const int row_shift,
                const int units_per_layer) {
  const int layer = blockIdx.y;
  const int base = blockIdx.x * (THREADS * TOK) + threadIdx.x;
  int t[TOK], c[TOK];
#pragma unroll
  for (int j = 0; j < TOK; ++j) {
    const int u = base + j * THREADS;
    if (POW2) {
      c[j] = u & (row_vecs - 1);
      t[j] = u >> row_shift;
    } else {
      t[j] = u / row_vecs;
      c[j] = u - t[j] * row_vecs;
    }
    if (u >= units_per_layer) t[j] = -1;
  }
  const char* kin = p.key + (long long)layer * p.key_layer;
  const char* vin = p.value + (long long)layer * p.val_layer;
  char* kout = p.kcache + (long long)layer * p.cache_layer;
  char* vout = p.vcache + (long long)layer * p.cache_layer;

  if (p.prefetch) {
#pragma unroll
    for (int j = 0; j < TOK; ++j)
      if (t[j] >= 0 && (c[j] & (128 / Vec::kBytes - 1)) == 0) {
        prefetch_l2(kin + (long long)t[j] * p.key_tok + (long long)c[j] * Vec::kBytes);
        prefetch_l2(vin + (long long)t[j] * p.val_tok + (long long)c[j] * Vec::kBytes);
        if (c[j] == 0 && (t[j] & 15) == 0 && p.slots != nullptr)
          prefetch_l2(p.slots + (long long)layer * p.slot_layer + t[j]);
      }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  SlotRaw raw[TOK];
  Vec rk[TOK], rv[TOK];
#pragma unroll
  for (int j = 0; j < TOK; ++j)
    if (t[j] >= 0) raw[j] = slot_fetch_begin(p, layer, t[j]);
#pragma unroll
  for (int j = 0; j < TOK; ++j)
    if (t[j] >= 0) {
      ld(rk[j], kin + (long long)t[j] * p.key_tok + (long long)c[j] * Vec::kBytes);
      ld(rv[j], vin + (long long)t[j] * p.val_tok + (long long)c[j] * Vec::kBytes);
    }
#pragma unroll
  for (int j = 0; j < TOK; ++j)
    if (t[j] >= 0) {
      const long long off = slot_offset(p, slot_fetch_end(p, raw[j], t[j]),
                                        (long long)layer * p.slot_layer + t[j]);
      if (off >= 0) {
        st(kout + off + (long long)c[j] * Vec::kBytes, rk[j]);
        st(vout + off + (long long)c[j] * Vec::kBytes, rv[j]);
      }
    }
}

// The same units walked by a persistent grid (at most one wave) with a two-deep register
// pipeline: the loads of the CTA's next tile are in flight while the current tile is stored.
// A tile is THREADS * TOK units of one layer; tiles are numbered layer by layer.
template <class Vec, int THREADS, int TOK, bool POW2>
__global__ void __launch_bounds__(THREADS)
write_rows_pair_persistent(const WriteParams p, const int row_vecs, const int row_shift,
                           const int units_per_layer, const int tiles_per_layer,
                           const int n_tiles) {
  struct Tile {
    int layer;
    int t[TOK], c[TOK];
    SlotRaw raw[TOK];
    Vec rk[TOK], rv[TOK];
  };
  auto locate = [&](Tile& x, int tile) {
    x.layer = tile / tiles_per_layer;
    const int base = (tile - x.layer * tiles_per_layer) * (THREADS * TOK) + threadIdx.x;
#pragma unroll
    for (int j = 0; j < TOK; ++j) {
      const int u = base + j * THREADS;
      if (POW2) {
        x.c[j] = u & (row_vecs - 1);
        x.t[j] = u >> row_shift;
      } else {
        x.t[j] = u / row_vecs;
        x.c[j] = u - x.t[j] * row_vecs;
      }
      if (u >= units_per_layer) x.t[j] = -1;
    }
  };
  auto load = [&](Tile& x) {
    const char* kin = p.key + (long long)x.layer * p.key_layer;
    const char* vin = p.value + (long long)x.layer * p.val_layer;
#pragma unroll
    for (int j = 0; j < TOK; ++j)
      if (x.t[j] >= 0) x.raw[j] = slot_fetch_begin(p, x.layer, x.t[j]);
#pragma unroll
    for (int j = 0; j < TOK; ++j)
      if (x.t[j] >= 0) {
        ld(x.rk[j], kin + (long long)x.t[j] * p.key_tok + (long long)x.c[j] * Vec::kBytes);
        ld(x.rv[j], vin + (long long)x.t[j] * p.val_tok + (long long)x.c[j] * Vec::kBytes);
      }
  };
  auto store = [&](const Tile& x) {
    char* kout = p.kcache + (long long)x.layer * p.cache_layer;
    char* vout = p.vcache + (long long)x.layer * p.cache_layer;
#pragma unroll
    for (int j = 0; j < TOK; ++j)
      if (x.t[j] >= 0) {
        const long long off = slot_offset(p, slot_fetch_end(p, x.raw[j], x.t[j]),
                                          (long long)x.layer * p.slot_layer + x.t[j]);
        if (off >= 0) {
          st(kout + off + (long long)x.c[j] * Vec::kBytes, x.rk[j]);
          st(vout + off + (long long)x.c[j] * Vec::kBytes, x.rv[j]);
        }
      }
  };

  Tile a, b;
  int tile = blockIdx.x;
  if (tile < n_tiles) {
    locate(a, tile);
    if (p.prefetch) {
      const char* kin = p.key + (long long)a.layer * p.key_layer;
      const char* vin = p.value + (long long)a.layer * p.val_layer;
#pragma unroll
      for (int j = 0; j < TOK; ++j)
        if (a.t[j] >= 0 && (a.c[j] & (128 / Vec::kBytes - 1)) == 0) {
          prefetch_l2(kin + (long long)a.t[j] * p.key_tok + (long long)a.c[j] * Vec::kBytes);
          prefetch_l2(vin + (long long)a.t[j] * p.val_tok + (long long)a.c[j] * Vec::kBytes);
        }
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tile >= n_tiles) return;
  load(a);
  for (;;) {
    int next = tile + gridDim.x;
    if (next < n_tiles) {
      locate(b, next);
      load(b);
    }
    store(a);
    if (next >= n_tiles) break;
    tile = next;
    next = tile + gridDim.x;
    if (next < n_tiles) {
      locate(a, next);
      load(a);
    }
    store(b);
    if (next >= n_tiles) break;
    tile = next;
  }
}

// VPT independent vectors per thread of the flattened (token, K|V, vector) space of one layer
// (blockIdx.y); every vector resolves its own slot.
template <class Vec, int THREADS, int VPT, bool POW2>
__global__ void __launch_bounds__(THREADS)
write_rows_multi(const WriteParams p, const int row_vecs, const int row_shift,
                 const int vecs_per_layer) {
  const int layer = blockIdx.y;
  const int base = blockIdx.x * (THREADS * VPT) + threadIdx.x;
  int t[VPT], c[VPT], kv[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = base + j * THREADS;
    int q;
    if (POW2) {
      c[j] = v & (row_vecs - 1);
      q = v >> row_shift;
    } else {
      q = v / row_vecs;
      c[j] = v - q * row_vecs;
    }
    kv[j] = q & 1;
    t[j] = v < vecs_per_layer ? (q >> 1) : -1;
  }
  const char* kin = p.key + (long long)layer * p.key_layer;
  const char* vin = p.value + (long long)layer * p.val_layer;
  char* kout = p.kcache + (long long)layer * p.cache_layer;
  char* vout = p.vcache + (long long)layer * p.cache_layer;

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  SlotRaw raw[VPT];
  Vec r[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (t[j] >= 0) raw[j] = slot_fetch_begin(p, layer, t[j]);
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (t[j] >= 0)
      ld(r[j], (kv[j] ? vin + (long long)t[j] * p.val_tok : kin + (long long)t[j] * p.key_tok) +
                   (long long)c[j] * Vec::kBytes);
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (t[j] >= 0) {
      const long long off = slot_offset(p, slot_fetch_end(p, raw[j], t[j]),
                                        (long long)layer * p.slot_layer + t[j]);
      if (off >= 0) st((kv[j] ? vout : kout) + off + (long long)c[j] * Vec::kBytes, r[j]);
    }
}

// One piece per lane per iteration; a warp-task is 32 consecutive pieces of
// the flattened (layer, token, K|V, piece) index space.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
write_rows_bulk(const WriteParams p, const long long n_items) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t bars[WARPS];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint64_t* bar = &bars[warp];
  unsigned char* buf = smem + ((size_t)warp * 32 + lane) * p.piece_bytes;

  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();

  const long long n_tasks = (n_items + 31) / 32;
  const long long warp_stride = (long long)gridDim.x * WARPS;
  unsigned parity = 0;

  for (long long task = (long long)blockIdx.x * WARPS + warp;
       task < n_tasks; task += warp_stride) {
    const long long item = task * 32 + lane;
    const char* src = nullptr;
    char* dst = nullptr;
    if (item < n_items) {
      // item = ((layer * T + t) * 2 + kv) * pieces_per_row + piece
      const int piece = (int)(item % p.pieces_per_row);
      long long q = item / p.pieces_per_row;
      const int kv = (int)(q & 1);
      q >>= 1;
      const int t = (int)(q % p.num_tokens);
      const int layer = (int)(q / p.num_tokens);
      const long long si = (long long)layer * p.slot_layer + t;
      const long long off =
          slot_offset(p, slot_fetch_end(p, slot_fetch_begin(p, layer, t), t), si);
      if (off >= 0) {
        const long long po = (long long)piece * p.piece_bytes;
        src = (kv ? p.value + (long long)layer * p.val_layer + (long long)t * p.val_tok
                  : p.key + (long long)layer * p.key_layer + (long long)t * p.key_tok) + po;
        dst = (kv ? p.vcache : p.kcache) + (long long)layer * p.cache_layer + off + po;
      }
    }
    const unsigned live = __ballot_sync(0xffffffffu, src != nullptr);
    if (live == 0) continue;
    if (lane == 0) mbar_expect_tx(bar, (unsigned)__popc(live) * (unsigned)p.piece_bytes);
    __syncwarp();
    if (src != nullptr) bulk_g2s(buf, src, (unsigned)p.piece_bytes, bar);
    const unsigned phase = parity;
    parity ^= 1u;
    const bool ok = mbar_wait_bounded(bar, phase);
    if (__any_sync(0xffffffffu, !ok)) {
      // The loads never landed: say so, store nothing, stop taking work.  One
      // more short bounded wait lets copies still in flight land before this
      // CTA's shared memory is released.
      if (lane == 0) report(p.err, kErrWaitTimeout, kWhereWrite, task, 0);
      mbar_wait_bounded(bar, phase, 100000000ull);
      break;
    }
    if (src != nullptr) {
      bulk_s2g(dst, buf, (unsigned)p.piece_bytes);
      bulk_commit();
      bulk_wait_read_all();
    }
    __syncwarp();
  }
  bulk_wait_all();
}

inline int ilog2_exact(long long x) {
  if (x <= 0 || (x & (x - 1)) != 0) return -1;
  int s = 0;
  while ((1ll << s) < x) ++s;
  return s;
}

// Tile choice: about six CTAs per SM (five to eight are resident at 32-48 registers), so a
// decode step - tens of MiB, where ramp-up and tail are a visible part of the run time - is
// one wave of short CTAs; 4 KiB ... 64 KiB of payload per CTA.
inline int auto_tile_bytes(const WriteParams& p, int sms) {
  const long long total = (long long)p.num_layers * p.num_tokens * 2 * p.row_bytes;
  const long long want = total / (6ll * sms);
  int tile = 4096;
  while (tile < 65536 && (long long)tile * 3 / 2 < want) tile *= 2;  // nearest power of two
  return tile;
}

template <class Vec, int VPT>
cudaError_t launch_vec(WriteParams p, int tile_bytes, int sms, cudaStream_t stream) {
  constexpr int THREADS = 256;
  const int row_vecs = p.row_bytes / Vec::kBytes;
  const int row_shift = ilog2_exact(row_vecs);
  if (tile_bytes <= 0) tile_bytes = auto_tile_bytes(p, sms);
  int tok_tile = tile_bytes / (2 * p.row_bytes);
  tok_tile = tok_tile < 1 ? 1 : (tok_tile > kMaxTokTile ? kMaxTokTile : tok_tile);
  if (tok_tile > p.num_tokens) tok_tile = p.num_tokens;
  p.tok_tile = tok_tile;
  p.tiles_per_layer = (p.num_tokens + tok_tile - 1) / tok_tile;
  const long long ctas = (long long)p.tiles_per_layer * p.num_layers;
  if (ctas > 0x7fffffffll) return cudaErrorInvalidConfiguration;
  if (row_shift >= 0)
    write_rows_vec<Vec, THREADS, VPT, true>
        <<<(unsigned)ctas, THREADS, 0, stream>>>(p, row_vecs, row_shift);
  else
    write_rows_vec<Vec, THREADS, VPT, false>
        <<<(unsigned)ctas, THREADS, 0, stream>>>(p, row_vecs, row_shift);
  return cudaGetLastError();
}

template <class Vec>
cudaError_t launch_direct(const WriteParams& p, bool pdl, cudaStream_t stream) {
  constexpr int THREADS = 256;
  const int row_vecs = p.row_bytes / Vec::kBytes;
  const int row_shift = ilog2_exact(row_vecs);
  const long long n_vec = (long long)p.num_layers * p.num_tokens * 2 * row_vecs;
  const long long ctas = (n_vec + THREADS - 1) / THREADS;
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
  if (row_shift >= 0)
    return cudaLaunchKernelEx(&cfg, write_rows_direct<Vec, THREADS, true>, p, row_vecs,
                              row_shift, n_vec);
  return cudaLaunchKernelEx(&cfg, write_rows_direct<Vec, THREADS, false>, p, row_vecs,
                            row_shift, n_vec);
}

// Launch attributes shared by the untiled kernels.
struct PdlConfig {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  PdlConfig(dim3 grid, int threads, bool pdl, cudaStream_t stream) {
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    if (pdl) {
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
    }
  }
};

// kind 5: (K, V) vector pairs, TOK units per thread, one CTA tile per THREADS * TOK units;
// kind 7: the same tiles walked by a persistent grid of `sms * ctas_per_sm` CTAs;
// kind 6: VPT independent vectors per thread.
template <class Vec, int N>
cudaError_t launch_wave(const WriteParams& p, int kind, bool pdl, int sms, int ctas_per_sm,
                        cudaStream_t stream) {
  constexpr int THREADS = 256;
  const int row_vecs = p.row_bytes / Vec::kBytes;
  const int row_shift = ilog2_exact(row_vecs);
  const long long per_layer = (long long)p.num_tokens * row_vecs * (kind == 6 ? 2 : 1);
  if (per_layer > 0x3fffffffll || p.num_layers > 65535) return cudaErrorInvalidConfiguration;
  const int tiles = (int)((per_layer + THREADS * N - 1) / (THREADS * N));
  if (kind == 7) {
    const long long n_tiles = (long long)tiles * p.num_layers;
    if (n_tiles > 0x7fffffffll) return cudaErrorInvalidConfiguration;
    long long grid = (long long)sms * (ctas_per_sm > 0 ? ctas_per_sm : 4);
    if (grid > n_tiles) grid = n_tiles;
    PdlConfig c(dim3((unsigned)grid), THREADS, pdl, stream);
    if (row_shift >= 0)
      return cudaLaunchKernelEx(&c.cfg, write_rows_pair_persistent<Vec, THREADS, N, true>, p,
                                row_vecs, row_shift, (int)per_layer, tiles, (int)n_tiles);
    return cudaLaunchKernelEx(&c.cfg, write_rows_pair_persistent<Vec, THREADS, N, false>, p,
                              row_vecs, row_shift, (int)per_layer, tiles, (int)n_tiles);
  }
  PdlConfig c(dim3((unsigned)tiles, (unsigned)p.num_layers), THREADS, pdl, stream);
  if (kind == 6) {
    if (row_shift >= 0)
      return cudaLaunchKernelEx(&c.cfg, write_rows_multi<Vec, THREADS, N, true>, p, row_vecs,
                                row_shift, (int)per_layer);
    return cudaLaunchKernelEx(&c.cfg, write_rows_multi<Vec, THREADS, N, false>, p, row_vecs,
                              row_shift, (int)per_layer);
  }
  if (row_shift >= 0)
    return cudaLaunchKernelEx(&c.cfg, write_rows_pair<Vec, THREADS, N, true>, p, row_vecs,
                              row_shift, (int)per_layer);
  return cudaLaunchKernelEx(&c.cfg, write_rows_pair<Vec, THREADS, N, false>, p, row_vecs,
                            row_shift, (int)per_layer);
}

template <class Vec>
cudaError_t launch_wave_n(const WriteParams& p, int kind, int n, bool pdl, int sms,
                          int ctas_per_sm, cudaStream_t stream) {
  if (n >= 4) return launch_wave<Vec, 4>(p, kind, pdl, sms, ctas_per_sm, stream);
  if (n >= 2) return launch_wave<Vec, 2>(p, kind, pdl, sms, ctas_per_sm, stream);
  return launch_wave<Vec, 1>(p, kind, pdl, sms, ctas_per_sm, stream);
}

template <class Vec>
cudaError_t launch_vec_vpt(const WriteParams& p, int tile_bytes, int vpt, int sms,
                           cudaStream_t stream) {
  if (vpt == 4) return launch_vec<Vec, 4>(p, tile_bytes, sms, stream);
  if (vpt == 8) return launch_vec<Vec, 8>(p, tile_bytes, sms, stream);
  return launch_vec<Vec, 2>(p, tile_bytes, sms, stream);
}

}  // namespace

const char* write_kernel_name(int variant, long long row_bytes, long long total_bytes) {
  const bool a32 = (row_bytes & 31) == 0;
  if (variant < 0) variant = a32 ? 3 : (total_bytes <= (16ll << 20) ? 4 : 0);
  switch (variant) {
    case 0: case 1: return "write_rows_vec";
    case 2: return "write_rows_bulk";
    case 3: case 4: return "write_rows_direct";
    case 5: return "write_rows_pair";
    case 6: return "write_rows_multi";
    case 7: return "write_rows_pair_persistent";
    default: return "unknown";
  }
}

cudaError_t launch_write(const WriteParams& p_in, int variant, int tile_bytes,
                         int vpt, int sms, bool pdl, cudaStream_t stream) {
  WriteParams p = p_in;
  p.block_shift = ilog2_exact(p.block_size);

  // 32-byte vectors need 32-byte alignment of every address they touch.
  auto aligned32 = [&]() {
    const uintptr_t ptrs = (uintptr_t)p.key | (uintptr_t)p.value |
                           (uintptr_t)p.kcache | (uintptr_t)p.vcache;
    const long long strides = p.key_tok | p.val_tok | p.key_layer | p.val_layer |
                              p.cache_layer | p.block_stride | p.slot_stride |
                              (long long)p.row_bytes;
    return ((ptrs | (uintptr_t)strides) & 31u) == 0;
  };
  const bool a32 = aligned32();
  if (variant < 0) {
    // Built-in choice, from measurement on B200: the untiled 32-byte kernel is the fastest
    // at every size from one layer of a decode step (2 MiB) to a 28-layer prefill chunk
    // (3.5 GiB).  Rows that cannot take 32-byte accesses use the untiled 16-byte kernel for
    // small launches and the tiled one for large launches.
    const long long total = (long long)p.num_layers * p.num_tokens * 2 * p.row_bytes;
    variant = a32 ? 3 : (total <= (16ll << 20) ? 4 : 0);
  }
  if (variant == 1 && !a32) variant = 0;
  if (variant == 3)
    return a32 ? launch_direct<V32>(p, pdl, stream) : launch_direct<V16>(p, pdl, stream);
  if (variant == 4) return launch_direct<V16>(p, pdl, stream);
  if (variant >= 5 && variant <= 7) {
    // tile_bytes doubles as "CTAs per SM" of the persistent form
    return a32 ? launch_wave_n<V32>(p, variant, vpt, pdl, sms, tile_bytes, stream)
               : launch_wave_n<V16>(p, variant, vpt, pdl, sms, tile_bytes, stream);
  }

  if (variant == 2) {
    // piece = the largest power-of-two divisor of the row, capped at 1 KiB
    int piece = 1024;
    while (piece > 16 && (p.row_bytes % piece) != 0) piece >>= 1;
    p.piece_bytes = piece;
    p.pieces_per_row = p.row_bytes / piece;
    const long long n_items =
        (long long)p.num_layers * p.num_tokens * 2 * p.pieces_per_row;
    constexpr int WARPS = 2;
    const size_t smem = (size_t)WARPS * 32 * piece;
    int dev = 0;
    cudaGetDevice(&dev);
    static bool attr_set[64] = {};
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(write_rows_bulk<WARPS>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           WARPS * 32 * 1024);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const long long tasks = (n_items + 31) / 32;
    long long ctas = (tasks + WARPS - 1) / WARPS;
    const long long resident = (long long)sms * ((200 * 1024) / (long long)(smem + 1024));
    if (ctas > resident) ctas = resident;
    if (ctas < 1) ctas = 1;
    write_rows_bulk<WARPS><<<(unsigned)ctas, WARPS * 32, smem, stream>>>(p, n_items);
    return cudaGetLastError();
  }
  if (variant == 1) return launch_vec_vpt<V32>(p, tile_bytes, vpt, sms, stream);
  return launch_vec_vpt<V16>(p, tile_bytes, vpt, sms, stream);
}

}  // namespace lms
