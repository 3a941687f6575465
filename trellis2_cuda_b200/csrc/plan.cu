// Execution plan: which output rows share a tile (128 or 256 rows), and which taps each tile has to visit.
//
// The reference schedules by a global stable sort of the gray->binary mask key and per-block tap lists
// (src/spconv.cu:34,47-75 of trellis2-cuda).  Here the sort key is (weight group, run of block_rows caller
// rows, mask key): rows with similar masks still become adjacent, which keeps the union mask of a tile
// close to its rows' own masks, but only inside a run of caller rows, so the gathers of one tile stay
// inside a region that fits the L2.  Weight groups are the 8 child slots of a 2x-subdivision conv.
// A plan made for one rank of a partitioned scene (t2sc_plan_create_split) has two groups of the other kind: rows none
// of whose taps reads a halo row (interior), and rows that do (boundary), the boundary tiles last, so that the interior
// tiles can run while the halo rows are still in flight.
// Everything is built on the device; no host round trip is needed to launch a conv from a plan.
#include "common.cuh"
#include <cub/cub.cuh>

namespace {


// Sort key of a 27-bit tap mask.  The reference sorts by the gray->binary decode of the mask as it stands
// (src/spconv.cu:34).  Here the bits are first reordered so that the taps that are most often absent on a
// surface shell lead: the 8 corner taps, then the 12 edge taps, then the 6 face taps, then the centre.  Rows
// that differ only in common taps then end up adjacent, which shrinks the union mask of a tile (measured on a
// 218k-voxel shell: active/computed taps 0.833 -> 0.855 for 128-row tiles).
__constant__ uint8_t TAP_RANK[27] = {0, 8, 1, 9, 20, 10, 2, 11, 3, 12, 21, 13, 22, 26, 23, 14, 24, 15, 4, 16, 5, 17, 25, 18, 6, 19, 7};
__device__ __forceinline__ uint32_t mask_key(uint32_t g) {
  uint32_t k = 0;
#pragma unroll
  for (int v = 0; v < 27; v++) k |= ((g >> v) & 1u) << (26 - TAP_RANK[v]);
  uint32_t b = k;         // gray -> binary: the XOR of all right shifts, as a prefix scan
  b ^= b >> 16; b ^= b >> 8; b ^= b >> 4; b ^= b >> 2; b ^= b >> 1;
  return b;
}

// key = group | block (block_bits wide) | mask key (27 bits), most significant first, with the `drop` least significant
// mask-key bits left out; K is uint32_t when that fits in 32 bits (half the sort traffic), else unsigned long long.
// halo_from > 0 (split plan, no src): group 1 = rows with a map entry >= halo_from (a row of a peer), group 0 = the rest
template <class K>
__global__ void k_plan_keys(const int* __restrict__ gray, const int* __restrict__ src, const uint32_t* __restrict__ nbr, uint32_t halo_from,
                            i64 m, i64 block_rows, int block_bits, int drop,
                            K* __restrict__ keys, int* __restrict__ iota, int* __restrict__ group_cnt) {
  // group sizes: counted per CTA in shared memory first (millions of rows on eight counters in global memory were the
  // whole time of this kernel)
  __shared__ int s_cnt[8];
  const bool grouped = src || halo_from;
  if (grouped && threadIdx.x < 8) s_cnt[threadIdx.x] = 0;
  if (grouped) __syncthreads();
  i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i < m) {
    int grp = 0; i64 nrow = i;
    if (src) { int s = src[i]; grp = s & 7; nrow = s >> 3; }
    else if (halo_from) {
      const uint32_t* e = nbr + i * 27;
#pragma unroll 9
      for (int v = 0; v < 27; v++) { const uint32_t r = __ldg(e + v); grp |= (r != NBR_EMPTY && r >= halo_from) ? 1 : 0; }
    }
    unsigned long long blk = (unsigned long long)(i / block_rows);
    const unsigned long long k = ((unsigned long long)grp << (27 + block_bits)) | (blk << 27) | mask_key((uint32_t)gray[nrow]);
    keys[i] = (K)(k >> drop);
    iota[i] = (int)i;
    if (grouped) atomicAdd(&s_cnt[grp], 1);
  }
  if (grouped) {
    __syncthreads();
    if (threadIdx.x < 8 && s_cnt[threadIdx.x]) atomicAdd(&group_cnt[threadIdx.x], s_cnt[threadIdx.x]);
  }
}

// The neighbour map in tile order: table[t][v][j] = entry of tap v of the j-th row of tile t (for a subdivision plan: of
// that child's parent), 0x80000000 for an absent neighbour and for j past the tile's rows.  One CTA per tile; the rows
// are read as they lie in the caller's map (27 consecutive words) and written tap-major through shared memory.
// HEADER: the same CTA first works out its tile from the group counts (extent, weight group, OR of the row masks), writes
// the tile descriptor, the plan's tap statistics and (CTA 0) the part bounds {0, first boundary tile, number of tiles}:
// the interior part of a split plan is tiles [bounds[0], bounds[1]), its boundary part [bounds[1], bounds[2]); any other
// plan is all interior.  Without HEADER the descriptors are read back (rebuild of the table alone).
constexpr uint32_t TABLE_ABSENT = 0x80000000u;
template <int TILE, bool HEADER>
__global__ void __launch_bounds__(256) k_plan_tiles_table(const uint32_t* __restrict__ nbr, const int* __restrict__ gray, const int* __restrict__ src,
                                                          const int* __restrict__ order, const int* __restrict__ group_cnt, int ngroups, int split,
                                                          i64 m, PlanTile* __restrict__ tiles, int* __restrict__ bounds,
                                                          unsigned long long* __restrict__ stats, uint32_t* __restrict__ table,
                                                          uint32_t* __restrict__ max_entry, int* __restrict__ hist, int win) {
  const int t = blockIdx.x;
  __shared__ int s_row[TILE];
  __shared__ uint32_t s_e[27 * (TILE + 1)];
  __shared__ uint32_t s_or;
  __shared__ int s_act, s_part;
  PlanTile tile;
  if constexpr (HEADER) {
    // first row / first tile of every group; a group's tiles never mix with another's
    int row = 0, tl = 0, g = 0, start = 0, rows = 0, first_boundary = 0;
    bool mine = false;
    for (int q = 0; q < ngroups; q++) {
      const int c = ngroups == 1 ? (int)m : group_cnt[q];
      const int nt = (c + TILE - 1) / TILE;
      if (q == 1) first_boundary = tl;
      if (!mine && t < tl + nt) { mine = true; g = q; start = row + (t - tl) * TILE; rows = min(TILE, row + c - start); }
      row += c; tl += nt;
    }
    if (t == 0 && threadIdx.x == 0) { bounds[0] = 0; bounds[1] = split ? first_boundary : tl; bounds[2] = tl; }
    if (!mine) return;
    if (threadIdx.x == 0) {       // this tile's bin row in the tap-count histogram: (window of `win` tiles within its part, part)
      const int part = (split && g >= 1) ? 1 : 0;
      s_or = 0; s_act = 0; s_part = (((t - (part ? first_boundary : 0)) / win) * 2 + part) * 32;
    }
    tile = PlanTile{start, rows, split ? 0 : g, 0};      // wbase holds the child slot (the conv multiplies by Co); the two parts of a split plan share one weight set
  } else {
    if (t >= bounds[2]) return;
    tile = tiles[t];
  }
  __syncthreads();
  uint32_t o = 0; int act = 0;
  for (int j = threadIdx.x; j < TILE; j += 256) {
    int nr = -1;
    if (j < tile.rows) {
      const int r = order[tile.start + j]; nr = src ? (src[r] >> 3) : r;
      if constexpr (HEADER) { const uint32_t gm = (uint32_t)gray[nr]; o |= gm; act += __popc(gm); }
    }
    s_row[j] = nr;
  }
  if constexpr (HEADER) {
    o = __reduce_or_sync(0xffffffffu, o); act = __reduce_add_sync(0xffffffffu, act);
    if ((threadIdx.x & 31) == 0) { atomicOr(&s_or, o); atomicAdd(&s_act, act); }
  }
  __syncthreads();
  if constexpr (HEADER) {
    if (threadIdx.x == 0) {
      uint32_t mask = s_or;
      if (mask == 0) mask = 1u << 13;       // no row of the tile has any neighbour: one tap of zero-filled rows still initialises the accumulators
      tile.mask = mask;
      tiles[t] = tile;
      atomicAdd(&stats[0], (unsigned long long)tile.rows * __popc(mask));
      atomicAdd(&stats[1], (unsigned long long)s_act);
      if (hist) atomicAdd(&hist[s_part + __popc(mask)], 1);       // tiles of this part with this many taps (k_plan_perm)
    }
  }
  uint32_t big = 0;         // the largest present entry: lets the bounds check skip its scan when every entry is in range
  // all of a thread's loads are issued before the first of them is used: one load latency per tile, not one per entry
  constexpr int PER = (TILE * 27 + 255) / 256;
  uint32_t val[PER];
#pragma unroll
  for (int k = 0; k < PER; k++) {
    const int e = threadIdx.x + 256 * k;
    val[k] = NBR_EMPTY;
    if (e < TILE * 27) { const int j = e / 27, v = e - j * 27, nr = s_row[j]; if (nr >= 0) val[k] = __ldg(nbr + (i64)nr * 27 + v); }
  }
#pragma unroll
  for (int k = 0; k < PER; k++) {
    const int e = threadIdx.x + 256 * k;
    if (e < TILE * 27) {
      const int j = e / 27, v = e - j * 27;
      if (val[k] == NBR_EMPTY) val[k] = TABLE_ABSENT; else big = max(big, val[k]);
      s_e[v * (TILE + 1) + j] = val[k];
    }
  }
  big = __reduce_max_sync(0xffffffffu, big);
  if ((threadIdx.x & 31) == 0 && big > *(volatile uint32_t*)max_entry) atomicMax(max_entry, big);
  __syncthreads();
  uint32_t* out = table + (i64)t * 27 * TILE;
  for (int e = threadIdx.x; e < TILE * 27; e += 256) {
    const int v = e / TILE, j = e - v * TILE;
    out[e] = s_e[v * (TILE + 1) + j];
  }
}

// perm[position] = tile: the tiles of each part ([b0,b1) and [b1,b2)) by falling tap count, within windows of `win`
// consecutive tiles (the whole part as it is used: windows of a few rounds were tried for plans over large maps, whose tile
// order keeps the gathers L2-local, and did not pay).  hist[(window * 2 + part) * 32 + taps] holds the tile counts
// (k_plan_tiles_table), cursor[] the next free slot of each bin.  Which of two tiles with the same tap count comes first
// is left to the order of the atomics: it changes who computes a tile, never a result.
__global__ void k_plan_perm(const PlanTile* __restrict__ tiles, const int* __restrict__ bounds, const int* __restrict__ hist,
                            int* __restrict__ cursor, int win, int* __restrict__ perm) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= bounds[2]) return;
  const int part = t >= bounds[1] ? 1 : 0, start = part ? bounds[1] : 0;
  const int w = (t - start) / win, bin = (w * 2 + part) * 32;
  const int taps = __popc(tiles[t].mask);
  int before = 0;
  for (int b = 27; b > taps; b--) before += hist[bin + b];
  perm[start + w * win + before + atomicAdd(&cursor[bin + taps], 1)] = t;
}

// entries at or above n_in (the rows of the feature array) become absent and are reported (status bit 8)
__global__ void k_plan_table_check(uint32_t* __restrict__ table, const int* __restrict__ ntiles, int per_tile, uint32_t n_in, int* status,
                                   const uint32_t* __restrict__ max_entry) {
  if (*max_entry < n_in) return;          // the usual case: nothing to blank, nothing to scan
  const i64 n = (i64)*ntiles * per_tile;
  bool bad = false;
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
    const uint32_t e = table[i];
    if (e != TABLE_ABSENT && e >= n_in) { table[i] = TABLE_ABSENT; bad = true; }
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(status, 256);
}

template <bool HEADER>
int plan_tiles_table(t2sc_ctx* ctx, t2sc_plan* p, const int32_t* gray, const int* gcnt, int ngroups, int* hist = nullptr, int win = 1) {
  if (p->n_out == 0) return T2SC_OK;
  if (p->tile_rows == 128)
    k_plan_tiles_table<128, HEADER><<<(unsigned)p->max_tiles, 256, 0, ctx->stream>>>(p->nbr, gray, p->src, p->order, gcnt, ngroups, p->split ? 1 : 0, p->n_out,
                                                                                       p->tiles, p->bounds, p->stats, p->tnbr, (uint32_t*)(p->meta + 11), hist, win);
  else
    k_plan_tiles_table<256, HEADER><<<(unsigned)p->max_tiles, 256, 0, ctx->stream>>>(p->nbr, gray, p->src, p->order, gcnt, ngroups, p->split ? 1 : 0, p->n_out,
                                                                                       p->tiles, p->bounds, p->stats, p->tnbr, (uint32_t*)(p->meta + 11), hist, win);
  T2_LAUNCHED(ctx);
  if (HEADER && hist) {
    const i64 bins = (cdiv_i(p->max_tiles, win) + 1) * 64;
    k_plan_perm<<<(unsigned)cdiv_i(p->max_tiles, 256), 256, 0, ctx->stream>>>(p->tiles, p->bounds, hist, hist + bins, win, p->perm);
    T2_LAUNCHED(ctx);
  }
  return T2SC_OK;
}

}  // namespace

// The table holds no entry at or above n_in: checked once per n_in, by t2sc_plan_check or by the first conv that comes
// with that n_in.  When n_in changes after a check the table is rebuilt from the caller's map first, because the earlier
// check may have blanked entries that are in range now.
int plan_table_prepare(t2sc_ctx* ctx, t2sc_plan* p, i64 n_in) {
  if (p->table_n_in == n_in || p->n_out == 0) return T2SC_OK;
  if (p->table_n_in >= 0) { int rc = plan_tiles_table<false>(ctx, p, nullptr, nullptr, 0); if (rc != T2SC_OK) return rc; }
  k_plan_table_check<<<2 * ctx->num_sms, 256, 0, ctx->stream>>>(p->tnbr, p->ntiles, 27 * p->tile_rows, (uint32_t)n_in, ctx->status, (const uint32_t*)(p->meta + 11));
  T2_LAUNCHED(ctx);
  p->table_n_in = n_in;
  return T2SC_OK;
}

extern "C" int t2sc_plan_check(t2sc_ctx* ctx, t2sc_plan* p, int64_t n_in) {
  T2_REQ(ctx, ctx && p, "null context or plan");
  T2_REQ(ctx, n_in >= p->n_rows && n_in < (1ll << 31), "n_in=%lld for a map over %lld rows", (long long)n_in, (long long)p->n_rows);
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  return plan_table_prepare(ctx, p, n_in);
}

static int plan_create(t2sc_ctx* ctx, const uint32_t* nbr, const int32_t* gray, int64_t n_rows,
                       const int32_t* src, int64_t m, int64_t halo_from, int64_t block_rows, int tile_rows, t2sc_plan** out) {
  T2_REQ(ctx, ctx && out, "null context or out");
  *out = nullptr;
  T2_REQ(ctx, n_rows >= 0 && m >= 0 && m < (1ll << 30) && n_rows < (1ll << 30), "n_rows=%lld m=%lld", (long long)n_rows, (long long)m);
  if (!src) T2_REQ(ctx, m == n_rows, "a submanifold plan has one output row per neighbour row (m=%lld n_rows=%lld)", (long long)m, (long long)n_rows);
  T2_REQ(ctx, m == 0 || (nbr && gray), "null tensor");
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  if (block_rows <= 0) block_rows = m <= (1 << 18) ? (m > 0 ? m : 1) : (1 << 16);   // small maps: one global sort; large: keep gathers L2-local
  if (tile_rows == 0) tile_rows = 128;
  T2_REQ(ctx, tile_rows == 128 || tile_rows == 256, "tile_rows=%d", tile_rows);
  const int TILE = tile_rows;
  T2_REQ(ctx, (m + block_rows - 1) / block_rows < (1ll << 23), "block_rows=%lld too small for m=%lld", (long long)block_rows, (long long)m);
  t2sc_plan* p = new t2sc_plan();
  p->n_out = m; p->n_rows = n_rows; p->n_in = n_rows; p->nbr = nbr; p->src = src; p->tile_rows = tile_rows;
  const int split = halo_from > 0 ? 1 : 0;
  p->split = split != 0;
  int ngroups = src ? 8 : (split ? 2 : 1);
  p->max_tiles = cdiv_i(m, TILE) + (src ? 8 : (split ? 2 : 0));
  Scratch scratch(ctx);            // sort buffers: back to the pool on every path out
  auto fail = [&](cudaError_t e) {
    t2sc_plan_destroy(ctx, p);
    return t2sc_fail(ctx, T2SC_ERR_CUDA, "t2sc_plan_create: %s", cudaGetErrorString(e));
  };
  cudaError_t e;
#define PL(call) do { if ((e = (call)) != cudaSuccess) return fail(e); } while (0)
  PL(t2_alloc(ctx, &p->order, (size_t)m));
  PL(t2_alloc(ctx, &p->tiles, (size_t)p->max_tiles));
  PL(t2_alloc(ctx, &p->perm, (size_t)p->max_tiles));
  PL(t2_alloc(ctx, &p->tnbr, (size_t)p->max_tiles * 27 * tile_rows));
  // one small block, one memset: group counts [0..8), part bounds [8..11), largest map entry [11], tap statistics (two u64) from int 12
  PL(t2_alloc(ctx, &p->meta, 16));
  p->bounds = p->meta + 8; p->ntiles = p->bounds + 2; p->stats = (unsigned long long*)(p->meta + 12);
  PL(cudaMemsetAsync(p->meta, 0, 16 * sizeof(int), ctx->stream));
  if (m > 0) {
    int block_bits = 0;
    while (((m + block_rows - 1) / block_rows) > (1ll << block_bits)) block_bits++;
    // the 3 least significant key bits (centre tap and two face taps) do not change the tiles' masks measurably
    // (active/computed 0.855 -> 0.853) and leaving them out saves a radix pass on maps sorted as one block
    // Up to five more go when that brings the key down to 32 bits (a large subdivision plan: 3 group bits + 6 block bits).
    int drop = 3;
    while (27 + block_bits + (src ? 3 : (split ? 1 : 0)) - drop > 32 && drop < 8) drop++;
    const int key_bits = 27 + block_bits + (src ? 3 : (split ? 1 : 0)) - drop;
    const bool narrow = key_bits <= 32;
    const size_t ksz = narrow ? sizeof(uint32_t) : sizeof(unsigned long long);
    char* buf = nullptr; char* tmp = nullptr; size_t tb = 0;
    const size_t koff = ((size_t)m * ksz + 255) & ~(size_t)255;
    PL(scratch.get(&buf, 2 * koff + (size_t)m * sizeof(int)));
    int* iota = (int*)(buf + 2 * koff);
    if (narrow) {
      uint32_t *keys = (uint32_t*)buf, *keys2 = (uint32_t*)(buf + koff);
      k_plan_keys<uint32_t><<<cdiv_i(m, 256), 256, 0, ctx->stream>>>(gray, src, nbr, (uint32_t)halo_from, m, block_rows, block_bits, drop, keys, iota, p->meta);
      ctx->launches++; PL(cudaGetLastError());
      PL(cub::DeviceRadixSort::SortPairs(nullptr, tb, keys, keys2, iota, p->order, (int)m, 0, key_bits, ctx->stream));
      PL(scratch.get(&tmp, tb));
      PL(cub::DeviceRadixSort::SortPairs(tmp, tb, keys, keys2, iota, p->order, (int)m, 0, key_bits, ctx->stream));
    } else {
      unsigned long long *keys = (unsigned long long*)buf, *keys2 = (unsigned long long*)(buf + koff);
      k_plan_keys<unsigned long long><<<cdiv_i(m, 256), 256, 0, ctx->stream>>>(gray, src, nbr, (uint32_t)halo_from, m, block_rows, block_bits, drop, keys, iota, p->meta);
      ctx->launches++; PL(cudaGetLastError());
      PL(cub::DeviceRadixSort::SortPairs(nullptr, tb, keys, keys2, iota, p->order, (int)m, 0, key_bits, ctx->stream));
      PL(scratch.get(&tmp, tb));
      PL(cub::DeviceRadixSort::SortPairs(tmp, tb, keys, keys2, iota, p->order, (int)m, 0, key_bits, ctx->stream));
    }
    // The order the conv's CTAs take the tiles in (k_plan_perm): by tap count when the rows were sorted as one block; plan
    // order when they were sorted inside runs (large maps: the runs keep concurrently running tiles L2-local).
    p->balanced = block_rows >= m;
    const int win = 1 << 30;
    const i64 bins = 2 * 64;
    int* hist = nullptr;
    if (p->balanced) {
      PL(scratch.get(&hist, (size_t)(2 * bins)));
      PL(cudaMemsetAsync(hist, 0, (size_t)(2 * bins) * sizeof(int), ctx->stream));
    }
    if (plan_tiles_table<true>(ctx, p, gray, p->meta, ngroups, hist, win) != T2SC_OK) return fail(cudaGetLastError());
  }
#undef PL
  *out = p;
  return T2SC_OK;
}

extern "C" int t2sc_plan_create(t2sc_ctx* ctx, const uint32_t* nbr, const int32_t* gray, int64_t n_rows,
                                const int32_t* src, int64_t m, int64_t block_rows, int tile_rows, t2sc_plan** out) {
  return plan_create(ctx, nbr, gray, n_rows, src, m, 0, block_rows, tile_rows, out);
}

extern "C" int t2sc_plan_create_split(t2sc_ctx* ctx, const uint32_t* nbr, const int32_t* gray, int64_t n_rows, int64_t n_own,
                                      int64_t block_rows, int tile_rows, t2sc_plan** out) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n_own > 0 && n_own < (1ll << 31), "n_own=%lld", (long long)n_own);
  return plan_create(ctx, nbr, gray, n_rows, nullptr, n_rows, n_own, block_rows, tile_rows, out);
}

extern "C" int t2sc_plan_parts(t2sc_ctx* ctx, t2sc_plan* p, int64_t* interior_tiles, int64_t* boundary_tiles) {
  T2_REQ(ctx, ctx && p, "null context or plan");
  int b[3] = {0, 0, 0};
  T2_CUDA(ctx, cudaMemcpyAsync(b, p->bounds, sizeof(b), cudaMemcpyDeviceToHost, ctx->stream));
  T2_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (interior_tiles) *interior_tiles = b[1] - b[0];
  if (boundary_tiles) *boundary_tiles = b[2] - b[1];
  return T2SC_OK;
}

extern "C" int t2sc_plan_set_input_rows(t2sc_ctx* ctx, t2sc_plan* p, int64_t n_in) {
  T2_REQ(ctx, ctx && p, "null context or plan");
  T2_REQ(ctx, n_in >= p->n_rows && n_in < (1ll << 31), "n_in=%lld for a map over %lld rows", (long long)n_in, (long long)p->n_rows);
  p->n_in = n_in;
  return T2SC_OK;
}

extern "C" int t2sc_plan_destroy(t2sc_ctx* ctx, t2sc_plan* p) {
  if (!p) return T2SC_OK;
  T2_REQ(ctx, ctx != nullptr, "null context");
  cudaSetDevice(ctx->device);
  t2_free(ctx, p->order); t2_free(ctx, p->tiles); t2_free(ctx, p->perm); t2_free(ctx, p->tnbr); t2_free(ctx, p->meta);
  delete p;
  return T2SC_OK;
}

extern "C" int t2sc_plan_stats(t2sc_ctx* ctx, t2sc_plan* p, int64_t* tiles, int64_t* computed_taps, int64_t* active_taps) {
  T2_REQ(ctx, ctx && p, "null context or plan");
  int nt = 0; unsigned long long st[2] = {0, 0};
  T2_CUDA(ctx, cudaMemcpyAsync(&nt, p->ntiles, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  T2_CUDA(ctx, cudaMemcpyAsync(st, p->stats, sizeof(st), cudaMemcpyDeviceToHost, ctx->stream));
  T2_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (tiles) *tiles = nt;
  if (computed_taps) *computed_taps = (int64_t)st[0];
  if (active_taps) *active_taps = (int64_t)st[1];
  return T2SC_OK;
}

extern "C" int t2sc_plan_order(t2sc_ctx* ctx, t2sc_plan* p, int32_t* order_out) {
  T2_REQ(ctx, ctx && p && (order_out || p->n_out == 0), "null argument");
  if (p->n_out) T2_CUDA(ctx, cudaMemcpyAsync(order_out, p->order, (size_t)p->n_out * sizeof(int), cudaMemcpyDeviceToDevice, ctx->stream));
  return T2SC_OK;
}
