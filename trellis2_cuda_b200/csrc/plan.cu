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
  uint32_t b = k;
#pragma unroll
  for (int v = 1; v < 27; v++) b ^= k >> v;
  return b;
}

// key = group | block (block_bits wide) | mask key (27 bits), most significant first
// halo_from > 0 (split plan, no src): group 1 = rows with a map entry >= halo_from (a row of a peer), group 0 = the rest
__global__ void k_plan_keys(const int* __restrict__ gray, const int* __restrict__ src, const uint32_t* __restrict__ nbr, uint32_t halo_from,
                            i64 m, i64 block_rows, int block_bits,
                            unsigned long long* __restrict__ keys, int* __restrict__ iota, int* __restrict__ group_cnt) {
  i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i >= m) return;
  int grp = 0; i64 nrow = i;
  if (src) { int s = src[i]; grp = s & 7; nrow = s >> 3; }
  else if (halo_from) {
    const uint32_t* e = nbr + i * 27;
#pragma unroll 9
    for (int v = 0; v < 27; v++) { const uint32_t r = __ldg(e + v); grp |= (r != NBR_EMPTY && r >= halo_from) ? 1 : 0; }
  }
  unsigned long long blk = (unsigned long long)(i / block_rows);
  keys[i] = ((unsigned long long)grp << (27 + block_bits)) | (blk << 27) | mask_key((uint32_t)gray[nrow]);
  iota[i] = (int)i;
  if (src || halo_from) atomicAdd(&group_cnt[grp], 1);
}

// one thread: tile offsets of the (up to 8) groups
// bounds[0..2] = {0, first boundary tile, number of tiles}: the interior part of a split plan is tiles
// [bounds[0], bounds[1]), its boundary part [bounds[1], bounds[2]); any other plan is all interior.
__global__ void k_plan_groups(const int* __restrict__ group_cnt, int ngroups, int split, i64 m, int TILE, int* __restrict__ gmeta, int* __restrict__ bounds) {
  // gmeta[g] = first row of group g, gmeta[16+g] = first tile of group g
  int row = 0, tile = 0;
  for (int g = 0; g < ngroups; g++) {
    int c = ngroups == 1 ? (int)m : group_cnt[g];
    gmeta[g] = row; gmeta[16 + g] = tile;
    row += c; tile += (c + TILE - 1) / TILE;
  }
  gmeta[ngroups] = row; gmeta[16 + ngroups] = tile;
  bounds[0] = 0; bounds[1] = split ? gmeta[16 + 1] : tile; bounds[2] = tile;
}

// one warp per tile: extent, weight base, OR of the row masks; also the plan's tap statistics
__global__ void k_plan_tiles(const int* __restrict__ gray, const int* __restrict__ src, const int* __restrict__ order,
                             const int* __restrict__ gmeta, int ngroups, int split, int TILE, const int* __restrict__ ntiles,
                             PlanTile* __restrict__ tiles, unsigned long long* __restrict__ stats) {
  int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= *ntiles) return;
  int g = 0;
  while (g + 1 < ngroups && t >= gmeta[16 + g + 1]) g++;
  int start = gmeta[g] + (t - gmeta[16 + g]) * TILE;
  int rows = min(TILE, gmeta[g + 1] - start);
  uint32_t o = 0; int act = 0;
  for (int j = lane; j < rows; j += 32) {
    int r = order[start + j];
    int nrow = src ? (src[r] >> 3) : r;
    uint32_t gm = (uint32_t)gray[nrow];
    o |= gm; act += __popc(gm);
  }
  o = __reduce_or_sync(0xffffffffu, o);
  act = __reduce_add_sync(0xffffffffu, act);
  if (o == 0) o = 1u << 13;       // no row of the tile has any neighbour: one tap of zero-filled rows still initialises the accumulators
  if (lane == 0) {
    tiles[t] = PlanTile{start, rows, split ? 0 : g, o};      // wbase holds the child slot (the conv multiplies by Co); the two parts of a split plan share one weight set
    atomicAdd(&stats[0], (unsigned long long)rows * __popc(o));
    atomicAdd(&stats[1], (unsigned long long)act);
  }
}

// The neighbour map in tile order: table[t][v][j] = entry of tap v of the j-th row of tile t (for a subdivision plan: of
// that child's parent), 0x80000000 for an absent neighbour and for j past the tile's rows.  One CTA per tile; the rows
// are read as they lie in the caller's map (27 consecutive words) and written tap-major through shared memory.
constexpr uint32_t TABLE_ABSENT = 0x80000000u;
template <int TILE>
__global__ void __launch_bounds__(256) k_plan_table(const uint32_t* __restrict__ nbr, const int* __restrict__ src, const int* __restrict__ order,
                                                    const PlanTile* __restrict__ tiles, const int* __restrict__ ntiles, uint32_t* __restrict__ table) {
  const int t = blockIdx.x;
  if (t >= *ntiles) return;
  __shared__ int s_row[TILE];
  __shared__ uint32_t s_e[27 * (TILE + 1)];
  const PlanTile tile = tiles[t];
  for (int j = threadIdx.x; j < TILE; j += 256) {
    int nr = -1;
    if (j < tile.rows) { const int r = order[tile.start + j]; nr = src ? (src[r] >> 3) : r; }
    s_row[j] = nr;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < TILE * 27; e += 256) {
    const int j = e / 27, v = e - j * 27, nr = s_row[j];
    uint32_t val = TABLE_ABSENT;
    if (nr >= 0) { val = __ldg(nbr + (i64)nr * 27 + v); if (val == NBR_EMPTY) val = TABLE_ABSENT; }
    s_e[v * (TILE + 1) + j] = val;
  }
  __syncthreads();
  uint32_t* out = table + (i64)t * 27 * TILE;
  for (int e = threadIdx.x; e < TILE * 27; e += 256) {
    const int v = e / TILE, j = e - v * TILE;
    out[e] = s_e[v * (TILE + 1) + j];
  }
}

// entries at or above n_in become absent and are reported (status bit 8)
__global__ void k_plan_table_check(uint32_t* __restrict__ table, const int* __restrict__ ntiles, int per_tile, uint32_t n_in, int* status) {
  const i64 n = (i64)*ntiles * per_tile;
  bool bad = false;
  for (i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
    const uint32_t e = table[i];
    if (e != TABLE_ABSENT && e >= n_in) { table[i] = TABLE_ABSENT; bad = true; }
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(status, 256);
}

int plan_table_build(t2sc_ctx* ctx, t2sc_plan* p) {
  if (p->n_out == 0) return T2SC_OK;
  if (p->tile_rows == 128)
    k_plan_table<128><<<(unsigned)p->max_tiles, 256, 0, ctx->stream>>>(p->nbr, p->src, p->order, p->tiles, p->ntiles, p->tnbr);
  else
    k_plan_table<256><<<(unsigned)p->max_tiles, 256, 0, ctx->stream>>>(p->nbr, p->src, p->order, p->tiles, p->ntiles, p->tnbr);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

}  // namespace

// Called by the conv launcher: the table holds no entry at or above n_in.  The check runs once per n_in; when n_in changes
// after a check the table is rebuilt from the caller's map first, because the earlier check may have blanked entries
// that are in range now.
int plan_table_prepare(t2sc_ctx* ctx, t2sc_plan* p, i64 n_in) {
  if (p->table_n_in == n_in || p->n_out == 0) return T2SC_OK;
  if (p->table_n_in >= 0) { int rc = plan_table_build(ctx, p); if (rc != T2SC_OK) return rc; }
  k_plan_table_check<<<2 * ctx->num_sms, 256, 0, ctx->stream>>>(p->tnbr, p->ntiles, 27 * p->tile_rows, (uint32_t)n_in, ctx->status);
  T2_LAUNCHED(ctx);
  p->table_n_in = n_in;
  return T2SC_OK;
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
  unsigned long long *keys = nullptr, *keys2 = nullptr; int *iota = nullptr, *gcnt = nullptr, *gmeta = nullptr; void* tmp = nullptr;
  auto fail = [&](cudaError_t e) {
    t2_free(ctx, keys); t2_free(ctx, keys2); t2_free(ctx, iota); t2_free(ctx, gcnt); t2_free(ctx, gmeta); t2_free(ctx, tmp);
    t2sc_plan_destroy(ctx, p);
    return t2sc_fail(ctx, T2SC_ERR_CUDA, "t2sc_plan_create: %s", cudaGetErrorString(e));
  };
  cudaError_t e;
#define PL(call) do { if ((e = (call)) != cudaSuccess) return fail(e); } while (0)
  PL(t2_alloc(ctx, &p->order, (size_t)m));
  PL(t2_alloc(ctx, &p->tiles, (size_t)p->max_tiles));
  PL(t2_alloc(ctx, &p->tnbr, (size_t)p->max_tiles * 27 * tile_rows));
  PL(t2_alloc(ctx, &p->bounds, 3));
  p->ntiles = p->bounds + 2;
  PL(t2_alloc(ctx, &p->stats, 2));
  PL(cudaMemsetAsync(p->bounds, 0, 3 * sizeof(int), ctx->stream));
  PL(cudaMemsetAsync(p->stats, 0, 2 * sizeof(unsigned long long), ctx->stream));
  if (m > 0) {
    PL(t2_alloc(ctx, &keys, (size_t)m)); PL(t2_alloc(ctx, &keys2, (size_t)m)); PL(t2_alloc(ctx, &iota, (size_t)m));
    PL(t2_alloc(ctx, &gcnt, 8)); PL(t2_alloc(ctx, &gmeta, 32));
    PL(cudaMemsetAsync(gcnt, 0, 8 * sizeof(int), ctx->stream));
    int block_bits = 0;
    while (((m + block_rows - 1) / block_rows) > (1ll << block_bits)) block_bits++;
    k_plan_keys<<<cdiv_i(m, 256), 256, 0, ctx->stream>>>(gray, src, nbr, (uint32_t)halo_from, m, block_rows, block_bits, keys, iota, gcnt);
    ctx->launches++; PL(cudaGetLastError());
    size_t tb = 0;
    int end_bit = 27 + block_bits + (src ? 3 : (split ? 1 : 0));
    // the 3 least significant key bits (centre tap and two face taps) do not change the tiles' masks measurably
    // (active/computed 0.855 -> 0.853) and leaving them out saves a radix pass on maps sorted as one block
    const int begin_bit = 3;
    PL(cub::DeviceRadixSort::SortPairs(nullptr, tb, keys, keys2, iota, p->order, (int)m, begin_bit, end_bit, ctx->stream));
    PL(t2_alloc(ctx, (char**)&tmp, tb));
    PL(cub::DeviceRadixSort::SortPairs(tmp, tb, keys, keys2, iota, p->order, (int)m, begin_bit, end_bit, ctx->stream));
    k_plan_groups<<<1, 1, 0, ctx->stream>>>(gcnt, ngroups, split, m, TILE, gmeta, p->bounds);
    ctx->launches++; PL(cudaGetLastError());
    k_plan_tiles<<<cdiv_i(p->max_tiles * 32, 256), 256, 0, ctx->stream>>>(gray, src, p->order, gmeta, ngroups, split, TILE, p->ntiles, p->tiles, p->stats);
    ctx->launches++; PL(cudaGetLastError());
    if (plan_table_build(ctx, p) != T2SC_OK) return fail(cudaGetLastError());
  }
#undef PL
  t2_free(ctx, keys); t2_free(ctx, keys2); t2_free(ctx, iota); t2_free(ctx, gcnt); t2_free(ctx, gmeta); t2_free(ctx, tmp);
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
  t2_free(ctx, p->order); t2_free(ctx, p->tiles); t2_free(ctx, p->tnbr); t2_free(ctx, p->bounds); t2_free(ctx, p->stats);
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
