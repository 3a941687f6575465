// Integer half of the path: voxel hash table, 27-tap neighbour maps, the reference's row order and
// per-block tap lists, 2x subdivision maps, row gather and the up-block skip add.
//
// Results are defined by the reference (src/spconv.cu:13-75, src/sdec.cu:21-57 of trellis2-cuda) and are
// bit-exact with it; the layout of the work is not.  The pool-backed builders hash 2x2x2 BRICKS of voxels
// (8 probes per row instead of 27, k_brick_*); the allocation-free builder keeps the per-voxel table with one
// 16-byte {key, row} slot per probe and one thread per (row, tap) entry (k_hash_insert / k_neighbors).
// Nothing is built on the host.
#include "common.cuh"
#include <cub/cub.cuh>

namespace {

struct __align__(16) Slot { unsigned long long key; uint32_t val; uint32_t pad; };
static constexpr unsigned long long KEY_EMPTY = ~0ull;

__device__ __forceinline__ uint32_t mix32(unsigned long long k) {   // src/spconv.cu:13
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; return (uint32_t)k;
}
__device__ __forceinline__ unsigned long long pack_key(int b, int x, int y, int z, int W, int H, int D) {  // src/spconv.cu:16
  return (((unsigned long long)b * W + x) * H + y) * D + z;
}

__global__ void k_hash_insert(const int4* __restrict__ coords, int n, int W, int H, int D, Slot* table, uint32_t mask) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int4 q = coords[i];
  unsigned long long k = pack_key(q.x, q.y, q.z, q.w, W, H, D);
  // at most `mask + 1` probes: the table holds >= 2n slots, so this bound is never reached on valid input
  for (uint32_t s = mix32(k) & mask, it = 0; it <= mask; s = (s + 1) & mask, ++it) {
    unsigned long long prev = atomicCAS(&table[s].key, KEY_EMPTY, k);
    if (prev == KEY_EMPTY || prev == k) { atomicMin(&table[s].val, (uint32_t)i); return; }  // duplicates: lowest row wins
  }
}

constexpr int NB_ROWS = 32;                 // rows per CTA of the neighbour kernel
constexpr int NB_THREADS = 288;             // 32 rows * 27 taps = 864 entries = 3 per thread
__global__ void __launch_bounds__(NB_THREADS) k_neighbors(const int4* __restrict__ coords, int n, int W, int H, int D,
                                                          const Slot* __restrict__ table, uint32_t mask,
                                                          uint32_t* __restrict__ nbr, int* __restrict__ gray, int* __restrict__ bin) {
  __shared__ uint32_t s_mask[NB_ROWS];
  i64 row0 = (i64)blockIdx.x * NB_ROWS;
  if (threadIdx.x < NB_ROWS) s_mask[threadIdx.x] = 0;
  __syncthreads();
  int rows = (int)min((i64)NB_ROWS, (i64)n - row0);
#pragma unroll
  for (int e = threadIdx.x; e < NB_ROWS * 27; e += NB_THREADS) {
    int lr = e / 27, v = e - lr * 27;
    if (lr >= rows) break;
    int4 q = coords[row0 + lr];
    int x = q.y + v / 9 - 1, y = q.z + (v / 3) % 3 - 1, z = q.w + v % 3 - 1;   // src/spconv.cu:27
    uint32_t r = NBR_EMPTY;
    if (x >= 0 && x < W && y >= 0 && y < H && z >= 0 && z < D) {
      unsigned long long k = pack_key(q.x, x, y, z, W, H, D);
      for (uint32_t s = mix32(k) & mask, it = 0; it <= mask; s = (s + 1) & mask, ++it) {
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(table + s));
        unsigned long long sk = ((unsigned long long)raw.y << 32) | raw.x;
        if (sk == KEY_EMPTY) break;
        if (sk == k) { r = raw.z; break; }
      }
    }
    nbr[(row0 + lr) * 27 + v] = r;
    if (r != NBR_EMPTY) atomicOr(&s_mask[lr], 1u << v);
  }
  __syncthreads();
  if (threadIdx.x < rows) {
    uint32_t g = s_mask[threadIdx.x], b = g;
#pragma unroll
    for (int v = 1; v < 27; v++) b ^= g >> v;       // gray -> binary, src/spconv.cu:34
    gray[row0 + threadIdx.x] = (int)g;
    if (bin) bin[row0 + threadIdx.x] = (int)b;
  }
}

// ---- brick table: one slot per occupied 2x2x2 block of voxels, holding the 8 row indices of its cells.
// The 27 neighbours of a voxel always lie in exactly 8 bricks (2 per axis), so a row costs 8 key probes and 8
// 32-byte value reads instead of 27 probes; the value reads of one row are shared by up to 8 taps each.
struct __align__(16) BrickVals { uint32_t v[8]; };

__device__ __forceinline__ unsigned long long brick_key(int b, int bx, int by, int bz, int Wb, int Hb, int Db) {
  return (((unsigned long long)b * Wb + bx) * Hb + by) * Db + bz;
}

__global__ void k_brick_insert(const int4* __restrict__ coords, int n, int Wb, int Hb, int Db, unsigned long long* keys,
                               BrickVals* vals, uint32_t mask) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int4 q = coords[i];
  unsigned long long k = brick_key(q.x, q.y >> 1, q.z >> 1, q.w >> 1, Wb, Hb, Db);
  int sub = (q.y & 1) | ((q.z & 1) << 1) | ((q.w & 1) << 2);
  for (uint32_t s = mix32(k) & mask, it = 0; it <= mask; s = (s + 1) & mask, ++it) {
    unsigned long long prev = atomicCAS(&keys[s], KEY_EMPTY, k);
    if (prev == KEY_EMPTY || prev == k) { atomicMin(&vals[s].v[sub], (uint32_t)i); return; }   // duplicates: lowest row wins
  }
}

// 8 threads per row, one per brick of the row's 3x3x3 neighbourhood; 32 rows per 256-thread CTA.
__global__ void __launch_bounds__(256) k_brick_neighbors(const int4* __restrict__ coords, int n, int W, int H, int D, int Wb, int Hb, int Db,
                                                         const unsigned long long* __restrict__ keys, const BrickVals* __restrict__ vals,
                                                         uint32_t mask, uint32_t* __restrict__ nbr, int* __restrict__ gray, int* __restrict__ bin) {
  const i64 row = (i64)blockIdx.x * 32 + (threadIdx.x >> 3);
  const int t = threadIdx.x & 7;                    // brick (sx, sy, sz) = bits 0, 1, 2 of t
  const bool live = row < n;
  uint32_t g = 0;
  if (live) {
    const int4 q = coords[row];
    const int x = q.y, y = q.z, z = q.w;
    // along one axis the offsets -1, 0, +1 fall into brick "lo" = (c-1)>>1 or "hi" = lo + 1: odd c -> {lo, lo, hi}, even c -> {lo, hi, hi}
    const int sx = t & 1, sy = (t >> 1) & 1, sz = t >> 2;
    const int bx = ((x - 1) >> 1) + sx, by = ((y - 1) >> 1) + sy, bz = ((z - 1) >> 1) + sz;
    BrickVals bv;
#pragma unroll
    for (int e = 0; e < 8; e++) bv.v[e] = NBR_EMPTY;
    if (bx >= 0 && by >= 0 && bz >= 0 && bx < Wb && by < Hb && bz < Db) {
      const unsigned long long k = brick_key(q.x, bx, by, bz, Wb, Hb, Db);
      for (uint32_t s = mix32(k) & mask, it = 0; it <= mask; s = (s + 1) & mask, ++it) {
        const unsigned long long sk = __ldg(keys + s);
        if (sk == KEY_EMPTY) break;
        if (sk == k) {
          const uint4 a = __ldg(reinterpret_cast<const uint4*>(vals + s)), b = __ldg(reinterpret_cast<const uint4*>(vals + s) + 1);
          bv.v[0] = a.x; bv.v[1] = a.y; bv.v[2] = a.z; bv.v[3] = a.w; bv.v[4] = b.x; bv.v[5] = b.y; bv.v[6] = b.z; bv.v[7] = b.w;
          break;
        }
      }
    }
    // The brick's 8 cells, by their fixed position e = (ex, ey, ez) in the brick: cell (2 bx + ex, 2 by + ey, 2 bz + ez) is the
    // row's tap (dx, dy, dz) when every offset is in -1 .. 1.  Every tap of the row lies in exactly one of the 8 bricks, so
    // the 8 threads write the row's 27 entries between them, and the cell's value is read with a constant index.  What
    // depends on one axis only is worked out once per axis: is the offset a tap offset (and the cell inside the grid), and
    // its share of the tap number v = (dx + 1) * 9 + (dy + 1) * 3 + (dz + 1) (src/spconv.cu:27).
    bool okx[2], oky[2], okz[2], inx[2], iny[2], inz[2]; int vx[2], vy[2], vz[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int cx = 2 * bx + h, cy = 2 * by + h, cz = 2 * bz + h;
      okx[h] = (unsigned)(cx - x + 1) <= 2u; vx[h] = (cx - x + 1) * 9; inx[h] = (unsigned)cx < (unsigned)W;
      oky[h] = (unsigned)(cy - y + 1) <= 2u; vy[h] = (cy - y + 1) * 3; iny[h] = (unsigned)cy < (unsigned)H;
      okz[h] = (unsigned)(cz - z + 1) <= 2u; vz[h] = cz - z + 1;       inz[h] = (unsigned)cz < (unsigned)D;
    }
    uint32_t* const out = nbr + row * 27;
#pragma unroll
    for (int e = 0; e < 8; e++) {
      const int ex = e & 1, ey = (e >> 1) & 1, ez = e >> 2;
      if (okx[ex] && oky[ey] && okz[ez]) {
        const int v = vx[ex] + vy[ey] + vz[ez];
        const uint32_t r = inx[ex] && iny[ey] && inz[ez] ? bv.v[e] : NBR_EMPTY;      // a neighbour outside the grid is absent (src/spconv.cu:28)
        out[v] = r;
        if (r != NBR_EMPTY) g |= 1u << v;
      }
    }
  }
  g |= __shfl_xor_sync(0xffffffffu, g, 1); g |= __shfl_xor_sync(0xffffffffu, g, 2); g |= __shfl_xor_sync(0xffffffffu, g, 4);
  if (live && t == 0) {
    uint32_t b = g;                                 // gray -> binary (src/spconv.cu:34): XOR of all right shifts, as a prefix scan
    b ^= b >> 16; b ^= b >> 8; b ^= b >> 4; b ^= b >> 2; b ^= b >> 1;
    gray[row] = (int)g;
    if (bin) bin[row] = (int)b;
  }
}

// one thread per query coordinate: the row of the voxel that sits there, or NBR_EMPTY
__global__ void k_brick_lookup(const int4* __restrict__ queries, i64 m, int W, int H, int D, int Wb, int Hb, int Db,
                               const unsigned long long* __restrict__ keys, const BrickVals* __restrict__ vals, uint32_t mask,
                               uint32_t* __restrict__ rows) {
  const i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i >= m) return;
  const int4 q = queries[i];
  uint32_t r = NBR_EMPTY;
  if (q.x >= 0 && q.y >= 0 && q.y < W && q.z >= 0 && q.z < H && q.w >= 0 && q.w < D) {
    const unsigned long long k = brick_key(q.x, q.y >> 1, q.z >> 1, q.w >> 1, Wb, Hb, Db);
    for (uint32_t s = mix32(k) & mask, it = 0; it <= mask; s = (s + 1) & mask, ++it) {
      const unsigned long long sk = __ldg(keys + s);
      if (sk == KEY_EMPTY) break;
      if (sk == k) { r = __ldg(&vals[s].v[(q.y & 1) | ((q.z & 1) << 1) | ((q.w & 1) << 2)]); break; }
    }
  }
  rows[i] = r;
}

__global__ void k_iota(int* p, int n) { int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) p[i] = i; }

// ---- valid(B1): one warp per block of B1 sorted rows
__global__ void k_block_or(const int* __restrict__ gray, const int* __restrict__ sorted, int n, int B1, int nb,
                           int* __restrict__ code, int* __restrict__ cnt) {
  int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (b >= nb) return;
  int o = 0;
  i64 lo = (i64)b * B1, hi = min((i64)n, lo + B1);
  for (i64 i = lo + lane; i < hi; i += 32) o |= gray[sorted[i]];
  o = __reduce_or_sync(0xffffffffu, (unsigned)o);
  if (lane == 0) { code[b] = o; cnt[b] = __popc(o); }
}
__global__ void k_block_list(const int* __restrict__ code, const int* __restrict__ seg, int nb, int* __restrict__ list) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  int c = code[b], s = seg[b];
  while (c) { list[s++] = __ffs(c) - 1; c &= c - 1; }
}

// ---- 2x subdivision
template <class T> __device__ __forceinline__ bool sub_keep(const T* sub, i64 e);
template <> __device__ __forceinline__ bool sub_keep<__half>(const __half* s, i64 e) { return __half2float(s[e]) > 0.f; }
template <> __device__ __forceinline__ bool sub_keep<__nv_bfloat16>(const __nv_bfloat16* s, i64 e) { return __bfloat162float(s[e]) > 0.f; }
template <> __device__ __forceinline__ bool sub_keep<uint8_t>(const uint8_t* s, i64 e) { return s[e] != 0; }

template <class T> __global__ void k_c2s_count(const T* __restrict__ sub, int n, int* __restrict__ cnt) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int c = 0;
#pragma unroll
  for (int s = 0; s < 8; s++) c += sub_keep<T>(sub, (i64)i * 8 + s);
  cnt[i] = c;
}
template <class T> __global__ void k_c2s_emit(const T* __restrict__ sub, const int4* __restrict__ co, const int* __restrict__ off,
                                              int n, int4* __restrict__ nco, int* __restrict__ src) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int r = off[i]; int4 q = co[i];
#pragma unroll
  for (int s = 0; s < 8; s++)
    if (sub_keep<T>(sub, (i64)i * 8 + s)) {
      nco[r] = make_int4(q.x, q.y * 2 + (s & 1), q.z * 2 + (s >> 1 & 1), q.w * 2 + (s >> 2 & 1));
      src[r++] = i * 8 + s;
    }
}

// ---- row gather / skip add, 16 bytes per thread
__global__ void k_gather_rows16(const uint4* __restrict__ x, const int* __restrict__ src, i64 m, int vec_per_row, uint4* __restrict__ y) {
  i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i >= m * vec_per_row) return;
  i64 r = i / vec_per_row; int c = (int)(i - r * vec_per_row);
  y[i] = __ldg(x + (i64)src[r] * vec_per_row + c);
}
template <class T> __global__ void k_add_skip(T* __restrict__ h, const T* __restrict__ x, const int* __restrict__ src, i64 m,
                                              int Co, int Cin, int rep) {
  i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i >= m * Co) return;
  i64 r = i / Co; int c = (int)(i - r * Co), p = src[r] >> 3, s = src[r] & 7, Cs = Cin / 8;
  h[i] = from_f<T>(to_f<T>(h[i]) + to_f<T>(x[(i64)p * Cin + s * Cs + c / rep]));
}

// 8 output channels per thread (16-byte accesses of h for the 16-bit types); Co % 8 == 0
template <class T> __global__ void k_add_skip8(T* __restrict__ h, const T* __restrict__ x, const int* __restrict__ src, i64 nvec,
                                               int vpr, int Cin, int rep) {
  const i64 i = blockIdx.x * (i64)blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const i64 r = nvec < (1ll << 31) ? (i64)((unsigned)i / (unsigned)vpr) : i / vpr;
  const int c0 = (int)(i - r * vpr) * 8, sv = src[r], Cs = Cin / 8;
  const T* xs = x + (i64)(sv >> 3) * Cin + (sv & 7) * Cs;
  T* hp = h + i * 8;
  T v[8];
  if constexpr (sizeof(T) == 2) *(uint4*)v = *(const uint4*)hp;
  else { *(float4*)v = *(const float4*)hp; *((float4*)v + 1) = *((const float4*)hp + 1); }
#pragma unroll
  for (int e = 0; e < 8; e++) v[e] = from_f<T>(to_f<T>(v[e]) + to_f<T>(xs[(c0 + e) / rep]));
  if constexpr (sizeof(T) == 2) *(uint4*)hp = *(const uint4*)v;
  else { *(float4*)hp = *(const float4*)v; *((float4*)hp + 1) = *((const float4*)v + 1); }
}

template <class T> void add_skip_pick(cudaStream_t st, void* h, const void* x, const int32_t* src, i64 m, int Co, int Cin, int rep) {
  if (Co % 8 == 0 && (uintptr_t)h % 16 == 0) {
    const i64 nvec = m * (Co / 8);
    k_add_skip8<T><<<cdiv_i(nvec, 256), 256, 0, st>>>((T*)h, (const T*)x, src, nvec, Co / 8, Cin, rep);
  } else {
    k_add_skip<T><<<cdiv_i(m * Co, 256), 256, 0, st>>>((T*)h, (const T*)x, src, m, Co, Cin, rep);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------ entry points
extern "C" int t2sc_build_neighbors(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                                    uint32_t* nbr, int32_t* gray, int32_t* sorted) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && n < (1ll << 30), "n=%lld", (long long)n);
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, coords && nbr && gray, "null tensor");
  T2_REQ(ctx, (uintptr_t)coords % 16 == 0, "coords must be 16-byte aligned");
  T2_REQ(ctx, W > 0 && H > 0 && D > 0, "grid extent %d %d %d", W, H, D);
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  uint32_t cap = 1; while (cap < 2u * (uint32_t)n) cap <<= 1;            // src/spconv.cu:40
  Scratch scratch(ctx);            // returned to the pool on every path out of this function
  int* bin = nullptr;
  char* table = nullptr;           // keys [cap] then brick rows [cap]: one allocation, one memset
  const int Wb = (W + 1) / 2, Hb = (H + 1) / 2, Db = (D + 1) / 2;
  const size_t table_bytes = (size_t)cap * (sizeof(unsigned long long) + sizeof(BrickVals));
  T2_CUDA(ctx, scratch.get(&table, table_bytes));
  unsigned long long* bkeys = (unsigned long long*)table; BrickVals* bvals = (BrickVals*)(table + (size_t)cap * sizeof(unsigned long long));
  T2_CUDA(ctx, cudaMemsetAsync(table, 0xff, table_bytes, ctx->stream));
  k_brick_insert<<<cdiv_i(n, 256), 256, 0, ctx->stream>>>((const int4*)coords, (int)n, Wb, Hb, Db, bkeys, bvals, cap - 1);
  T2_LAUNCHED(ctx);
  if (sorted) T2_CUDA(ctx, scratch.get(&bin, (size_t)n));
  k_brick_neighbors<<<cdiv_i(n, 32), 256, 0, ctx->stream>>>((const int4*)coords, (int)n, W, H, D, Wb, Hb, Db, bkeys, bvals, cap - 1, nbr, gray, bin);
  T2_LAUNCHED(ctx);
  if (sorted) {
    int *bs = nullptr, *iota = nullptr; char* tmp = nullptr; size_t tb = 0;
    T2_CUDA(ctx, scratch.get(&bs, (size_t)n));
    T2_CUDA(ctx, scratch.get(&iota, (size_t)n));
    k_iota<<<cdiv_i(n, 256), 256, 0, ctx->stream>>>(iota, (int)n);
    T2_LAUNCHED(ctx);
    // the key has 27 significant bits; radix sort is stable, so ties keep ascending row order
    T2_CUDA(ctx, cub::DeviceRadixSort::SortPairs(nullptr, tb, bin, bs, iota, sorted, (int)n, 0, 27, ctx->stream));
    T2_CUDA(ctx, scratch.get(&tmp, tb));
    T2_CUDA(ctx, cub::DeviceRadixSort::SortPairs(tmp, tb, bin, bs, iota, sorted, (int)n, 0, 27, ctx->stream));
  }
  return T2SC_OK;
}

extern "C" int t2sc_valid_taps(t2sc_ctx* ctx, const int32_t* gray, const int32_t* sorted, int64_t n, int B1,
                               int32_t* seg, int32_t* list, int64_t* total_host) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && B1 > 0, "n=%lld B1=%d", (long long)n, B1);
  if (total_host) *total_host = 0;
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, gray && sorted && seg && list, "null tensor");
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  int nb = cdiv_i(n, B1);
  Scratch scratch(ctx);
  int* code = nullptr; char* tmp = nullptr; size_t tb = 0;
  T2_CUDA(ctx, scratch.get(&code, (size_t)nb));
  T2_CUDA(ctx, cudaMemsetAsync(seg, 0, sizeof(int), ctx->stream));
  k_block_or<<<cdiv_i((i64)nb * 32, 256), 256, 0, ctx->stream>>>(gray, sorted, (int)n, B1, nb, code, seg + 1);
  T2_LAUNCHED(ctx);
  T2_CUDA(ctx, cub::DeviceScan::InclusiveSum(nullptr, tb, seg + 1, seg + 1, nb, ctx->stream));
  T2_CUDA(ctx, scratch.get(&tmp, tb));
  T2_CUDA(ctx, cub::DeviceScan::InclusiveSum(tmp, tb, seg + 1, seg + 1, nb, ctx->stream));
  k_block_list<<<cdiv_i(nb, 256), 256, 0, ctx->stream>>>(code, seg, nb, list);
  T2_LAUNCHED(ctx);
  if (total_host) {
    int tot = 0;
    T2_CUDA(ctx, cudaMemcpyAsync(&tot, seg + nb, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    T2_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *total_host = tot;
  }
  return T2SC_OK;
}

extern "C" int t2sc_subdivide_count(t2sc_ctx* ctx, const void* sub, int sub_dtype, int64_t n, int32_t* off, int64_t* m_host) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && n < (1ll << 28), "n=%lld", (long long)n);
  T2_REQ(ctx, sub_dtype == T2SC_F16 || sub_dtype == T2SC_BF16 || sub_dtype == T2SC_U8, "sub dtype %d", sub_dtype);
  if (m_host) *m_host = 0;
  T2_REQ(ctx, off != nullptr, "null off");
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  T2_CUDA(ctx, cudaMemsetAsync(off, 0, sizeof(int), ctx->stream));
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, sub != nullptr, "null sub");
  Scratch scratch(ctx);
  int* cnt = nullptr; char* tmp = nullptr; size_t tb = 0;
  T2_CUDA(ctx, scratch.get(&cnt, (size_t)n));
  int g = cdiv_i(n, 256);
  if (sub_dtype == T2SC_F16) k_c2s_count<__half><<<g, 256, 0, ctx->stream>>>((const __half*)sub, (int)n, cnt);
  else if (sub_dtype == T2SC_BF16) k_c2s_count<__nv_bfloat16><<<g, 256, 0, ctx->stream>>>((const __nv_bfloat16*)sub, (int)n, cnt);
  else k_c2s_count<uint8_t><<<g, 256, 0, ctx->stream>>>((const uint8_t*)sub, (int)n, cnt);
  T2_LAUNCHED(ctx);
  T2_CUDA(ctx, cub::DeviceScan::InclusiveSum(nullptr, tb, cnt, off + 1, (int)n, ctx->stream));
  T2_CUDA(ctx, scratch.get(&tmp, tb));
  T2_CUDA(ctx, cub::DeviceScan::InclusiveSum(tmp, tb, cnt, off + 1, (int)n, ctx->stream));
  if (m_host) {
    int m = 0;
    T2_CUDA(ctx, cudaMemcpyAsync(&m, off + n, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    T2_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *m_host = m;
  }
  return T2SC_OK;
}

extern "C" int t2sc_subdivide_emit(t2sc_ctx* ctx, const void* sub, int sub_dtype, const int32_t* coords, const int32_t* off,
                                   int64_t n, int32_t* child_coords, int32_t* src) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && n < (1ll << 28), "n=%lld", (long long)n);
  T2_REQ(ctx, sub_dtype == T2SC_F16 || sub_dtype == T2SC_BF16 || sub_dtype == T2SC_U8, "sub dtype %d", sub_dtype);
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, sub && coords && off && child_coords && src, "null tensor");
  T2_REQ(ctx, (uintptr_t)coords % 16 == 0 && (uintptr_t)child_coords % 16 == 0, "coords must be 16-byte aligned");
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  int g = cdiv_i(n, 256);
  if (sub_dtype == T2SC_F16)
    k_c2s_emit<__half><<<g, 256, 0, ctx->stream>>>((const __half*)sub, (const int4*)coords, off, (int)n, (int4*)child_coords, src);
  else if (sub_dtype == T2SC_BF16)
    k_c2s_emit<__nv_bfloat16><<<g, 256, 0, ctx->stream>>>((const __nv_bfloat16*)sub, (const int4*)coords, off, (int)n, (int4*)child_coords, src);
  else
    k_c2s_emit<uint8_t><<<g, 256, 0, ctx->stream>>>((const uint8_t*)sub, (const int4*)coords, off, (int)n, (int4*)child_coords, src);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

extern "C" int t2sc_gather_rows(t2sc_ctx* ctx, const void* x, const int32_t* src, int64_t m, int C, int dtype, void* y) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  size_t row_bytes = (size_t)C * dtype_size(dtype);
  T2_REQ(ctx, m >= 0 && C > 0 && row_bytes % 16 == 0, "m=%lld C=%d: rows must be a multiple of 16 bytes", (long long)m, C);
  if (m == 0) return T2SC_OK;
  T2_REQ(ctx, x && src && y && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0, "null or unaligned tensor");
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  int vpr = (int)(row_bytes / 16);
  k_gather_rows16<<<cdiv_i(m * vpr, 256), 256, 0, ctx->stream>>>((const uint4*)x, src, m, vpr, (uint4*)y);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

extern "C" int t2sc_add_skip(t2sc_ctx* ctx, void* h, const void* x, const int32_t* src, int64_t m, int Co, int Cin, int rep, int dtype) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, m >= 0 && Co > 0 && Cin % 8 == 0 && rep > 0 && Co == (Cin / 8) * rep, "m=%lld Co=%d Cin=%d rep=%d", (long long)m, Co, Cin, rep);
  if (m == 0) return T2SC_OK;
  T2_REQ(ctx, h && x && src, "null tensor");
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  if (dtype == T2SC_F16) add_skip_pick<__half>(ctx->stream, h, x, src, m, Co, Cin, rep);
  else if (dtype == T2SC_BF16) add_skip_pick<__nv_bfloat16>(ctx->stream, h, x, src, m, Co, Cin, rep);
  else if (dtype == T2SC_F32) add_skip_pick<float>(ctx->stream, h, x, src, m, Co, Cin, rep);
  else return t2sc_fail(ctx, T2SC_ERR_ARG, "dtype %d", dtype);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}


// Neighbour rows of the contiguous row range [row_lo, row_hi) only, against the hash of ALL n rows: what one rank
// of a Morton-range partition needs (its owned rows, with global row indices in the map).  nbr [row_hi-row_lo, 27],
// gray [row_hi-row_lo].  No counterpart in the reference, which is single-GPU.
extern "C" int t2sc_build_neighbors_range(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                                          int64_t row_lo, int64_t row_hi, uint32_t* nbr, int32_t* gray) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && n < (1ll << 30) && row_lo >= 0 && row_lo <= row_hi && row_hi <= n, "n=%lld range [%lld,%lld)", (long long)n, (long long)row_lo, (long long)row_hi);
  if (row_hi == row_lo) return T2SC_OK;
  T2_REQ(ctx, coords && nbr && gray, "null tensor");
  T2_REQ(ctx, (uintptr_t)coords % 16 == 0, "coords must be 16-byte aligned");
  T2_REQ(ctx, W > 0 && H > 0 && D > 0, "grid extent %d %d %d", W, H, D);
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  uint32_t cap = 1; while (cap < 2u * (uint32_t)n) cap <<= 1;
  Scratch scratch(ctx);
  char* table = nullptr;
  const int Wb = (W + 1) / 2, Hb = (H + 1) / 2, Db = (D + 1) / 2;
  const size_t table_bytes = (size_t)cap * (sizeof(unsigned long long) + sizeof(BrickVals));
  T2_CUDA(ctx, scratch.get(&table, table_bytes));
  unsigned long long* bkeys = (unsigned long long*)table; BrickVals* bvals = (BrickVals*)(table + (size_t)cap * sizeof(unsigned long long));
  T2_CUDA(ctx, cudaMemsetAsync(table, 0xff, table_bytes, ctx->stream));
  k_brick_insert<<<cdiv_i(n, 256), 256, 0, ctx->stream>>>((const int4*)coords, (int)n, Wb, Hb, Db, bkeys, bvals, cap - 1);
  T2_LAUNCHED(ctx);
  const i64 m = row_hi - row_lo;
  k_brick_neighbors<<<cdiv_i(m, 32), 256, 0, ctx->stream>>>((const int4*)coords + row_lo, (int)m, W, H, D, Wb, Hb, Db, bkeys, bvals, cap - 1, nbr, gray, nullptr);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

// Rows of arbitrary query coordinates in the same voxel hash: what the reference's other hash users need of it
// (vhash_find of src/mesh.cu:7-19, used by the dual-grid quad search :54-72, and the hash half of the grid-sample
// neighbour build, src/glb.cu:545-552).
extern "C" int t2sc_voxel_lookup(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                                 const int32_t* queries, int64_t m, uint32_t* rows) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && n < (1ll << 30) && m >= 0, "n=%lld m=%lld", (long long)n, (long long)m);
  if (m == 0) return T2SC_OK;
  T2_REQ(ctx, queries && rows && (n == 0 || coords), "null tensor");
  T2_REQ(ctx, (uintptr_t)coords % 16 == 0 && (uintptr_t)queries % 16 == 0, "coords and queries must be 16-byte aligned");
  T2_REQ(ctx, W > 0 && H > 0 && D > 0, "grid extent %d %d %d", W, H, D);
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  uint32_t cap = 2; while (cap < 2u * (uint32_t)n) cap <<= 1;
  Scratch scratch(ctx);
  char* table = nullptr;
  const int Wb = (W + 1) / 2, Hb = (H + 1) / 2, Db = (D + 1) / 2;
  const size_t table_bytes = (size_t)cap * (sizeof(unsigned long long) + sizeof(BrickVals));
  T2_CUDA(ctx, scratch.get(&table, table_bytes));
  unsigned long long* bkeys = (unsigned long long*)table; BrickVals* bvals = (BrickVals*)(table + (size_t)cap * sizeof(unsigned long long));
  T2_CUDA(ctx, cudaMemsetAsync(table, 0xff, table_bytes, ctx->stream));
  if (n > 0) {
    k_brick_insert<<<cdiv_i(n, 256), 256, 0, ctx->stream>>>((const int4*)coords, (int)n, Wb, Hb, Db, bkeys, bvals, cap - 1);
    T2_LAUNCHED(ctx);
  }
  k_brick_lookup<<<cdiv_i(m, 256), 256, 0, ctx->stream>>>((const int4*)queries, m, W, H, D, Wb, Hb, Db, bkeys, bvals, cap - 1, rows);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

// ------------------------------------------------------------------------------------------ allocation-free variant
// The hash table of this variant is a fixed array inside the library image instead of pool memory.
static __device__ __align__(256) unsigned char g_static_table[(size_t)2 * T2SC_STATIC_MAX_ROWS * sizeof(Slot)];
static Slot* g_static_table_ptr[64] = {nullptr};      // device address of the array, per device, resolved on first use

extern "C" int t2sc_build_neighbors_static(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                                           uint32_t* nbr, int32_t* gray) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0, "n=%lld", (long long)n);
  if (n > T2SC_STATIC_MAX_ROWS)
    return t2sc_fail(ctx, T2SC_ERR_UNSUPPORTED, "t2sc_build_neighbors_static: %lld rows exceed the built-in table (at most %d rows); "
                     "use t2sc_build_neighbors, which takes its table from the memory pool", (long long)n, T2SC_STATIC_MAX_ROWS);
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, coords && nbr && gray, "null tensor");
  T2_REQ(ctx, (uintptr_t)coords % 16 == 0, "coords must be 16-byte aligned");
  T2_REQ(ctx, W > 0 && H > 0 && D > 0, "grid extent %d %d %d", W, H, D);
  T2_REQ(ctx, ctx->device >= 0 && ctx->device < 64, "device %d", ctx->device);
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!g_static_table_ptr[ctx->device]) {
    // In host code the array's name is only a handle; the kernels need its address on THIS device.
    void* p = nullptr;
    T2_CUDA(ctx, cudaGetSymbolAddress(&p, g_static_table));
    g_static_table_ptr[ctx->device] = (Slot*)p;
  }
  Slot* table = g_static_table_ptr[ctx->device];
  uint32_t cap = 1; while (cap < 2u * (uint32_t)n) cap <<= 1;
  // the array keeps the previous call's keys: every slot this call can probe is reset to "empty" first
  T2_CUDA(ctx, cudaMemsetAsync(table, 0xff, (size_t)cap * sizeof(Slot), ctx->stream));
  k_hash_insert<<<cdiv_i(n, 256), 256, 0, ctx->stream>>>((const int4*)coords, (int)n, W, H, D, table, cap - 1);
  T2_LAUNCHED(ctx);
  k_neighbors<<<cdiv_i(n, NB_ROWS), NB_THREADS, 0, ctx->stream>>>((const int4*)coords, (int)n, W, H, D, table, cap - 1, nbr, gray, nullptr);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}
