// tcgen05 / TMEM masked implicit-GEMM sparse convolution for sm_100a (fp16 or bf16 in, fp32 accumulate).
//
// Computes the operator of src/spconv.cu:91-150 (trellis2-cuda): for every output row and every tap
// present in its tile, y[row, co] += x[nbr[row, v], :] . w[co, v, :].  The reference runs 32-64 row tiles
// through mma.sync with register-staged copies; this kernel is organised around the Blackwell units:
//
//   * persistent CTAs, one per SM, walk (plan tile x BN output channels) work items.  A plan tile is MH
//     128-row halves (MH = 1 or 2); each half has its own TMEM accumulator and all halves consume the
//     same weight slab, which halves the L2 -> SM weight traffic of the 128-row schedule;
//   * warps 0-3 gather the A operand: one 16-byte cp.async per (row, 8 channels), zero-filled for absent
//     neighbours, written straight into the 128-byte-swizzled K-major layout tcgen05 reads.  (TMA
//     tile::gather4 was measured for this job and moves 128-byte rows three times slower.)  Everything that
//     does not depend on the channel chunk is done once per tap, so a copy is two instructions;
//   * warp 5 and the last warp of the base set copy each tile's neighbour-map rows into a [27 taps][rows] table in
//     shared memory (4-byte cp.async, a whole tile in flight at once), one tile ahead of the gather warps, so
//     that neither a tap nor a new tile starts with a chain of dependent loads;
//   * one lane of warp 4 streams the B operand (the tap's [BN x 64] weight slab) with a 3-D TMA tile load
//     from the weights in their checkpoint layout [Co,27,Ci] - no re-layout, no cluster multicast;
//   * one lane of warp 6 issues tcgen05.mma (M=128, N=BN, K=16) per half into TMEM and releases smem stages /
//     publishes accumulators with tcgen05.commit; when 2*MH*BN <= 512 columns the accumulators are double
//     buffered so the epilogue of one tile overlaps the main loop of the next;
//   * 4*MH epilogue warps drain the accumulators with tcgen05.ld and apply the fused epilogue (bias,
//     LayerNorm, activation, residual, skip) with the reference's rounding points, one thread per output
//     row, and scatter rows back to the caller's order.
//
// The roles run their instructions in order, and their per-unit instruction paths (not the pipeline depth) bound
// the narrow layers: every role keeps its loop short, fetches the next tile's descriptor early and branches once
// per unit at most.
//
// Every mbarrier wait is bounded: a wait that runs out sets the context's status word, the CTA stops
// blocking, drains and frees its TMEM; the host reports T2SC_ERR_DEVICE.
#include "umma_common.cuh"

namespace {
using namespace umma;

// ------------------------------------------------------------------------------------------ kernel
// Warp roles: 0-3 gather A (cp.async), 4 weights (TMA), 5 and the last warp of the base set fill the neighbour-index table,
// 6 MMA issue + TMEM owner, 7.. epilogue (4 warps per 128-row half).
// A unit is one (tap, 64-channel chunk): 16 KB of gathered rows per 128-row half, one weight slab, four MMAs per half.
// One pipeline stage holds U consecutive units of a tile.  Every role pays one barrier round trip per STAGE (a wait
// that answers after ~100 clocks, an arrival or commit), in order, whatever the stage holds; with one unit per stage
// that is ~400 clocks per unit against 64 to 256 clocks of tensor time at Co <= 128, so narrow layers take U = 2 or 4.
// G = gather groups of four warps.  G = 1: the four gather warps fill every stage together.  G = 2 (128-row tiles):
// a second group of four warps sits behind the epilogue warps and the groups fill alternate stages, so one group's
// barrier round trips and index reads overlap the other group's copies.
//
// Neighbour indices reach the gather warps through a per-TILE table in shared memory ([27 taps][rows], two buffers).  The
// plan keeps the map in exactly that form, tile by tile, so one lane fetches a tile's table with ONE bulk copy (13.8 KB
// per 128 rows) a tile ahead and the gather warps meet one barrier per tile.  A warp issues roughly one instruction per ten
// clocks here, so anything that costs instructions per (row, tap) in the kernel - a ring slot per tap, or warps that
// transpose map rows into the table - took longer than the tile's MMAs at 64 and 128 channels.
// Only the peer-memory form, whose map arrives with the call, still has two index warps that build the table from map
// rows (4-byte cp.async, one 108-byte row per warp instruction), mark absent / out-of-range entries and flag the taps
// that read a peer.
template <int BN, int MH, int G, int U, bool PEERS, class T>
__global__ void __launch_bounds__(num_threads(MH, G), 1) k_conv_umma(const __grid_constant__ CUtensorMap tmw, const ConvArgs a) {
  static_assert(G == 1 || (G == 2 && MH == 1), "a second gather group only fits beside 128-row tiles");
  constexpr int UNIT = stage_bytes(BN, MH);          // MH gathered A halves + one weight slab
  constexpr int STAGE = U * UNIT;
  constexpr int S = num_stages(BN, MH, U);
  constexpr int B_BYTES = BN * 128;
  constexpr int NB = num_acc_bufs(BN, MH);            // accumulator buffers, each MH halves of BN columns
  constexpr int TMEM_COLS = NB * MH * BN < 32 ? 32 : NB * MH * BN;
  constexpr int ROWS = MH * TILE_M;
  constexpr int PITCH = PEERS ? tab_pitch(MH) : ROWS;  // the index warps write a map row per instruction: an odd pitch keeps that conflict-free
  constexpr int TABW = 27 * PITCH;
  constexpr int NGW = 4 * G;                          // gather warps

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint32_t* itab = (uint32_t*)(smem + S * STAGE);      // NTAB x [27][PITCH] neighbour indices, one table per tile in flight
  uint64_t* bars = (uint64_t*)(itab + NTAB * TABW);    // full[S] empty[S] accf[2] acce[2] tready[NTAB] tfree[NTAB]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * S + 4 + 2 * NTAB);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 2);   // [0] a wait gave up, [1] the wait limit
  const void** peer_base = (const void**)(tmem_slot + 4);      // the peers' array addresses (PEERS only)
  uint32_t* tab_remote = (uint32_t*)(peer_base + 8);           // PEERS: [NTAB][2 index warps][32 taps] does the tap read any row of a peer?
  uint32_t* peer_rows = tab_remote + NTAB * 64;                // PEERS: rows of every peer's array (bounds of the map entries)
  // epilogue staging: LayerNorm gamma / beta of the row, and per epilogue warp the bias values of its current item
  uint8_t* epi_s = (uint8_t*)(((uintptr_t)(smem + S * STAGE + aux_bytes(MH) - epi_bytes(MH)) + 15) & ~(uintptr_t)15);
  float* gamma_s = (float*)epi_s; float* beta_s = gamma_s + 256;
  T* bias_s = (T*)(beta_s + 256);                              // [4 * MH epilogue warps][256]

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * S, bar_accf = bar_empty + 8 * S, bar_acce = bar_accf + 16,
                 bar_tready = bar_acce + 16, bar_tfree = bar_tready + 8 * NTAB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nchunk = a.Ci / KCH;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, NUM_PROD_THREADS + 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(bar_accf + 8 * b, 1); mbar_init(bar_acce + 8 * b, 128 * MH); }
    for (int r = 0; r < NTAB; r++) { mbar_init(bar_tready + 8 * r, PEERS ? 2 : 1); mbar_init(bar_tfree + 8 * r, NGW); }   // two index warps (or the one loader lane) fill, every gather warp releases
    for (int r = 0; r < NTAB * 64; r++) tab_remote[r] = 0;
    abort_flag[0] = 0; abort_flag[1] = a.wait_limit;
    if (PEERS) for (int r = 0; r < 8; r++) { peer_base[r] = a.xp[r]; peer_rows[r] = a.xp_rows[r]; }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (a.ep.ln) {        // the whole row is one accumulator (n_cot == 1): column = index
    for (int i = threadIdx.x; i < BN; i += blockDim.x) { gamma_s[i] = a.ep.gamma ? a.ep.gamma[i] : 1.f; beta_s[i] = a.ep.beta ? a.ep.beta[i] : 0.f; }
  }
  if (warp == WARP_MMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // dense_rows > 0 (t2sc_linear): there is no plan; tile t is rows [t * ROWS, t * ROWS + ROWS) with one tap
  const bool dense = a.dense_rows > 0;
  const int tile0 = dense ? 0 : *a.tile_lo, ntiles = dense ? (a.dense_rows + ROWS - 1) / ROWS : *a.tile_hi - tile0;
  const PlanTile* const tiles = a.tiles + tile0;
  auto tile_at = [&](int t) {
    if (dense) return PlanTile{t * ROWS, min(ROWS, a.dense_rows - t * ROWS), 0, 1u};
    return tiles[t];
  };
  const int nitems = ntiles * a.n_cot;
  // Work items of this CTA.  With a.perm (plans over maps sorted as one block, up to 262,144 rows): position g in the
  // launch's item list is tile a.perm[g / n_cot] - the plan's tiles by falling tap count - and column slab g % n_cot, and the
  // CTAs take the positions round by round in alternating direction, so that the CTA with the longest tile of one round
  // gets the shortest of the next.  Tiles differ 9..27 in taps: taken in plan order the busiest SM had 14 % more taps than
  // the mean on a 1,702-tile map (measured: 4-6 % of the conv's time there).  Without a.perm (large maps, whose plans sort
  // inside runs of caller rows so that concurrently running tiles gather from the same part of the array): plan order,
  // CTA b takes items b, b + grid, ...; permuting those tiles, even within windows of four rounds, cost 3 % on 67,176 tiles.
  auto item_at = [&](int k) {
    const int g = k * (int)gridDim.x + ((k & 1) && a.perm ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
    return g < nitems ? g : -1;
  };
  auto tidx_of = [&](int item) { const int t = item / a.n_cot; return (dense || !a.perm) ? t : a.perm[tile0 + t] - tile0; };
  auto tile_of = [&](int item) { return tile_at(tidx_of(item)); };

  if (warp < 4 || (G == 2 && warp >= warp_group2(MH))) {
    // ===================================================================== A producer: gather rows into the swizzled tile
    const int g = warp < 4 ? 0 : 1;                                            // gather group (G == 2: fills the units with it % 2 == g)
    const T* x = (const T*)a.x;          // PEERS: the local array, xp[self_rank]
    const int t = threadIdx.x & 127, jbase = t >> 3, c16 = t & 7;              // both groups start at a multiple of 128 threads
    const uint32_t dst_thread = (uint32_t)(jbase * 128 + ((c16 ^ (jbase & 7)) << 4));   // (jbase + 16 i) & 7 == jbase & 7
    uint32_t it = 0, tt = 0;
    bool alive = true;
    const bool prof = diag(a, 8); long long w_idx = 0, w_empty = 0, t_role = clock64();
    int item_n = item_at(0);
    PlanTile tile_next = item_n >= 0 ? tile_of(item_n) : PlanTile{};
    for (int k = 0; item_n >= 0; k++, tt++) {
      const PlanTile tile = tile_next;
      item_n = item_at(k + 1);
      if (item_n >= 0) tile_next = tile_of(item_n);     // in flight while this tile is gathered
      const uint32_t buf = tt % NTAB;
      // Every gather warp waits for every tile's table, also one that has none of the tile's units (G == 2): a warp can
      // then never release a buffer twice within one phase of its barrier.
      if (threadIdx.x == 0) trace(a, 0, 0, tt);
      if (!dense) alive &= mbar_wait_t(bar_tready + 8 * buf, (tt / NTAB) & 1, abort_flag, a.status, 32, prof, w_idx);
      if (threadIdx.x == 0) trace(a, 0, 1, tt);
      const uint32_t* tab = itab + buf * TABW + jbase;
      const int nunits = __popc(tile.mask) * nchunk;
      uint32_t mk = tile.mask;        // taps still to come; the current tap is its lowest set bit, c the current chunk
      int c = 0, held_tap = -1;       // held_tap: the tap whose indices are in idx[] / sz[] / rp[]
      uint32_t idx[8 * MH], sz[8 * MH];       // rows jbase + 16 i; rows 128.. are the second half, stored right behind the first
      const T* rp[PEERS ? 8 * MH : 1];
      bool remote = false;
      for (int u0 = 0; u0 < nunits; u0 += U, it++) {
        const int nu = nunits - u0 < U ? nunits - u0 : U;      // a tile's last stage may be short
        // G == 2: the groups alternate stages.  A group waits on stages two apart, never more than the stage count apart,
        // so it cannot run two phases ahead of a stage, where a parity wait would pass by mistake.
        if (G == 2 && (int)(it & 1) != g) {
          for (int k = 0; k < nu; k++) if (++c == nchunk) { c = 0; mk &= mk - 1; }
          continue;
        }
        const uint32_t st = it % S;
        alive &= mbar_wait_t(bar_empty + 8 * st, ((it / S) & 1) ^ 1, abort_flag, a.status, 1, prof, w_empty);
        if ((threadIdx.x & 127) == 0) trace(a, 4, 3, it);          // stage-level events (first 64 stages): the gather group holds a free stage
#pragma unroll
        for (int k = 0; k < U; k++) {
          if (k >= nu) break;
          const int v = __ffs(mk) - 1;
          if (v != held_tap) {
            held_tap = v;
            // Table entries: row number (PEERS: (owner << PEER_SHIFT) | row), or RING_ABSENT.  Everything that does not
            // depend on the channel chunk is done here, once per tap, so that a copy costs two instructions (address,
            // cp.async): the gather warps run these in order.
            if (dense) {
#pragma unroll
              for (int i = 0; i < 8 * MH; i++) idx[i] = jbase + 16 * i < tile.rows ? (uint32_t)(tile.start + jbase + 16 * i) : RING_ABSENT;
            } else {
#pragma unroll
              for (int i = 0; i < 8 * MH; i++) idx[i] = tab[v * PITCH + 16 * i];
            }
            // PEERS: almost every tap reads local rows only (the index warps say so per tap) and takes the plain path with
            // the owner bits masked off.  For a tap with rows of a peer the addresses are formed here: a table load between
            // the copies below would be ordered after each of them and serialise the loop.
            if constexpr (PEERS) {
              remote = (tab_remote[buf * 64 + v] | tab_remote[buf * 64 + 32 + v]) != 0;
              if (__builtin_expect(remote, 0)) {
#pragma unroll
                for (int i = 0; i < 8 * MH; i++)
                  rp[i] = idx[i] != RING_ABSENT ? (const T*)peer_base[idx[i] >> PEER_SHIFT] + (i64)(idx[i] & PEER_ROW_MASK) * a.Ci + c16 * 8 : x;
              }
            }
#pragma unroll
            for (int i = 0; i < 8 * MH; i++) {
              sz[i] = (~idx[i] >> 27) & 16u;                                 // 16 bytes, or 0 = zero-fill for an absent neighbour
              idx[i] &= PEERS ? PEER_ROW_MASK : 0x7FFFFFFFu;                 // absent -> row 0, a valid address that is not read
            }
          }
          // After a wait was given up this thread loads and signals nothing more: the table may hold anything, and an
          // arrival on a barrier whose phase is still waiting for bytes in flight would overrun its count.
          if (alive && !diag(a, 1)) {
            const uint32_t dst = smem_base + st * STAGE + k * UNIT + dst_thread;
            const T* xs = x + c * KCH + c16 * 8;
            if (PEERS && __builtin_expect(remote, 0)) {          // one branch per unit, not per copy: a P2P load when the owner is a peer
#pragma unroll
              for (int i = 0; i < 8 * MH; i++) cp_async16(dst + i * (16 * 128), rp[i] + c * KCH, sz[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 8 * MH; i++) cp_async16(dst + i * (16 * 128), xs + (i64)idx[i] * a.Ci, sz[i]);
            }
          }
          if (++c == nchunk) { c = 0; mk &= mk - 1; }
        }
        if (alive) cp_async_arrive_noinc(bar_full + 8 * st);     // this thread's arrival, delivered when its copies have landed
        if ((threadIdx.x & 127) == 0) trace(a, 0, 3, it);          // ... has issued its copies
      }
      // the tile's last indices are in registers: the index warps may refill this table
      __syncwarp();
      if (lane == 0 && alive && !dense) mbar_arrive(bar_tfree + 8 * buf);
      if (threadIdx.x == 0) trace(a, 0, 2, tt);
    }
    cp_async_wait_all();
    if (prof && blockIdx.x == 0 && threadIdx.x == 0)
      printf("[t2sc prof] gather: total %lld clk, wait index table %lld, wait stage free %lld, units %u\n", clock64() - t_role, w_idx, w_empty, it);
  } else if (warp == WARP_TMA) {
    // ===================================================================== B producer (weights by TMA): one lane does it all
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;        // false once a wait was given up: nothing more is loaded or signalled
      int item_n = item_at(0);
      PlanTile tile_next = item_n >= 0 ? tile_of(item_n) : PlanTile{};
      for (int k = 0; item_n >= 0 && alive; k++) {
        const int cot = item_n % a.n_cot;
        const PlanTile tile = tile_next;
        item_n = item_at(k + 1);
        if (item_n >= 0) tile_next = tile_of(item_n);
        const int wrow = tile.wbase * a.Co + cot * BN;
        const int nunits = __popc(tile.mask) * nchunk;
        uint32_t mk = tile.mask;
        int c = 0;
        for (int u0 = 0; u0 < nunits; u0 += U, it++) {
          const int nu = nunits - u0 < U ? nunits - u0 : U;
          const uint32_t st = it % S;
          alive &= mbar_wait(bar_empty + 8 * st, ((it / S) & 1) ^ 1, abort_flag, a.status, 2);
          if (!alive) break;
          trace(a, 1, 1, it);                                      // ... the weight lane holds the stage
          const bool mute = diag(a, 16) && it == 0;      // bounded-wait test: this stage never fills, the MMA lane's wait runs out
          if (!mute) {
            if (diag(a, 2)) mbar_arrive(bar_full + 8 * st);
            else mbar_arrive_expect_tx(bar_full + 8 * st, nu * B_BYTES);
          }
#pragma unroll
          for (int k = 0; k < U; k++) {
            if (k >= nu) break;
            if (!mute && !diag(a, 2))
              tma_load_3d(smem_base + st * STAGE + k * UNIT + MH * A_BYTES, &tmw, c * KCH, __ffs(mk) - 1, wrow, bar_full + 8 * st);
            if (++c == nchunk) { c = 0; mk &= mk - 1; }
          }
        }
        trace(a, 1, 0, (uint32_t)k);
      }
    }
    __syncwarp();
  } else if (!PEERS && (warp == WARP_IDX || warp == warp_idx2(MH))) {
    // ===================================================================== neighbour-index table: one bulk copy per tile
    if (warp == WARP_IDX && lane == 0 && !dense) {
      uint32_t tt = 0;
      int item_n = item_at(0);
      int tidx_next = item_n >= 0 ? tidx_of(item_n) : 0;
      for (int k = 0; item_n >= 0; k++, tt++) {
        const int tidx = tidx_next;
        item_n = item_at(k + 1);
        if (item_n >= 0) tidx_next = tidx_of(item_n);      // the next tile's number is in flight while this table is fetched
        const uint32_t buf = tt % NTAB;
        trace(a, 2, 0, tt);
        if (!mbar_wait(bar_tfree + 8 * buf, ((tt / NTAB) & 1) ^ 1, abort_flag, a.status, 64)) break;
        trace(a, 2, 1, tt);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the gather warps' reads of this buffer come before the copy's writes
        mbar_arrive_expect_tx(bar_tready + 8 * buf, TABW * 4);
        bulk_load(smem_u32(itab + buf * TABW), a.tnbr + (i64)(tile0 + tidx) * TABW, TABW * 4, bar_tready + 8 * buf);
        trace(a, 2, 3, tt);
      }
    }
    __syncwarp();
  } else if (warp == WARP_IDX || warp == warp_idx2(MH)) {
    // ===================================================================== peer-memory form: neighbour-index table built from map rows
    // Two index warps, each serving half of the tile's rows, one tile ahead of the gather warps.  Tile descriptors are
    // fetched two tiles ahead and row numbers one tile ahead, so no dependent load sits on a tile boundary; the map rows
    // themselves go from global to shared memory by cp.async, a whole half tile in flight at once and no register per entry.
    const int ih = warp == WARP_IDX ? 0 : 1;
    constexpr int HROWS = ROWS / 2, NR = HROWS / 32;
    uint32_t tt = 0;
    bool oob = false;         // a present map entry pointed past the end of its feature array: read as absent and reported
    const bool prof = diag(a, 8); long long w_free = 0, w_load = 0, t_role = clock64();
    auto rows_of = [&](const PlanTile& tl, int* nr) {
#pragma unroll
      for (int i = 0; i < NR; i++) {
        const int j = ih * HROWS + lane + 32 * i;
        nr[i] = -1;
        if (j < tl.rows) { const int r = a.order[tl.start + j]; nr[i] = a.src ? (a.src[r] >> 3) : r; }
      }
    };
    auto desc_of = [&](int k) { const int it_ = item_at(k); return it_ >= 0 ? tile_of(it_) : PlanTile{}; };
    int nr[NR], nr_next[NR];
    PlanTile tile_n0 = desc_of(0), tile_n1 = desc_of(1);
    rows_of(tile_n0, nr);
    for (int k = 0; item_at(k) >= 0; k++, tt++) {
      const PlanTile tile_n2 = desc_of(k + 2);
      rows_of(tile_n1, nr_next);                               // in flight while this tile is served
      const uint32_t buf = tt % NTAB;
      // warp-uniform: the fill below is a warp-wide exchange of row numbers, and after a wait was given up nothing more
      // is written or signalled
      if (ih == 0 && lane == 0) trace(a, 2, 0, tt);
      if (!__all_sync(0xffffffffu, mbar_wait_t(bar_tfree + 8 * buf, ((tt / NTAB) & 1) ^ 1, abort_flag, a.status, 64, prof, w_free))) break;
      if (ih == 0 && lane == 0) trace(a, 2, 1, tt);
      uint32_t* tab = itab + buf * TABW + ih * HROWS;
      long long t_l0 = prof ? clock64() : 0;
#pragma unroll
      for (int i = 0; i < NR; i++) {
#pragma unroll 8
        for (int l = 0; l < 32; l++) {
          const int row = __shfl_sync(0xffffffffu, nr[i], l);            // lane l holds the row; lanes 0..26 copy one tap of it each
          if (lane < 27) {
            uint32_t* dst = tab + lane * PITCH + 32 * i + l;
            if (row >= 0 && !diag(a, 32)) cp_async4(smem_u32(dst), a.nbr + (i64)row * 27 + lane);
            else *dst = RING_ABSENT;                                       // rows past the end of a short tile
          }
        }
      }
      cp_async_wait_all();
      __syncwarp();
      if (ih == 0 && lane == 0) trace(a, 2, 2, tt);
      if (prof) w_load += clock64() - t_l0;
      // Second pass over the landed entries, lane = tap: absent and out-of-range entries become RING_ABSENT (bit 31), and
      // in the peer-memory form each tap learns whether any of its rows lives on another rank.
      if (lane < 27) {
        bool rem = false;
#pragma unroll 8
        for (int j = 0; j < HROWS; j++) {
          const uint32_t e = tab[lane * PITCH + j];
          if (e == RING_ABSENT) continue;
          bool bad;
          if constexpr (!PEERS) bad = e >= a.n_in;                   // NBR_EMPTY is above every row count
          else {
            const uint32_t owner = e >> PEER_SHIFT;
            bad = e == NBR_EMPTY || owner >= (uint32_t)a.npeers || (e & PEER_ROW_MASK) >= peer_rows[owner & 7];
            rem |= !bad && (int)owner != a.self_rank;
          }
          if (bad) { oob |= e != NBR_EMPTY; tab[lane * PITCH + j] = RING_ABSENT; }
        }
        if constexpr (PEERS) tab_remote[buf * 64 + ih * 32 + lane] = rem;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tready + 8 * buf);
      if (ih == 0 && lane == 0) trace(a, 2, 3, tt);
#pragma unroll
      for (int i = 0; i < NR; i++) nr[i] = nr_next[i];
      tile_n0 = tile_n1; tile_n1 = tile_n2;
    }
    if (__any_sync(0xffffffffu, oob) && lane == 0) atomicOr(a.status, 256);
    if (prof && blockIdx.x == 0 && lane == 0 && ih == 0)
      printf("[t2sc prof] index warp: total %lld clk, wait table free %lld, map rows in flight %lld, tiles %u\n", clock64() - t_role, w_free, w_load, tt);
  } else if (warp == WARP_MMA) {
    // ===================================================================== MMA issuer: one lane waits, issues and commits
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BN, a.is_bf16);
      const uint64_t desc0 = umma_desc(smem_base);      // every operand's descriptor is this + (its byte offset >> 4): the start-address field cannot overflow within 227 KB
      uint32_t it = 0, acc_it = 0;
      bool alive = true;        // false once a wait was given up: no more MMAs or commits
      const bool prof = diag(a, 8); long long w_full = 0, w_acc = 0, w_issue = 0, w_commit = 0, t_role = clock64();
      int item_n = item_at(0);
      PlanTile tile_next = item_n >= 0 ? tile_of(item_n) : PlanTile{};
      for (int k = 0; item_n >= 0 && alive; k++, acc_it++) {
        const PlanTile tile = tile_next;
        item_n = item_at(k + 1);
        if (item_n >= 0) tile_next = tile_of(item_n);
        const uint32_t buf = acc_it % NB, aph = (acc_it / NB) & 1;
        trace(a, 3, 0, acc_it);
        alive &= mbar_wait_t(bar_acce + 8 * buf, aph ^ 1, abort_flag, a.status, 4, prof, w_acc);
        if (!alive) break;
        trace(a, 3, 1, acc_it);
        tc_fence_after();                       // the epilogue's tcgen05.ld of this buffer come before the MMAs that overwrite it
        const uint32_t d_tmem = tmem_base + buf * (MH * BN);
        const int halves = tile.rows > TILE_M ? MH : 1;
        const int nunits = __popc(tile.mask) * nchunk;
        for (int u0 = 0; u0 < nunits; u0 += U, it++) {
          const int nu = nunits - u0 < U ? nunits - u0 : U;
          const uint32_t s = it % S, ph = (it / S) & 1;
          // No tcgen05 fence after this wait (the operands are shared-memory data published by the barrier, not tcgen05
          // results) and no proxy fence either: the copies' completion is delivered through the barrier itself
          // (cp.async.mbarrier.arrive.noinc); a fence.proxy.async here was measured at 3-12 % of the kernel time.
          trace(a, 3, 3, it);                                      // ... the MMA lane starts waiting for it
          alive &= mbar_wait_t(bar_full + 8 * s, ph, abort_flag, a.status, 8, prof, w_full);
          if (!alive) break;
          trace(a, 1, 2, it);                                      // ... the stage is full
          long long ti0 = prof ? clock64() : 0;
          if (!diag(a, 4)) {
            const uint64_t ds = desc0 + (uint64_t)(s * (STAGE >> 4));          // descriptor of the stage's first byte
#pragma unroll
            for (int k = 0; k < U; k++) {
              if (k >= nu) break;
#pragma unroll
              for (int h = 0; h < MH; h++) {
                if (h < halves)
                  tc_mma_k64(d_tmem + h * BN, ds + ((k * UNIT + h * A_BYTES) >> 4), ds + ((k * UNIT + MH * A_BYTES) >> 4), idesc, u0 + k > 0 ? 1u : 0u);
              }
            }
          }
          long long ti1 = prof ? clock64() : 0;
          tc_commit(bar_empty + 8 * s);
          trace(a, 1, 3, it);                                      // ... its MMAs are issued and the commit is behind them
          if (prof) { w_issue += ti1 - ti0; w_commit += clock64() - ti1; }
        }
        if (alive) tc_commit(bar_accf + 8 * buf);
        trace(a, 3, 2, acc_it);
      }
      if (prof && blockIdx.x == 0)
        printf("[t2sc prof] mma: total %lld clk, wait stage full %lld, wait accumulator free %lld, mma issue %lld, commit %lld, steps %u, tiles %u\n",
               clock64() - t_role, w_full, w_acc, w_issue, w_commit, it, acc_it);
    }
    __syncwarp();
  } else {
    // ===================================================================== epilogue
    const bool has_skip = a.ep.skip_x != nullptr;
    const int q = warp & 3, half = (warp - WARP_EPI0) >> 2, j = half * TILE_M + q * 32 + lane;
    uint32_t acc_it = 0;
    const bool prof = diag(a, 8); long long w_accf = 0, t_role = clock64();
    int item_n = item_at(0);
    PlanTile tile_next = item_n >= 0 ? tile_of(item_n) : PlanTile{};
    for (int k = 0; item_n >= 0; k++, acc_it++) {
      const int cot = item_n % a.n_cot;
      const PlanTile tile = tile_next;
      item_n = item_at(k + 1);
      if (item_n >= 0) tile_next = tile_of(item_n);
      const uint32_t buf = acc_it % NB, aph = (acc_it / NB) & 1;
      const int orow = j < tile.rows ? (dense ? tile.start + j : a.order[tile.start + j]) : -1;
      const int wcol0 = tile.wbase * a.Co + cot * BN;      // bias index of this item's first column
      int sp = 0, ss = 0;
      if (has_skip && orow >= 0) { int sv = a.ep.skip_src[orow]; sp = sv >> 3; ss = sv & 7; }
      // this warp's copy of the item's bias values, in flight while it waits for the accumulator
      T* const bias_w = bias_s + (warp - WARP_EPI0) * 256;
      if (a.ep.bias) {
        __syncwarp();                                     // the previous item's reads of the copy are done
        if (lane < BN / 8) ((uint4*)bias_w)[lane] = __ldg((const uint4*)((const T*)a.ep.bias + wcol0) + lane);
        __syncwarp();
      }
      // warp-uniform (tcgen05.ld is warp-collective); after a wait was given up nothing more is read or signalled
      if (warp == WARP_EPI0 && lane == 0) trace(a, 4, 0, acc_it);
      if (!__all_sync(0xffffffffu, mbar_wait_t(bar_accf + 8 * buf, aph, abort_flag, a.status, 16, prof, w_accf))) break;
      if (warp == WARP_EPI0 && lane == 0) trace(a, 4, 1, acc_it);
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (MH * BN) + half * BN;
      if (!diag(a, 64)) epilogue_row<BN, T>(a, taddr, orow, cot, a.ep.bias ? bias_w : nullptr, gamma_s, beta_s, sp, ss);
      tc_fence_before();
      mbar_arrive(bar_acce + 8 * buf);
      if (warp == WARP_EPI0 && lane == 0) trace(a, 4, 2, acc_it);
    }
    if (prof && blockIdx.x == 0 && warp == WARP_EPI0 && lane == 0)
      printf("[t2sc prof] epilogue: total %lld clk, wait accumulator full %lld (busy %lld), tiles %u\n", clock64() - t_role, w_accf, clock64() - t_role - w_accf, acc_it);
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag[0]) {        // a wait gave up: let copies still in flight land before the smem and TMEM are released
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {}
    __syncthreads();
  }
  if (warp == WARP_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

template <int BN, int MH, int G, int U, bool PEERS, class T>
int launch_p(t2sc_ctx* ctx, const CUtensorMap& tm, const ConvArgs& args, i64 max_items) {
  constexpr int smem = num_stages(BN, MH, U) * U * stage_bytes(BN, MH) + aux_bytes(MH) + 1024;
  static_assert(smem <= SMEM_BUDGET && num_stages(BN, MH, U) >= 2, "shared memory budget");
  static bool attr_set[16] = {};
  if (!attr_set[ctx->device & 15]) {
    T2_CUDA(ctx, cudaFuncSetAttribute(k_conv_umma<BN, MH, G, U, PEERS, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[ctx->device & 15] = true;
  }
  int grid = (int)(max_items < ctx->num_sms ? max_items : ctx->num_sms);
  k_conv_umma<BN, MH, G, U, PEERS, T><<<grid, num_threads(MH, G), smem, ctx->stream>>>(tm, args);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

// Which form runs.  128-row tiles with Co <= 128 (accumulator tiles of 32..128 columns): two gather groups and two units
// per stage (measured 5-12 % faster than one unit per stage at 64 and 128 channels; four units per stage are no better
// than two).  Co % 256 == 0: one unit per stage (a stage is 48 KB there), the second gather group only for Ci = 64.
// 256-row tiles and the peer-memory form: one group, one unit per stage.  The diagnostic build can force one unit per
// stage (T2SC_UNITS=1) to compare the forms.
template <int BN, int MH, class T>
int launch_bn(t2sc_ctx* ctx, const CUtensorMap& tm, const ConvArgs& args, i64 max_items) {
  if (args.npeers > 0) return launch_p<BN, MH, 1, 1, true, T>(ctx, tm, args, max_items);
  if constexpr (MH == 1 && BN <= 128) {
#ifdef T2SC_DIAG
    static const int force_u = [] { const char* e = getenv("T2SC_UNITS"); return e ? atoi(e) : 0; }();
    if (force_u == 1) return args.Ci == KCH ? launch_p<BN, MH, 2, 1, false, T>(ctx, tm, args, max_items) : launch_p<BN, MH, 1, 1, false, T>(ctx, tm, args, max_items);
#endif
    return launch_p<BN, MH, 2, 2, false, T>(ctx, tm, args, max_items);
  } else {
    if constexpr (MH == 1) {
      if (args.Ci == KCH) return launch_p<BN, MH, 2, 1, false, T>(ctx, tm, args, max_items);
    }
    return launch_p<BN, MH, 1, 1, false, T>(ctx, tm, args, max_items);
  }
}

template <int MH, class T>
int launch_t(t2sc_ctx* ctx, int BN, const CUtensorMap& tm, const ConvArgs& args, i64 max_items) {
  switch (BN) {
    case 256: return launch_bn<256, MH, T>(ctx, tm, args, max_items);
    case 128: return launch_bn<128, MH, T>(ctx, tm, args, max_items);
    case 64: return launch_bn<64, MH, T>(ctx, tm, args, max_items);
    default: return launch_bn<32, MH, T>(ctx, tm, args, max_items);
  }
}

int pick_bn(int Co) {
  for (int bn : {256, 128, 64, 32}) if (Co % bn == 0) return bn;
  return 0;
}

}  // namespace

bool conv_umma_supported(int dtype, int Ci, int Co, const EpiDev& ep) {
  (void)ep;
  return (dtype == T2SC_F16 || dtype == T2SC_BF16) && Ci % KCH == 0 && Co % 32 == 0;
}

bool conv_umma_fuses_ln(int Co) { return pick_bn(Co) == Co; }

int conv_umma_launch(t2sc_ctx* ctx, const t2sc_plan* plan, const void* x, const void* w, i64 w_rows, const EpiDev& ep, void* y,
                     int dtype, i64 n_in, int Ci, int Co, int part, const void* const* x_peers, const int64_t* rows_peers, int n_peers,
                     int self_rank, const uint32_t* peer_nbr) {
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  const int BN = pick_bn(Co);
  T2_REQ(ctx, BN > 0, "Co=%d", Co);
  T2_REQ(ctx, !ep.ln || Co == BN, "fused LayerNorm needs the whole row in one tile (Co=%d)", Co);
  EncodeTiledFn enc = encode_fn();
  if (!enc) return t2sc_fail(ctx, T2SC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  // weights [w_rows, 27, Ci] as a 3-D tensor (innermost first): Ci, 27, w_rows; box = 64 channels x 1 tap x BN rows
  CUtensorMap tm;
  cuuint64_t dims[3] = {(cuuint64_t)Ci, 27, (cuuint64_t)w_rows};
  cuuint64_t strides[2] = {(cuuint64_t)Ci * 2, (cuuint64_t)Ci * 2 * 27};
  cuuint32_t box[3] = {(cuuint32_t)KCH, 1, (cuuint32_t)BN};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult cr = enc(&tm, dtype == T2SC_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return t2sc_fail(ctx, T2SC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for weights [%lld,27,%d]", (int)cr, (long long)w_rows, Ci);
  ConvArgs args;
  diag_args(args);
#ifdef T2SC_DIAG
  static long long* trace_buf = nullptr;
  const char* trace_path = getenv("T2SC_TRACE");
  if (trace_path) {
    if (!trace_buf) T2_CUDA(ctx, cudaMalloc(&trace_buf, 5 * 4 * 64 * sizeof(long long)));
    T2_CUDA(ctx, cudaMemsetAsync(trace_buf, 0, 5 * 4 * 64 * sizeof(long long), ctx->stream));
    args.trace = trace_buf;
  }
#endif
  args.n_in = (uint32_t)n_in;
  args.npeers = n_peers; args.self_rank = self_rank;
  for (int r = 0; r < 8; r++) { args.xp[r] = r < n_peers ? x_peers[r] : nullptr; args.xp_rows[r] = r < n_peers ? (uint32_t)rows_peers[r] : 0u; }
  if (n_peers == 0) { int prc = plan_table_prepare(ctx, const_cast<t2sc_plan*>(plan), n_in); if (prc != T2SC_OK) return prc; }
  args.tnbr = plan->tnbr;
  args.perm = plan->balanced ? plan->perm : nullptr;
  args.x = x; args.y = y; args.nbr = peer_nbr ? peer_nbr : plan->nbr; args.order = plan->order; args.src = plan->src;
  args.tiles = plan->tiles; args.tile_lo = tile_part(plan, part).lo; args.tile_hi = tile_part(plan, part).hi; args.status = ctx->status;
  args.Ci = Ci; args.Co = Co; args.n_cot = Co / BN; args.is_bf16 = dtype == T2SC_BF16; args.ep = ep;
  i64 max_items = plan->max_tiles * args.n_cot;
  int rc;
  if (plan->tile_rows == 2 * TILE_M)
    rc = dtype == T2SC_BF16 ? launch_t<2, __nv_bfloat16>(ctx, BN, tm, args, max_items) : launch_t<2, __half>(ctx, BN, tm, args, max_items);
  else
    rc = dtype == T2SC_BF16 ? launch_t<1, __nv_bfloat16>(ctx, BN, tm, args, max_items) : launch_t<1, __half>(ctx, BN, tm, args, max_items);
#ifdef T2SC_DIAG
  if (rc == T2SC_OK && args.trace) {        // every launch overwrites the file: the last launch of the process is what is kept
    static long long host_trace[5 * 4 * 64];
    T2_CUDA(ctx, cudaMemcpyAsync(host_trace, args.trace, sizeof(host_trace), cudaMemcpyDeviceToHost, ctx->stream));
    T2_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (FILE* f = fopen(getenv("T2SC_TRACE"), "wb")) { fwrite(host_trace, 1, sizeof(host_trace), f); fclose(f); }
  }
#endif
  return rc;
}

// y [n,Co] = x [n,Ci] . w [Co,Ci]^T through the same kernel: no neighbour map, one "tap" whose gather reads the output
// row's own input row, weights as a [Co,1,Ci] tensor.  The fused epilogue is the conv's.
int linear_umma_launch(t2sc_ctx* ctx, const void* x, const void* w, const EpiDev& ep, void* y, int dtype, i64 n, int Ci, int Co) {
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  const int BN = pick_bn(Co);
  T2_REQ(ctx, BN > 0, "Co=%d", Co);
  T2_REQ(ctx, !ep.ln || Co == BN, "fused LayerNorm needs the whole row in one tile (Co=%d)", Co);
  EncodeTiledFn enc = encode_fn();
  if (!enc) return t2sc_fail(ctx, T2SC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap tm;
  cuuint64_t dims[3] = {(cuuint64_t)Ci, 1, (cuuint64_t)Co};
  cuuint64_t strides[2] = {(cuuint64_t)Ci * 2, (cuuint64_t)Ci * 2};
  cuuint32_t box[3] = {(cuuint32_t)KCH, 1, (cuuint32_t)BN};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult cr = enc(&tm, dtype == T2SC_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return t2sc_fail(ctx, T2SC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for weights [%d,%d]", (int)cr, Co, Ci);
  ConvArgs args;
  diag_args(args);
  args.dense_rows = (int)n; args.n_in = (uint32_t)n;
  args.npeers = 0; args.self_rank = 0;
  for (int r = 0; r < 8; r++) { args.xp[r] = nullptr; args.xp_rows[r] = 0; }
  args.tnbr = nullptr; args.nbr = nullptr; args.order = nullptr; args.src = nullptr; args.tiles = nullptr;
  args.tile_lo = nullptr; args.tile_hi = nullptr; args.status = ctx->status;
  args.x = x; args.y = y;
  args.Ci = Ci; args.Co = Co; args.n_cot = Co / BN; args.is_bf16 = dtype == T2SC_BF16; args.ep = ep;
  const i64 max_items = (i64)cdiv_i(n, TILE_M) * args.n_cot;
  return dtype == T2SC_BF16 ? launch_t<1, __nv_bfloat16>(ctx, BN, tm, args, max_items) : launch_t<1, __half>(ctx, BN, tm, args, max_items);
}
