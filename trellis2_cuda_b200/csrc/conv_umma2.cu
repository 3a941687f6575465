// Two-SM (tcgen05 cta_group::2) variant of the masked implicit-GEMM sparse convolution, for Co % 256 == 0.
//
// Same operator as conv_umma.cu (src/spconv.cu:91-150 of trellis2-cuda).  A cluster of two CTAs on neighbouring SMs
// works on one 256-row plan tile: each CTA gathers the A rows of its own 128-row half and loads only HALF of every
// weight slab (128 of the 256 output channels); the leader CTA issues tcgen05.mma with cta_group::2 (M = 256 over
// the pair, N = 256, K = 16), which reads A from both CTAs and the two weight halves from the two CTAs, and each
// CTA's TMEM receives the accumulator of its own 128 rows.  A pipeline stage is therefore 16 KB + 16 KB instead of
// 16 KB + 32 KB: six stages fit instead of four (the single-CTA kernel starves on stage depth), and the weight
// traffic from L2 halves.
//
// Cross-CTA signalling uses only: remote mbarrier arrives (mapa), tcgen05.commit to a barrier of the peer, and two
// cluster barriers.  No TMA load here is a cluster-wide load: every CTA fetches its own bytes.
#include "umma_common.cuh"
#include <cuda_runtime.h>

namespace {
using namespace umma;

constexpr int P_WARP_TMA = 4, P_WARP_IDX = 5, P_WARP_MMA = 6, P_WARP_RELAY = 7, P_WARP_EPI0 = 8;
constexpr int P_THREADS = 12 * 32;
constexpr int P_BN = 256;                        // output channels per work item (both CTAs together)
constexpr int P_BHALF = P_BN / 2 * 128;          // bytes of this CTA's half of a weight slab
constexpr int P_STAGE = A_BYTES + P_BHALF;       // 32 KB
constexpr int P_AUX = IDX_SLOTS * TILE_M * 4 + 512;
constexpr int P_S = (SMEM_BUDGET - 1024 - P_AUX) / P_STAGE > 8 ? 8 : (SMEM_BUDGET - 1024 - P_AUX) / P_STAGE;
constexpr int P_SMEM = P_S * P_STAGE + P_AUX + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t cta) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta)); return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {      // waits for arrivals that may come from the peer CTA
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try_cluster(bar, parity)) return true;
  long long t0 = clock64();
  while (!mbar_try_cluster(bar, parity)) {
    if (abort_flag[0] || clock64() - t0 > ((long long)abort_flag[1] << WAIT_LIMIT_SHIFT)) { abort_flag[0] = 1; atomicOr(status, code); return false; }
  }
  return true;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_commit2(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_mma2(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__host__ __device__ constexpr uint32_t umma_idesc2(int is_bf16) {       // M = 256 over the CTA pair, N = 256
  return (1u << 4) | ((is_bf16 ? 1u : 0u) << 7) | ((is_bf16 ? 1u : 0u) << 10) | ((uint32_t)(P_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// Warp roles per CTA: 0-3 gather A of this CTA's 128 rows, 4 this CTA's half of the weights (TMA), 5 neighbour-index ring,
// 6 TMEM owner and (leader only) MMA issue, 7 relay (peer: "stage landed" -> leader; leader: "stage free" -> both), 8-11 epilogue.
template <class T>
__global__ void __launch_bounds__(P_THREADS, 1) k_conv_umma2(const __grid_constant__ CUtensorMap tmw, const ConvArgs a) {
  constexpr int S = P_S;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint32_t* ring = (uint32_t*)(smem + S * P_STAGE);
  uint64_t* bars = (uint64_t*)(ring + IDX_SLOTS * TILE_M);   // full[S] empty[S] pfull[S] accf[2] acce[2] iready[] ifree[]
  uint32_t* tmem_slot = (uint32_t*)(bars + 3 * S + 4 + 2 * IDX_SLOTS);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * S, bar_pfull = bar_empty + 8 * S, bar_accf = bar_pfull + 8 * S,
                 bar_acce = bar_accf + 16, bar_iready = bar_acce + 16, bar_ifree = bar_iready + 8 * IDX_SLOTS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, NUM_PROD_THREADS + 1 + (leader ? 1 : 0)); mbar_init(bar_empty + 8 * s, 1); mbar_init(bar_pfull + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(bar_accf + 8 * b, 1); mbar_init(bar_acce + 8 * b, 256); }   // both CTAs' epilogue threads
    for (int r = 0; r < IDX_SLOTS; r++) { mbar_init(bar_iready + 8 * r, 1); mbar_init(bar_ifree + 8 * r, NUM_PROD_THREADS / 32); }
    abort_flag[0] = 0; abort_flag[1] = a.wait_limit;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == P_WARP_MMA) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tile0 = *a.tile_lo, ntiles = *a.tile_hi - tile0;
  const PlanTile* const tiles = a.tiles + tile0;
  const int nitems = ntiles * a.n_cot;
  const int nchunk = a.Ci / KCH;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int row0 = rank * TILE_M;                   // this CTA's rows inside the 256-row tile

  if (warp < 4) {
    // ===================================================================== A producer
    const T* x = (const T*)a.x;
    const int t = threadIdx.x, jbase = t >> 3, c16 = t & 7;
    const uint32_t dst_thread = (uint32_t)(jbase * 128 + ((c16 ^ (jbase & 7)) << 4));
    uint32_t it = 0, iit = 0;
    bool alive = true;        // false once a wait was given up: the index ring may then hold anything, so no more loads
    const bool prof = diag(a, 8); long long w_empty = 0, w_idx = 0, t_role = clock64();
    for (int item = pair; item < nitems; item += npairs) {
      const PlanTile tile = tiles[item / a.n_cot];
      for (uint32_t mk = tile.mask; mk; mk &= mk - 1, iit++) {
        const uint32_t slot = iit % IDX_SLOTS, iph = (iit / IDX_SLOTS) & 1;
        { long long t0 = clock64(); alive &= mbar_wait(bar_iready + 8 * slot, iph, abort_flag, a.status, 32); if (prof) w_idx += clock64() - t0; }
        uint32_t idx[8];
#pragma unroll
        for (int i = 0; i < 8; i++) idx[i] = ring[slot * TILE_M + jbase + 16 * i];
        __syncwarp();
        if (lane == 0 && alive) mbar_arrive(bar_ifree + 8 * slot);       // one arrival per gather warp: arrivals on one barrier serialise
        for (int c = 0; c < nchunk; c++, it++) {
          const uint32_t s = it % S, ph = (it / S) & 1;
          { long long t0 = clock64(); alive &= mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, a.status, 1); if (prof) w_empty += clock64() - t0; }
          const uint32_t dst = smem_base + s * P_STAGE + dst_thread;
          const T* xs = x + c * KCH + c16 * 8;
          if (!alive) continue;       // after a wait was given up: no more loads, no more arrivals
          if (!diag(a, 1)) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const bool present = idx[i] != NBR_EMPTY;
              cp_async16(dst + i * (16 * 128), present ? (const void*)(xs + (i64)idx[i] * a.Ci) : (const void*)x, present ? 16u : 0u);
            }
          }
          cp_async_arrive_noinc(bar_full + 8 * s);
        }
      }
    }
    cp_async_wait_all();
    if (prof && blockIdx.x < 2 && threadIdx.x == 0)
      printf("[t2sc prof pair] gather rank %u: total %lld clk, wait stage free %lld, wait index ring %lld, steps %u\n", rank, clock64() - t_role, w_empty, w_idx, it);
  } else if (warp == P_WARP_TMA) {
    // ===================================================================== this CTA's half of every weight slab
    uint32_t it = 0;
    for (int item = pair; item < nitems; item += npairs) {
      const int tile_id = item / a.n_cot, cot = item - tile_id * a.n_cot;
      const PlanTile tile = tiles[tile_id];
      const int wrow = tile.wbase * a.Co + cot * P_BN + rank * (P_BN / 2);
      for (uint32_t mk = tile.mask; mk; mk &= mk - 1) {
        const int v = __ffs(mk) - 1;
        for (int c = 0; c < nchunk; c++, it++) {
          const uint32_t s = it % S, ph = (it / S) & 1;
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, a.status, 2))) goto tma_done;
          if (lane == 0) {
            if (diag(a, 2)) mbar_arrive(bar_full + 8 * s);
            else {
              mbar_arrive_expect_tx(bar_full + 8 * s, P_BHALF);
              tma_load_3d(smem_base + s * P_STAGE + A_BYTES, &tmw, c * KCH, v, wrow, bar_full + 8 * s);
            }
          }
          __syncwarp();
        }
      }
    }
  tma_done:;
  } else if (warp == P_WARP_IDX) {
    // ===================================================================== neighbour indices of this CTA's rows
    uint32_t iit = 0;
    bool oob = false;         // a present map entry at or past the end of x: read as absent and reported
    for (int item = pair; item < nitems; item += npairs) {
      const PlanTile tile = tiles[item / a.n_cot];
      int nr[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int j = row0 + lane + 32 * i;
        nr[i] = -1;
        if (j < tile.rows) { const int r = a.order[tile.start + j]; nr[i] = a.src ? (a.src[r] >> 3) : r; }
      }
      for (uint32_t mk = tile.mask; mk; mk &= mk - 1, iit++) {
        const int v = __ffs(mk) - 1;
        const uint32_t slot = iit % IDX_SLOTS, iph = (iit / IDX_SLOTS) & 1;
        uint32_t val[4];
#pragma unroll
        for (int i = 0; i < 4; i++) val[i] = nr[i] < 0 ? NBR_EMPTY : __ldg(a.nbr + (i64)nr[i] * 27 + v);
        if (!__all_sync(0xffffffffu, mbar_wait(bar_ifree + 8 * slot, iph ^ 1, abort_flag, a.status, 64))) goto idx_done;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          oob |= val[i] + 1u > a.n_in;                    // NBR_EMPTY + 1 wraps to 0
          ring[slot * TILE_M + lane + 32 * i] = val[i] >= a.n_in ? NBR_EMPTY : val[i];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_iready + 8 * slot);
      }
    }
  idx_done:
    if (__any_sync(0xffffffffu, oob) && lane == 0) atomicOr(a.status, 256);
  } else if (warp == P_WARP_RELAY) {
    // ===================================================================== peer: tell the leader that a stage has landed here
    if (leader) {
      // leader: one commit per stage lands on bar_pfull; pass it on as "stage free" to the producers of both CTAs
      uint32_t it = 0;
      for (int item = pair; item < nitems; item += npairs) {
        const PlanTile tile = tiles[item / a.n_cot];
        const int ksteps = __popc(tile.mask) * nchunk;
        for (int k = 0; k < ksteps; k++, it++) {
          const uint32_t s = it % S, ph = (it / S) & 1;
          if (!__all_sync(0xffffffffu, mbar_wait(bar_pfull + 8 * s, ph, abort_flag, a.status, 512))) goto relay_done;
          if (lane == 0) {
            mbar_arrive(bar_empty + 8 * s);
            asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(mapa(bar_empty + 8 * s, 1)) : "memory");
          }
          __syncwarp();
        }
      }
    } else {
      uint32_t it = 0;
      const bool prof = diag(a, 8); long long w_f = 0, t_role = clock64();
      for (int item = pair; item < nitems; item += npairs) {
        const PlanTile tile = tiles[item / a.n_cot];
        const int ksteps = __popc(tile.mask) * nchunk;
        for (int k = 0; k < ksteps; k++, it++) {
          const uint32_t s = it % S, ph = (it / S) & 1;
          { long long t0 = clock64(); const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status, 128)); if (prof) w_f += clock64() - t0;
            if (!ok) goto relay_done; }
          // relaxed: the leader never reads this CTA's shared memory with loads; with cta_group::2 each SM's tensor core
          // reads its own shared memory, so only the timing has to cross (a release at cluster scope costs ~900 clk here)
          if (lane == 0) asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(mapa(bar_full + 8 * s, 0)) : "memory");
          __syncwarp();
        }
      }
      if (prof && blockIdx.x == 1 && lane == 0) printf("[t2sc prof pair] relay: total %lld clk, wait local stage %lld, steps %u\n", clock64() - t_role, w_f, it);
    }
  relay_done:;
  } else if (warp == P_WARP_MMA) {
    // ===================================================================== leader: MMA issue for the pair
    if (leader) {
      const uint32_t idesc = umma_idesc2(a.is_bf16);
      uint32_t it = 0, acc_it = 0;
      const bool prof = diag(a, 8); long long w_full = 0, w_pfull = 0, w_acc = 0, t_role = clock64();
      for (int item = pair; item < nitems; item += npairs, acc_it++) {
        const PlanTile tile = tiles[item / a.n_cot];
        const uint32_t buf = acc_it & 1, aph = (acc_it >> 1) & 1;
        { long long t0 = clock64(); const bool ok = __all_sync(0xffffffffu, mbar_wait_cluster(bar_acce + 8 * buf, aph ^ 1, abort_flag, a.status, 4)); if (prof) w_acc += clock64() - t0;
          if (!ok) goto mma_done; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * P_BN;
        const int ksteps = __popc(tile.mask) * nchunk;
        for (int k = 0; k < ksteps; k++, it++) {
          const uint32_t s = it % S, ph = (it / S) & 1;
          { long long t0 = clock64(); const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, abort_flag, a.status, 8)); if (prof) w_full += clock64() - t0;
            if (!ok) goto mma_done; }
          tc_fence_after();
          if (lane == 0) {
            const uint64_t ad = umma_desc(smem_base + s * P_STAGE), bd = umma_desc(smem_base + s * P_STAGE + A_BYTES);
#pragma unroll
            for (int kk = 0; kk < KCH / 16 && !diag(a, 4); kk++) tc_mma2(d_tmem, ad + 2 * kk, bd + 2 * kk, idesc, (k > 0 || kk > 0) ? 1u : 0u);
            tc_commit2(bar_pfull + 8 * s);                    // "MMAs of this stage are done": the relay warp frees the stage in both CTAs
          }
          __syncwarp();
        }
        if (lane == 0) { tc_commit2(bar_accf + 8 * buf); tc_commit2(mapa(bar_accf + 8 * buf, 1)); }
        __syncwarp();
      }
      if (prof && blockIdx.x == 0 && lane == 0)
        printf("[t2sc prof pair] leader mma: total %lld clk, wait own stage %lld, wait peer stage %lld, wait accumulators %lld, steps %u\n",
               clock64() - t_role, w_full, w_pfull, w_acc, it);
    }
  mma_done:;
  } else {
    // ===================================================================== epilogue of this CTA's 128 rows
    const bool has_skip = a.ep.skip_x != nullptr;
    const int q = warp & 3, j = row0 + q * 32 + lane;
    const uint32_t acce_leader = mapa(bar_acce, 0);
    uint32_t acc_it = 0;
    for (int item = pair; item < nitems; item += npairs, acc_it++) {
      const int tile_id = item / a.n_cot, cot = item - tile_id * a.n_cot;
      const PlanTile tile = tiles[tile_id];
      const uint32_t buf = acc_it & 1, aph = (acc_it >> 1) & 1;
      const int orow = j < tile.rows ? a.order[tile.start + j] : -1;
      const int wcol0 = tile.wbase * a.Co + cot * P_BN;
      int sp = 0, ss = 0;
      if (has_skip && orow >= 0) { int sv = a.ep.skip_src[orow]; sp = sv >> 3; ss = sv & 7; }
      if (!__all_sync(0xffffffffu, mbar_wait_cluster(bar_accf + 8 * buf, aph, abort_flag, a.status, 16))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * P_BN;
      epilogue_row<P_BN, T>(a, taddr, orow, cot, a.ep.bias ? (const T*)a.ep.bias + wcol0 : nullptr, a.ep.gamma, a.ep.beta, sp, ss);
      tc_fence_before();
      mbar_arrive_cluster(acce_leader + 8 * buf);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {}
    __syncthreads();
  }
  cluster_sync_all();                               // neither CTA frees TMEM or leaves while the other may still signal it
  if (warp == P_WARP_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

bool conv_umma2_supported(const t2sc_plan* plan, int dtype, int Ci, int Co, const EpiDev& ep) {
  return plan->tile_rows == 256 && (dtype == T2SC_F16 || dtype == T2SC_BF16) && Ci % KCH == 0 && Co % P_BN == 0 && (!ep.ln || Co == P_BN);
}

int conv_umma2_launch(t2sc_ctx* ctx, const t2sc_plan* plan, const void* x, const void* w, i64 w_rows, const EpiDev& ep, void* y,
                      int dtype, i64 n_in, int Ci, int Co, int part) {
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  static EncodeTiledFn2 enc = [] {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return (EncodeTiledFn2)p;
  }();
  if (!enc) return t2sc_fail(ctx, T2SC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap tm;
  cuuint64_t dims[3] = {(cuuint64_t)Ci, 27, (cuuint64_t)w_rows};
  cuuint64_t strides[2] = {(cuuint64_t)Ci * 2, (cuuint64_t)Ci * 2 * 27};
  cuuint32_t box[3] = {(cuuint32_t)KCH, 1, (cuuint32_t)(P_BN / 2)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult cr = enc(&tm, dtype == T2SC_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return t2sc_fail(ctx, T2SC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)cr);
  ConvArgs args;
  args.tnbr = nullptr;
  args.x = x; args.y = y; args.nbr = plan->nbr; args.order = plan->order; args.src = plan->src;
  args.tiles = plan->tiles; args.tile_lo = tile_part(plan, part).lo; args.tile_hi = tile_part(plan, part).hi; args.status = ctx->status;
  args.Ci = Ci; args.Co = Co; args.n_cot = Co / P_BN; args.is_bf16 = dtype == T2SC_BF16; args.ep = ep; args.npeers = 0;
  diag_args(args);
  args.n_in = (uint32_t)n_in;
  const i64 max_items = plan->max_tiles * args.n_cot;
  int pairs = (int)(max_items < ctx->num_sms / 2 ? max_items : ctx->num_sms / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(P_THREADS); cfg.dynamicSmemBytes = P_SMEM; cfg.stream = ctx->stream;
  cudaLaunchAttribute attr; attr.id = cudaLaunchAttributeClusterDimension; attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  // A persistent grid must be co-resident: not every SM can be paired (GPCs with an odd number of usable SMs), so ask
  // how many 2-CTA clusters fit at once and launch no more than that.
  static int max_clusters[16][2] = {};
  int& mc = max_clusters[ctx->device & 15][dtype == T2SC_BF16];
  if (dtype == T2SC_BF16) T2_CUDA(ctx, cudaFuncSetAttribute(k_conv_umma2<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
  else T2_CUDA(ctx, cudaFuncSetAttribute(k_conv_umma2<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
  if (mc == 0) {
    cfg.gridDim = dim3(2 * (ctx->num_sms / 2));
    if (dtype == T2SC_BF16) T2_CUDA(ctx, cudaOccupancyMaxActiveClusters(&mc, k_conv_umma2<__nv_bfloat16>, &cfg));
    else T2_CUDA(ctx, cudaOccupancyMaxActiveClusters(&mc, k_conv_umma2<__half>, &cfg));
    if (mc < 1) return t2sc_fail(ctx, T2SC_ERR_UNSUPPORTED, "no 2-CTA cluster of the pair kernel fits on this device");
  }
  if (pairs > mc) pairs = mc;
  cfg.gridDim = dim3(2 * pairs);
  if (dtype == T2SC_BF16) T2_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_conv_umma2<__nv_bfloat16>, tm, args));
  else T2_CUDA(ctx, cudaLaunchKernelEx(&cfg, k_conv_umma2<__half>, tm, args));
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}
