// Shared pieces of the tcgen05 sparse-conv kernels: constants, kernel arguments, PTX wrappers, UMMA descriptors.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <cstdlib>

namespace umma {

constexpr int TILE_M = 128;
constexpr int KCH = 64;                      // channels per pipeline step = one 128-byte swizzle row
constexpr int A_BYTES = TILE_M * 128;
constexpr int NUM_PROD_THREADS = 128;
constexpr int WARP_TMA = 4, WARP_IDX = 5, WARP_MMA = 6, WARP_EPI0 = 7;
// Diagnostic build (python -m trellis2_cuda_b200.build --diag -> libt2sc_diag.so): measurement switches that disable
// parts of the kernel, per-role wait timers and a settable wait limit.  None of it exists in the shipped library:
// kDiag is a compile-time false there and every test on it folds away.
#ifdef T2SC_DIAG
constexpr bool kDiag = true;
#else
constexpr bool kDiag = false;
#endif
constexpr bool kProfileWaits = kDiag;
constexpr int IDX_SLOTS = 8;                       // index ring of the two-SM kernel: one slot per (tile, tap)
constexpr int NTAB = 2;                            // neighbour-index tables of the single-CTA kernel: one per tile in flight
constexpr uint32_t RING_ABSENT = 0x80000000u;      // index entry of an absent neighbour (row numbers are below 2^30)
// Peer-memory form: a present map entry is (owner << PEER_SHIFT) | row with owner < 8 and row < 2^28, so bit 31 stays
// free for RING_ABSENT whatever the owner.
constexpr int PEER_SHIFT = 28;
constexpr uint32_t PEER_ROW_MASK = (1u << PEER_SHIFT) - 1;
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;   // ~2 s at boost clock
constexpr int WAIT_LIMIT_SHIFT = 10;                    // the limit travels to the kernel in units of 1024 cycles
constexpr int SMEM_BUDGET = 227 * 1024;

// warps: 4 gather, weights, indices, MMA, 4 per 128-row half for the epilogue, a second index warp (each serves half the
// rows), and with two gather groups (128-row tiles) four more gather warps, which start at thread 384 = 3 x 128
__host__ __device__ constexpr int num_threads(int MH, int G = 1) { return (8 + 4 * MH + (G == 2 ? 4 : 0)) * 32; }
__host__ __device__ constexpr int warp_idx2(int MH) { return 7 + 4 * MH; }
__host__ __device__ constexpr int warp_group2(int MH) { return 8 + 4 * MH; }
__host__ __device__ constexpr int stage_bytes(int BN, int MH) { return MH * A_BYTES + BN * 128; }
// A tile's neighbour indices, [27 taps][rows], tap-major with an odd pitch: the index warps write one map row (27 taps)
// per instruction and the gather warps read 16 rows of one tap, both without bank conflicts.
__host__ __device__ constexpr int tab_pitch(int MH) { return MH * TILE_M + 1; }
__host__ __device__ constexpr int tab_words(int MH) { return 27 * tab_pitch(MH); }
// Epilogue staging behind the tables and barriers: LayerNorm gamma and beta (fp32, up to 256 columns each) and one block of up
// to 256 bias values per epilogue warp.
__host__ __device__ constexpr int epi_bytes(int MH) { return 2048 + MH * 2048 + 16; }
__host__ __device__ constexpr int aux_bytes(int MH) { return NTAB * tab_words(MH) * 4 + 1024 + epi_bytes(MH); }
__host__ __device__ constexpr int num_stages(int BN, int MH, int U = 1) {
  int s = (SMEM_BUDGET - 1024 - aux_bytes(MH)) / (U * stage_bytes(BN, MH));
#ifdef T2SC_MAX_STAGES
  if (s > T2SC_MAX_STAGES) s = T2SC_MAX_STAGES;      // measurement aid
#endif
  return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int num_acc_bufs(int BN, int MH) { return 2 * MH * BN <= 512 ? 2 : 1; }

struct ConvArgs {
  const void* x; void* y; const uint32_t* nbr; const int* order; const int* src;
  const uint32_t* tnbr;     // the plan's map in tile order, [tile][27][rows]: one bulk copy per tile (not in the peer-memory form)
  const PlanTile* tiles; const int* tile_lo; const int* tile_hi; int* status;      // this launch covers tiles [*tile_lo, *tile_hi)
  const int* perm;          // the plan's tiles of each part by falling tap count (positions -> tile numbers), or null: plan order
  int Ci, Co, n_cot, is_bf16;
  int npeers, self_rank;    // npeers > 0: map entries are (owner << PEER_SHIFT) | row and rows are read from xp[owner]; xp[self_rank] is local
  const void* xp[8];
  uint32_t n_in;            // rows of x (PEERS: unused, see xp_rows); a map entry at or above it is reported and read as absent
  uint32_t xp_rows[8];      // PEERS: rows of every peer's array
  int dense_rows;           // > 0: no neighbour map at all - a plain row-major GEMM over this many rows (t2sc_linear): tile t is rows
                            // [t * tile rows, ...), its one "tap" reads input row = output row, weights are [Co, 1, Ci]
  long long* trace;         // diagnostic build only (T2SC_TRACE=file): per-tile timestamps of CTA 0's roles, [role][event][tile < 64]
  int wait_limit;           // bounded waits give up after this many cycles >> WAIT_LIMIT_SHIFT
  int dbg_skip;             // diagnostic build only (T2SC_DEBUG_SKIP), always 0 in the shipped library: 1 = no A gather, 2 = no B load,
                            // 4 = no MMA, 8 = CTA 0 prints where each role waited, 16 = the weight lane never signals its first stage,
                            // 32 = no neighbour-index loads, 64 = no epilogue
  EpiDev ep;
};

__device__ __forceinline__ bool diag(const ConvArgs& a, int bits) { return kDiag && (a.dbg_skip & bits) != 0; }
// diagnostic build: timestamp of event `ev` (0..3) of role `role` (0 gather, 1 weights, 2 index, 3 MMA, 4 epilogue) at the
// CTA's `tile`-th tile, CTA 0 only
__device__ __forceinline__ void trace(const ConvArgs& a, int role, int ev, uint32_t tile) {
  if (kDiag && a.trace && blockIdx.x == 0 && tile < 64) a.trace[(role * 4 + ev) * 64 + tile] = clock64();
}
// Host side: the shipped library always runs with no switch set and the full wait limit; the diagnostic build reads
// T2SC_DEBUG_SKIP (bit mask above) and T2SC_WAIT_LIMIT_CYCLES from the environment.
static inline void diag_args(ConvArgs& args) {
  args.dbg_skip = 0;
  args.trace = nullptr;
  args.dense_rows = 0;
  args.perm = nullptr;
  args.wait_limit = (int)(WAIT_LIMIT_CYCLES >> WAIT_LIMIT_SHIFT);
#ifdef T2SC_DIAG
  static const int dbg_skip = [] { const char* e = getenv("T2SC_DEBUG_SKIP"); return e ? atoi(e) : 0; }();
  static const long long limit = [] { const char* e = getenv("T2SC_WAIT_LIMIT_CYCLES"); return e ? atoll(e) : WAIT_LIMIT_CYCLES; }();
  args.dbg_skip = dbg_skip;
  args.wait_limit = (int)((limit >> WAIT_LIMIT_SHIFT) > 0 ? (limit >> WAIT_LIMIT_SHIFT) : 1);
#endif
}

// ------------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
#ifndef T2SC_WAIT_HINT_NS
#define T2SC_WAIT_HINT_NS 2000
#endif
// The same with a suspend-time hint: the thread sleeps in hardware until the phase completes or the hint runs out, so a
// long wait does not keep re-issuing polls that compete with the working warps for issue slots and the shared-memory path.
__device__ __forceinline__ bool mbar_try_sleep(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"((uint32_t)T2SC_WAIT_HINT_NS) : "memory");
  return ok != 0;
}
// Bounded wait.  After any wait in the CTA has given up, all later waits return at once.
// Returns false when the wait was given up (now, or earlier by any thread of the CTA): what the barrier guards has then
// NOT happened, and the caller must not touch memory whose address depends on it.
// abort_flag[0] is the CTA's "a wait gave up" flag, abort_flag[1] the limit in units of 2^WAIT_LIMIT_SHIFT cycles.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (abort_flag[0] || clock64() - t0 > ((long long)abort_flag[1] << WAIT_LIMIT_SHIFT)) { abort_flag[0] = 1; atomicOr(status, code); return false; }
#if T2SC_WAIT_HINT_NS > 0
    if (mbar_try_sleep(bar, parity)) return true;
#else
    if (mbar_try(bar, parity)) return true;
#endif
  }
}
// diagnostic build: waits that also add their duration to a per-role counter
__device__ __forceinline__ bool mbar_wait_t(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code, bool prof, long long& acc) {
  if (!prof) return mbar_wait(bar, parity, abort_flag, status, code);
  long long t0 = clock64();
  const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
  acc += clock64() - t0;
  return ok;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// arrive on `bar` once all cp.async issued so far by this thread have landed (pending count +1 now, -1 then)
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// the arrival itself, delivered once all cp.async issued so far by this thread have landed
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// untiled bulk copy global -> shared, completion counted in bytes on `bar`; addresses and size multiples of 16
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The four K = 16 MMAs of one 64-channel unit as ONE instruction block: the operand descriptors of steps 1..3 are the
// step-0 descriptors + 32, 64, 96 bytes along K (+2, +4, +6 in the address field, which sits in the low word and cannot
// carry out of it), only step 0 can be the tile's first MMA (accumulate = 0 overwrites the accumulator).  The MMA lane
// runs about one instruction per ten clocks, so the descriptor arithmetic is kept to one add per operand and step.
__device__ __forceinline__ void tc_mma_k64(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p, t;\n\t.reg .b32 al, ah, bl, bh, x;\n\t.reg .b64 a, b;\n\t"
               "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, %4, %4;\n\t"
               "mov.b64 {al, ah}, %1;\n\tmov.b64 {bl, bh}, %2;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "add.u32 x, al, 2;\n\tmov.b64 a, {x, ah};\n\tadd.u32 x, bl, 2;\n\tmov.b64 b, {x, bh};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
               "add.u32 x, al, 4;\n\tmov.b64 a, {x, ah};\n\tadd.u32 x, bl, 4;\n\tmov.b64 b, {x, bh};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
               "add.u32 x, al, 6;\n\tmov.b64 a, {x, ah};\n\tadd.u32 x, bl, 6;\n\tmov.b64 b, {x, bh};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile, rows of 128 bytes, 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address
  d |= (uint64_t)1 << 16;                      // leading byte offset: unused with swizzled K-major, set to 1
  d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                      // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                      // 128-byte swizzle
  return d;
}
__host__ __device__ constexpr uint32_t umma_idesc(int N, int is_bf16) {
  return (1u << 4)                              // D = fp32
       | ((is_bf16 ? 1u : 0u) << 7)             // A format
       | ((is_bf16 ? 1u : 0u) << 10)            // B format
       | ((uint32_t)(N >> 3) << 17)             // N
       | ((uint32_t)(TILE_M >> 4) << 24);       // M
}

template <class T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h);
}
template <class T> __device__ __forceinline__ float2 unpack2(uint32_t v);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t v) { return __half22float2(*reinterpret_cast<__half2*>(&v)); }
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v)); }


// The epilogue keeps a 32-column block of a row as 16 packed pairs of the storage type between its ops: an op unpacks
// (shifts), computes in fp32 and packs again (ONE conversion per pair), which is the storage rounding the reference's
// separate kernels apply after every op, and the block is stored as it stands.
template <class T>
__device__ __forceinline__ void add_packed32(uint32_t* hp, const uint4* src) {       // hp += 32 values of the storage type at src (16-byte aligned)
#pragma unroll
  for (int g = 0; g < 4; g++) {
    const uint4 bv = src[g]; const uint32_t* w32 = (const uint32_t*)&bv;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 f = unpack2<T>(w32[e]), h = unpack2<T>(hp[g * 4 + e]);
      hp[g * 4 + e] = pack2<T>(h.x + f.x, h.y + f.y);
    }
  }
}

// Fused epilogue of one output row (this thread's TMEM lane) over the BN accumulator columns at `taddr`, in 32-column blocks:
// round -> + bias -> LayerNorm -> activation -> + residual -> + skip, each rounded to the storage type, then stores.
// All lanes of the warp must call it (tcgen05.ld is warp-collective); orow < 0 loads but does not store.
// bias points at the item's first column (or is null); gamma / beta at the row's first column (LayerNorm only, may be null).
// The kernels hand in copies in shared memory: a per-element load from global memory here costs its full latency once per
// block, because one epilogue warp per scheduler has nothing else to run meanwhile.
template <int BN, class T>
__device__ __forceinline__ void epilogue_row(const ConvArgs& a, uint32_t taddr, int orow, int cot, const T* bias, const float* gamma, const float* beta, int sp, int ss) {
  T* y = (T*)a.y;
  const T* res = (const T*)a.ep.residual; const T* skx = (const T*)a.ep.skip_x;
  float mean = 0.f, rstd = 1.f;
  if (a.ep.ln) {      // whole row lives in this accumulator (n_cot == 1)
    // ONE statistics pass over TMEM (every tcgen05.ld round trip counts: at Co <= 128 the epilogue is as long as the tile's
    // MMAs): sums of (h - K) and (h - K)^2 with K = the row's first value, so that mean = K + S1/n and var = S2/n - (S1/n)^2
    // lose nothing to cancellation that matters beside the storage rounding of the result.
    float s1 = 0.f, s2 = 0.f, K = 0.f;
    for (int cc = 0; cc < BN / 32; cc++) {
      uint32_t r[32]; tc_ld32(taddr + cc * 32, r); tc_wait_ld();
      uint32_t hp[16];
#pragma unroll
      for (int i = 0; i < 16; i++) hp[i] = pack2<T>(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      if (bias) add_packed32<T>(hp, (const uint4*)(bias + cc * 32));
      if (cc == 0) K = unpack2<T>(hp[0]).x;
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const float2 h = unpack2<T>(hp[i]);
        const float d0 = h.x - K, d1 = h.y - K;
        s1 += d0 + d1; s2 = fmaf(d0, d0, fmaf(d1, d1, s2));
      }
    }
    const float m1 = s1 / (float)BN;
    mean = K + m1;
    rstd = rsqrtf(fmaxf(s2 / (float)BN - m1 * m1, 0.f) + a.ep.eps);
  }
  // The residual row is read one 32-column block ahead: a block's four 16-byte loads are in flight while the block
  // before it is converted and stored, instead of a load latency per block.
  const uint4* rp = res && orow >= 0 ? (const uint4*)(res + (i64)orow * a.Co + cot * BN) : nullptr;
  uint4 rnext[4];
  if (rp) {
#pragma unroll
    for (int g = 0; g < 4; g++) rnext[g] = __ldg(rp + g);
  }
  for (int cc = 0; cc < BN / 32; cc++) {
    uint32_t r[32]; tc_ld32(taddr + cc * 32, r);
    uint4 rcur[4];
    if (rp) {
#pragma unroll
      for (int g = 0; g < 4; g++) rcur[g] = rnext[g];
      if (cc + 1 < BN / 32) {
#pragma unroll
        for (int g = 0; g < 4; g++) rnext[g] = __ldg(rp + (cc + 1) * 4 + g);
      }
    }
    tc_wait_ld();
    if (orow < 0) continue;
    const int col = cot * BN + cc * 32;
    uint32_t hp[16];
#pragma unroll
    for (int i = 0; i < 16; i++) hp[i] = pack2<T>(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    if (bias) add_packed32<T>(hp, (const uint4*)(bias + cc * 32));
    if (a.ep.ln) {
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const float2 h = unpack2<T>(hp[i]);
        float v0 = rstd * (h.x - mean), v1 = rstd * (h.y - mean);
        if (gamma) { v0 *= gamma[cc * 32 + 2 * i]; v1 *= gamma[cc * 32 + 2 * i + 1]; }
        if (beta) { v0 += beta[cc * 32 + 2 * i]; v1 += beta[cc * 32 + 2 * i + 1]; }
        hp[i] = pack2<T>(v0, v1);
      }
    }
    if (a.ep.act == T2SC_ACT_SILU) {          // one branch per block, not per element
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const float2 h = unpack2<T>(hp[i]);
        hp[i] = pack2<T>(__fdividef(h.x, 1.f + __expf(-h.x)), __fdividef(h.y, 1.f + __expf(-h.y)));
      }
    } else if (a.ep.act) {
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const float2 h = unpack2<T>(hp[i]);
        hp[i] = pack2<T>(act_apply(h.x, a.ep.act), act_apply(h.y, a.ep.act));
      }
    }
    if (rp) add_packed32<T>(hp, rcur);
    if (skx) {
      const T* sx = skx + (i64)sp * a.ep.skip_cin + ss * (a.ep.skip_cin / 8);
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const float2 h = unpack2<T>(hp[i]);
        hp[i] = pack2<T>(h.x + to_f<T>(sx[(col + 2 * i) / a.ep.skip_rep]), h.y + to_f<T>(sx[(col + 2 * i + 1) / a.ep.skip_rep]));
      }
    }
    // the block's 64 bytes as two 32-byte stores (whole sectors) when the row allows it, else four 16-byte ones
    T* const yb = y + (i64)orow * a.Co + col;
    if (((uintptr_t)yb & 31) == 0) {
#pragma unroll
      for (int g = 0; g < 2; g++)
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(yb + g * 16), "r"(hp[g * 8]), "r"(hp[g * 8 + 1]), "r"(hp[g * 8 + 2]),
                     "r"(hp[g * 8 + 3]), "r"(hp[g * 8 + 4]), "r"(hp[g * 8 + 5]), "r"(hp[g * 8 + 6]), "r"(hp[g * 8 + 7]) : "memory");
    } else {
      uint4* yp = (uint4*)yb;
#pragma unroll
      for (int g = 0; g < 4; g++) yp[g] = make_uint4(hp[g * 4], hp[g * 4 + 1], hp[g * 4 + 2], hp[g * 4 + 3]);
    }
  }
}

}  // namespace umma
