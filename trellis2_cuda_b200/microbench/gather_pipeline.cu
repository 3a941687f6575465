// Gather pipeline microbenchmark: the conv kernel's producer/consumer stage pipeline without the tensor core.
// Build and run: make -C trellis2_cuda_b200/microbench gather_pipeline && trellis2_cuda_b200/microbench/gather_pipeline
// 128 gather threads fill stages of ROWS x 128 B; one consumer warp waits "full", spins `delay` clocks, arrives "empty".
// MODE 0: full = cp.async.mbarrier.arrive.noinc per thread (count 128)
// MODE 1: full = commit_group / wait_group<LAG> + fence.proxy.async + one arrive per warp (count 4), signalled at the top of a later iteration
// MODE 2: as 0 without the copies (skeleton);  MODE 3: as 1 without the copies
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cstdint>
#define CK(x) do { cudaError_t e=(x); if(e!=cudaSuccess){printf("CUDA %s: %s\n",#x,cudaGetErrorString(e)); exit(1);} } while(0)
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, uint32_t n) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(n) : "memory"); }
__device__ __forceinline__ void cp16p(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template<int N> __device__ __forceinline__ void waitg() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t c) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(c) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ void arrive_noinc(uint32_t bar) { asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  long long t0 = clock64();
  while (!mbar_try(bar, parity)) if (clock64() - t0 > 2000000000ll) return false;
  return true;
}

template<int MODE, int S, int LAG, int ROWS, int ZF = 1, int GT = 128>
__global__ void __launch_bounds__(GT + 32, 1) k_pipe(const uint4* __restrict__ x, const int* __restrict__ idx, int stages_total, int row_vec, int nidx, int delay, int chunks, unsigned long long* sink) {
  extern __shared__ uint4 sm[];
  constexpr int PER = ROWS / (GT / 8), RSTEP = GT / 8;
  int* sidx = (int*)(sm + S * ROWS * 8);
  uint64_t* bars = (uint64_t*)(sidx + nidx);
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  for (int i = t; i < nidx; i += blockDim.x) sidx[i] = idx[(size_t)blockIdx.x * nidx + i];
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(sm), bfull = (uint32_t)__cvta_generic_to_shared(bars), bempty = bfull + 8 * S;
  constexpr bool GROUPS = (MODE == 1 || MODE == 3), COPY = (MODE < 2 || MODE >= 4), FREE = (MODE >= 4 && MODE != 7);   // MODE 4: no back-pressure, noinc arrivals; 5: no back-pressure, commit + wait_group<3>; 6: copies only
  if (t == 0) {
    for (int s = 0; s < S; s++) { mbar_init(bfull + 8 * s, GROUPS ? GT / 32 : GT); mbar_init(bempty + 8 * s, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool ok = true;
  if (warp < GT / 32) {
    const int c16 = t & 7, jb = t >> 3;
    const uint32_t dst_thread = jb * 128 + ((c16 ^ (jb & 7)) << 4);
    int r[PER];
    long long tw = 0, ti = 0, ta = 0, tl = 0, tt0 = clock64();
    for (int it = 0; it < stages_total && ok; it++) {
      const int c = it % chunks;
      if (c == 0) {
        const int* ip = sidx + (((it / chunks) * ROWS) % nidx);
#pragma unroll
        for (int i = 0; i < PER; i++) r[i] = ip[jb + RSTEP * i];
      }
      if (GROUPS && it >= LAG) {            // stage it-LAG has landed: publish it
        waitg<LAG - 1>();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bfull + 8 * ((it - LAG) % S));
      }
      const int st = it % S;
      long long c0 = clock64();
      if (MODE == 7) { if (it >= S) ok = mbar_wait(bfull + 8 * st, ((it / S) & 1) ^ 1); } else if (!FREE) ok = mbar_wait(bempty + 8 * st, ((it / S) & 1) ^ 1);
      const uint32_t dst = sbase + st * ROWS * 128 + dst_thread;
      const uint4* xs = x + c16 + c * 8;
      long long c1 = clock64();
      if (COPY) {
#pragma unroll
        for (int i = 0; i < PER; i++) { const bool p = r[i] >= 0;
          if (ZF == 1) cp16(dst + i * RSTEP * 128, p ? (const void*)(xs + (size_t)r[i] * row_vec) : (const void*)x, p ? 16u : 0u);
          else if (ZF == 0) cp16p(dst + i * RSTEP * 128, p ? (const void*)(xs + (size_t)r[i] * row_vec) : (const void*)(x + c16));
          else if (p) cp16p(dst + i * RSTEP * 128, (const void*)(xs + (size_t)r[i] * row_vec)); }
      }
      long long c2 = clock64();
      if (MODE == 5) { commit(); waitg<3>(); } else if (MODE == 6) {} else if (GROUPS) commit(); else arrive_noinc(bfull + 8 * st);
      long long c3 = clock64();
      tw += c1 - c0; ti += c2 - c1; ta += c3 - c2;
    }
    if (blockIdx.x == 0 && t == 0 && sink[2]) printf("    warp0: per stage: wait %lld issue %lld arrive %lld total %lld\n", tw / stages_total, ti / stages_total, ta / stages_total, (clock64() - tt0) / stages_total);
    if (GROUPS) {
      waitg<0>();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      for (int it = stages_total - LAG; it < stages_total; it++) if (it >= 0 && lane == 0) mbar_arrive(bfull + 8 * (it % S));
    }
    waitg<0>();
  } else {
    for (int it = 0; it < stages_total && ok && MODE != 5 && MODE != 6 && MODE != 7; it++) {
      const int st = it % S;
      ok = mbar_wait(bfull + 8 * st, (it / S) & 1);
      if (delay) { long long t0 = clock64(); while (clock64() - t0 < delay) {} }
      __syncwarp();
      if (lane == 0) mbar_arrive(bempty + 8 * st);
    }
  }
  if (!ok) sink[1] = 1;
  __syncthreads();
  if (sm[t].x == 0x1234567) sink[0] = 1;
}

// Groups of gather warps fill ALTERNATE stages (group g takes stages it % G == g), so one group's handshake and index
// loads overlap the other groups' copies instead of every gather warp idling at the same moment.
template<int S, int ROWS, int GT, int G>
__global__ void __launch_bounds__(GT + 32, 1) k_pipe2(const uint4* __restrict__ x, const int* __restrict__ idx, int stages_total, int row_vec, int nidx, int delay, int chunks, unsigned long long* sink) {
  extern __shared__ uint4 sm[];
  constexpr int GS = GT / G, RSTEP = GS / 8, PER = ROWS / RSTEP;
  int* sidx = (int*)(sm + S * ROWS * 8);
  uint64_t* bars = (uint64_t*)(sidx + nidx);
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  for (int i = t; i < nidx; i += blockDim.x) sidx[i] = idx[(size_t)blockIdx.x * nidx + i];
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(sm), bfull = (uint32_t)__cvta_generic_to_shared(bars), bempty = bfull + 8 * S;
  if (t == 0) {
    for (int s = 0; s < S; s++) { mbar_init(bfull + 8 * s, GS); mbar_init(bempty + 8 * s, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool ok = true;
  if (warp < GT / 32) {
    const int g = t / GS, tg = t % GS, c16 = tg & 7, jb = tg >> 3;
    const uint32_t dst_thread = jb * 128 + ((c16 ^ (jb & 7)) << 4);
    long long tw = 0, ti = 0, ta = 0, tt0 = clock64(); int ns = 0;
    for (int it = g; it < stages_total && ok; it += G, ns++) {
      const int c = it % chunks;
      const int* ip = sidx + (((it / chunks) * ROWS) % nidx);
      const int st = it % S;
      long long c0 = clock64();
      ok = mbar_wait(bempty + 8 * st, ((it / S) & 1) ^ 1);
      const uint32_t dst = sbase + st * ROWS * 128 + dst_thread;
      const uint4* xs = x + c16 + c * 8;
      long long c1 = clock64();
#pragma unroll
      for (int i0 = 0; i0 < PER; i0 += 16) {
        int r[16];
#pragma unroll
        for (int i = 0; i < 16; i++) r[i] = ip[jb + RSTEP * (i0 + i)];
#pragma unroll
        for (int i = 0; i < 16; i++) { const bool p = r[i] >= 0; cp16(dst + (i0 + i) * RSTEP * 128, p ? (const void*)(xs + (size_t)r[i] * row_vec) : (const void*)x, p ? 16u : 0u); }
      }
      long long c2 = clock64();
      arrive_noinc(bfull + 8 * st);
      tw += c1 - c0; ti += c2 - c1; ta += clock64() - c2;
    }
    if (blockIdx.x == 0 && t == 0 && sink[2]) printf("    warp0: per own stage: wait %lld issue %lld arrive %lld total %lld\n", tw / ns, ti / ns, ta / ns, (clock64() - tt0) / ns);
    waitg<0>();
  } else {
    for (int it = 0; it < stages_total && ok; it++) {
      const int st = it % S;
      ok = mbar_wait(bfull + 8 * st, (it / S) & 1);
      if (delay) { long long t0 = clock64(); while (clock64() - t0 < delay) {} }
      __syncwarp();
      if (lane == 0) mbar_arrive(bempty + 8 * st);
    }
  }
  if (!ok) sink[1] = 1;
  __syncthreads();
  if (sm[t].x == 0x1234567) sink[0] = 1;
}

int main() {
  int nrows = 217821, row_bytes = 512, stages = 4000, nsm = 148, nidx = 8192;
  size_t xbytes = (size_t)nrows * row_bytes;
  uint4* x; CK(cudaMalloc(&x, xbytes)); CK(cudaMemset(x, 1, xbytes));
  unsigned long long* sink; CK(cudaMalloc(&sink, 32)); CK(cudaMemset(sink, 0, 32)); { unsigned long long one = 1; CK(cudaMemcpy(sink + 2, &one, 8, cudaMemcpyHostToDevice)); }
  std::vector<int> h((size_t)nsm * nidx); srand(1);
  for (int b = 0; b < nsm; b++) for (int i = 0; i < nidx; i++) {
    int base = (int)(((long long)b * nrows) / nsm);
    h[(size_t)b * nidx + i] = (rand() % 10 == 0) ? -1 : (base + rand() % 4096) % nrows;
  }
  int* idx; CK(cudaMalloc(&idx, h.size() * 4)); CK(cudaMemcpy(idx, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  auto run = [&](const char* name, auto kern, int S, int rows, int delay, int chunks, int T = 160) {
    int smem = S * rows * 128 + nidx * 4 + 2 * S * 8 + 64;
    CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    float ms = 0;
    for (int rep = 0; rep < 2; rep++) {
      cudaEventRecord(e0);
      kern<<<nsm, T, smem>>>(x, idx, stages, row_bytes / 16, nidx, delay, chunks, sink);
      cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms, e0, e1);
    }
    double bytes = (double)nsm * stages * rows * 128;
    printf("%-28s S=%d rows=%3d delay=%4d chunks=%d: %.3f ms  %6.1f GB/s/SM  %.0f clk/stage\n", name, S, rows, delay, chunks, ms, bytes / ms / 1e6 / nsm, ms * 1e-3 * 1.9e9 / stages);
  };
  for (int delay : {0, 400}) { int chunks = 2;
    run("copies only (no barriers)", k_pipe<6, 4, 1, 256, 1>, 4, 256, delay, chunks);
    run("no back-pressure, noinc arrivals", k_pipe<4, 4, 1, 256, 1>, 4, 256, delay, chunks);
    run("4 warps fill each stage together", k_pipe<0, 4, 1, 256, 1>, 4, 256, delay, chunks);
    run("4 warps fill each stage together", k_pipe<0, 6, 1, 256, 1>, 6, 256, delay, chunks);
    run("groups + wait_group, lag 3", k_pipe<1, 4, 3, 256, 1>, 4, 256, delay, chunks);
    run("2 groups x 2 warps, alternate stages", k_pipe2<4, 256, 128, 2>, 4, 256, delay, chunks);
    run("4 groups x 1 warp, alternate stages", k_pipe2<4, 256, 128, 4>, 4, 256, delay, chunks);
    run("4 groups x 1 warp, alternate stages", k_pipe2<6, 256, 128, 4>, 6, 256, delay, chunks);
    run("4 warps together, 128-row stages", k_pipe<0, 8, 1, 128, 1>, 8, 128, delay, chunks);
    run("2 groups x 2 warps, 128-row stages", k_pipe2<8, 128, 128, 2>, 8, 128, delay, chunks);
    run("4 groups x 1 warp, 128-row stages", k_pipe2<8, 128, 128, 4>, 8, 128, delay, chunks);
  }
  run("skeleton (no copies), 4 warps together", k_pipe<2, 4, 1, 256, 1>, 4, 256, 0, 2);
  unsigned long long hs[2]; CK(cudaMemcpy(hs, sink, 16, cudaMemcpyDeviceToHost));
  printf("wait gave up: %llu\n", hs[1]);
  return 0;
}
