// Build and run: make -C trellis2_cuda_b200/microbench mbarrier_pingpong && trellis2_cuda_b200/microbench/mbarrier_pingpong
// Minimal two-role mbarrier ping-pong: how many clocks per iteration does a full/empty stage handshake cost?
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#define CK(x) do { cudaError_t e=(x); if(e!=cudaSuccess){printf("CUDA %s: %s\n",#x,cudaGetErrorString(e)); return 1;} } while(0)
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t c) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(c) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ void arrive_noinc(uint32_t bar) { asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;
  long long t0 = clock64();
  while (!mbar_try(bar, parity)) if (clock64() - t0 > 2000000000ll) return false;
  return true;
}
// PT / CT: producer / consumer threads that take part (1 or 32); S stages; NOINC: producer arrives with cp.async noinc
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) { asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_relaxed(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.relaxed.cta.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
template <int V> __device__ __forceinline__ bool wait_v(uint32_t bar, uint32_t parity) {
  long long t0 = clock64();
  if (V == 1) { while (!mbar_try_relaxed(bar, parity)) if (clock64() - t0 > 2000000000ll) return false; return true; }
  if (V == 3) { while (!mbar_test(bar, parity)) if (clock64() - t0 > 2000000000ll) return false; return true; }
  return mbar_wait(bar, parity);
}
// volatile-counter handshake (V == 4): no mbarrier at all
template <int S>
__global__ void k_flag(int iters, unsigned long long* out) {
  __shared__ volatile int prod_cnt, cons_cnt;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { prod_cnt = 0; cons_cnt = 0; }
  __syncthreads();
  long long t0 = clock64(); bool ok = true;
  if (lane == 0) {
    if (warp == 0) for (int it = 0; it < iters && ok; it++) {
      long long w0 = clock64();
      while (it - cons_cnt >= S) if (clock64() - w0 > 2000000000ll) { ok = false; break; }
      __threadfence_block(); prod_cnt = it + 1;
    } else for (int it = 0; it < iters && ok; it++) {
      long long w0 = clock64();
      while (prod_cnt <= it) if (clock64() - w0 > 2000000000ll) { ok = false; break; }
      __threadfence_block(); cons_cnt = it + 1;
    }
  }
  long long t1 = clock64();
  if (blockIdx.x == 0 && lane == 0) out[warp] = (unsigned long long)(t1 - t0);
  if (!ok) out[2] = 1;
}
__device__ float g_sink;
__device__ __forceinline__ void spin(int d) {            // d/4 dependent FMAs: about d clocks, no clock reads
  float x = 1.0f;
#pragma unroll 1
  for (int i = 0; i < d / 4; i++) x = fmaf(x, 1.0000001f, 0.5f);
  if (x == 123.456f) g_sink = x;
}
template <int S, int PT, int CT, bool NOINC, int V = 0>
__global__ void k_pp(int iters, unsigned long long* out, int pdelay = 0, int cdelay = 0) {
  constexpr int STR = V == 2 ? 128 : 8;
  __shared__ __align__(128) uint8_t bar_mem[2 * S * STR];
  const uint32_t bfull = (uint32_t)__cvta_generic_to_shared(bar_mem), bempty = bfull + STR * S;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { for (int s = 0; s < S; s++) { mbar_init(bfull + STR * s, PT); mbar_init(bempty + STR * s, CT); } asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  __syncthreads();
  bool ok = true;
  long long t0 = clock64();
  if (warp == 0) {
    if (lane < PT) for (int it = 0; it < iters && ok; it++) {
      const int s = it % S;
      ok = wait_v<V>(bempty + STR * s, ((it / S) & 1) ^ 1);
      spin(pdelay);
      if (NOINC) arrive_noinc(bfull + STR * s); else if (V == 1) mbar_arrive_relaxed(bfull + STR * s); else mbar_arrive(bfull + STR * s);
    }
  } else {
    if (lane < CT) for (int it = 0; it < iters && ok; it++) {
      const int s = it % S;
      ok = wait_v<V>(bfull + STR * s, (it / S) & 1);
      spin(cdelay);
      if (V == 1) mbar_arrive_relaxed(bempty + STR * s); else mbar_arrive(bempty + STR * s);
    }
  }
  long long t1 = clock64();
  if (blockIdx.x == 0 && lane == 0) out[warp] = (unsigned long long)(t1 - t0);
  if (!ok) out[2] = 1;
}
// one thread, no partner: wait on an already-completed phase + arrive on a never-completing barrier: cost of the instruction pair
__global__ void k_solo(int iters, unsigned long long* out) {
  __shared__ uint64_t bars[2];
  const uint32_t b0 = (uint32_t)__cvta_generic_to_shared(bars), b1 = b0 + 8;
  // (1 << 20) - 1 is the largest valid count; 20000 arrivals never complete that barrier
  if (threadIdx.x == 0) { mbar_init(b0, 1); mbar_init(b1, (1 << 20) - 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  __syncthreads();
  long long t0 = clock64(); int okc = 0;
  if (threadIdx.x == 0) for (int it = 0; it < iters; it++) { okc += mbar_try(b0, 1); mbar_arrive(b1); }
  long long t1 = clock64();
  if (threadIdx.x == 0) { out[0] = (unsigned long long)(t1 - t0); out[1] = okc; }
}
// the same ping-pong, but each role asks about its NEXT stage before doing this stage's work, so the try_wait latency
// overlaps the work instead of sitting in front of it
template <int S>
__global__ void k_peek(int iters, unsigned long long* out, int pdelay, int cdelay) {
  __shared__ __align__(8) uint64_t bars[2 * S];
  const uint32_t bfull = (uint32_t)__cvta_generic_to_shared(bars), bempty = bfull + 8 * S;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { for (int s = 0; s < S; s++) { mbar_init(bfull + 8 * s, 1); mbar_init(bempty + 8 * s, 1); } asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  __syncthreads();
  bool ok = true;
  long long t0 = clock64();
  if (lane == 0) {
    if (warp == 0) {
      bool tok = mbar_try(bempty, 1);
      for (int it = 0; it < iters && ok; it++) {
        const int s = it % S, n = (it + 1) % S;
        if (!tok) ok = mbar_wait(bempty + 8 * s, ((it / S) & 1) ^ 1);
        tok = mbar_try(bempty + 8 * n, (((it + 1) / S) & 1) ^ 1);
        spin(pdelay);
        mbar_arrive(bfull + 8 * s);
      }
    } else {
      bool tok = mbar_try(bfull, 0);
      for (int it = 0; it < iters && ok; it++) {
        const int s = it % S, n = (it + 1) % S;
        if (!tok) ok = mbar_wait(bfull + 8 * s, (it / S) & 1);
        tok = mbar_try(bfull + 8 * n, ((it + 1) / S) & 1);
        spin(cdelay);
        mbar_arrive(bempty + 8 * s);
      }
    }
  }
  long long t1 = clock64();
  if (blockIdx.x == 0 && lane == 0) out[warp] = (unsigned long long)(t1 - t0);
  if (!ok) out[2] = 1;
}
// single thread: every try_wait result decides a branch, so the loop time is the instruction's latency, not its throughput
__global__ void k_lat(int iters, unsigned long long* out) {
  __shared__ uint64_t bars[2];
  const uint32_t b0 = (uint32_t)__cvta_generic_to_shared(bars), b1 = b0 + 8;
  if (threadIdx.x == 0) { mbar_init(b0, 1); mbar_init(b1, (1 << 20) - 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long t0 = clock64(); int n = 0;
    for (int it = 0; it < iters; it++) { if (!mbar_try(b0, 1)) break; n++; }
    long long t1 = clock64();
    for (int it = 0; it < iters; it++) { if (!mbar_try(b0, 1)) break; mbar_arrive(b1); n++; }
    long long t2 = clock64();
    for (int it = 0; it < iters; it++) { mbar_arrive(b1); }
    long long t3 = clock64();
    out[0] = (unsigned long long)(t1 - t0); out[1] = (unsigned long long)(t2 - t1); out[2] = (unsigned long long)(t3 - t2); out[3] = n;
  }
}
int main() {
  unsigned long long* out; CK(cudaMalloc(&out, 64)); unsigned long long h[4];
  const int iters = 20000;
  auto rep = [&](const char* name) { cudaError_t e = cudaDeviceSynchronize(); if (e != cudaSuccess) printf("  error: %s\n", cudaGetErrorString(e)); e = cudaGetLastError(); if (e != cudaSuccess) printf("  launch error: %s\n", cudaGetErrorString(e)); cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost); printf("%-44s producer %6.1f clk/iter  consumer %6.1f clk/iter  gave_up %llu\n", name, (double)h[0] / iters, (double)h[1] / iters, h[2]); cudaMemset(out, 0, 64); };
  CK(cudaMemset(out, 0, 64));
  k_solo<<<1, 32>>>(iters, out); { cudaError_t e = cudaDeviceSynchronize(); printf("solo status: %s / %s\n", cudaGetErrorString(e), cudaGetErrorString(cudaGetLastError())); } cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost); printf("solo try_wait(ready)+arrive: %.1f clk/iter (ok %llu)\n", (double)h[0] / iters, h[1]); cudaMemset(out, 0, 64);
  k_pp<4, 1, 1, false><<<148, 64>>>(iters, out); rep("S=4 1 thread each");
  k_pp<2, 1, 1, false><<<148, 64>>>(iters, out); rep("S=2 1 thread each");
  k_pp<8, 1, 1, false><<<148, 64>>>(iters, out); rep("S=8 1 thread each");
  k_pp<4, 32, 1, false><<<148, 64>>>(iters, out); rep("S=4 32 producers, 1 consumer");
  k_pp<4, 32, 32, false><<<148, 64>>>(iters, out); rep("S=4 32 producers, 32 consumers");
  k_pp<4, 32, 1, true><<<148, 64>>>(iters, out); rep("S=4 32 producers noinc, 1 consumer");
  k_pp<4, 1, 1, true><<<148, 64>>>(iters, out); rep("S=4 1 producer noinc, 1 consumer");
  k_lat<<<1, 32>>>(iters, out); cudaDeviceSynchronize(); cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost);
  printf("one thread: try_wait->branch %.1f clk, try_wait->branch->arrive %.1f clk, arrive only %.1f clk (n %llu)\n", (double)h[0] / iters, (double)h[1] / iters, (double)h[2] / iters, h[3]); cudaMemset(out, 0, 64);
  for (int d : {0, 100, 300, 600}) {
    char nm[96];
    snprintf(nm, 96, "S=4 both work %d clk", d); k_pp<4, 1, 1, false><<<148, 64>>>(iters, out, d, d); rep(nm);
    snprintf(nm, 96, "S=4 both work %d clk, peek ahead", d); k_peek<4><<<148, 64>>>(iters, out, d, d); rep(nm);
    snprintf(nm, 96, "S=4 producer work %d clk, peek ahead", d); k_peek<4><<<148, 64>>>(iters, out, d, 0); rep(nm);
    snprintf(nm, 96, "S=2 both work %d clk, peek ahead", d); k_peek<2><<<148, 64>>>(iters, out, d, d); rep(nm);
  }
  return 0;
}
