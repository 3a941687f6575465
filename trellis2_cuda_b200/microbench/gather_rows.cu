// Build and run: make -C trellis2_cuda_b200/microbench gather_rows && trellis2_cuda_b200/microbench/gather_rows
// Gather microbenchmark: indices staged in shared memory (as the conv kernel does), persistent loop,
// varying producer warps, mapping and stages in flight.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cstdint>
#define CK(x) do { cudaError_t e=(x); if(e!=cudaSuccess){printf("CUDA %s: %s\n",#x,cudaGetErrorString(e)); exit(1);} } while(0)
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template<int N> __device__ __forceinline__ void waitg() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// MAP 0: 8 threads per row (coalesced 128 B per row, 4 rows per warp instr); MAP 1: one thread per row (8 cp.async to the same row)
template<int MAP, int DEPTH>
__global__ void k_gather(const uint4* __restrict__ x, const int* __restrict__ idx, int rows_per_stage, int stages_total, int row_vec, int nidx, unsigned long long* sink) {
  extern __shared__ uint4 sm[];
  int* sidx = (int*)(sm + DEPTH * rows_per_stage * 8);
  const int T = blockDim.x, t = threadIdx.x;
  for (int i = t; i < nidx; i += T) sidx[i] = idx[(size_t)blockIdx.x * nidx + i];
  __syncthreads();
  uint32_t sbase = (uint32_t)__cvta_generic_to_shared(sm);
  if (MAP == 0) {
    const int c16 = t & 7, jb = t >> 3, per = rows_per_stage / (T / 8);
    int r[16];
    for (int s = 0; s < stages_total; s++) {
      uint32_t dst = sbase + (s % DEPTH) * rows_per_stage * 128 + jb * 128 + ((c16 ^ (jb & 7)) << 4);
      if ((s & 3) == 0) {
        const int* ip = sidx + ((s * rows_per_stage) % nidx);
#pragma unroll
        for (int i = 0; i < 16; i++) if (i < per) r[i] = ip[jb + (T / 8) * i];
      }
      const uint4* xs = x + c16 + (s & 3) * 8;
#pragma unroll
      for (int i = 0; i < 16; i++) if (i < per) cp16(dst + i * (T / 8) * 128, xs + (size_t)r[i] * row_vec);
      commit(); waitg<DEPTH - 1>();
    }
  } else {
    const int per = rows_per_stage / T;     // rows per thread per stage (>=1 needs T <= rows)
    for (int s = 0; s < stages_total; s++) {
      const int* ip = sidx + ((s * rows_per_stage) % nidx);
      for (int i = 0; i < per; i++) {
        int j = t + T * i; int r = ip[j];
        uint32_t dst = sbase + (s % DEPTH) * rows_per_stage * 128 + j * 128;
        const uint4* src = x + (size_t)r * row_vec;
#pragma unroll
        for (int c = 0; c < 8; c++) cp16(dst + ((c ^ (j & 7)) << 4), src + c);
      }
      commit(); waitg<DEPTH - 1>();
    }
  }
  waitg<0>();
  if (sm[t].x == 0x1234567) sink[0] = 1;
}

int main() {
  int nrows = 217821, row_bytes = 512, stages = 2000, nsm = 148, nidx = 8192;
  size_t xbytes = (size_t)nrows * row_bytes;
  uint4* x; CK(cudaMalloc(&x, xbytes)); CK(cudaMemset(x, 1, xbytes));
  unsigned long long* sink; CK(cudaMalloc(&sink, 8));
  for (int local = 0; local < 2; local++) {
    std::vector<int> h((size_t)nsm * nidx); srand(1);
    for (int b = 0; b < nsm; b++) for (int i = 0; i < nidx; i++) {
      int base = (int)(((long long)b * nrows) / nsm);
      h[(size_t)b * nidx + i] = local ? (base + rand() % 4096) % nrows : rand() % nrows;
    }
    int* idx; CK(cudaMalloc(&idx, h.size() * 4)); CK(cudaMemcpy(idx, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    auto run = [&](const char* name, auto kern, int T, int depth, int rows_per_stage) {
      int smem = depth * rows_per_stage * 128 + nidx * 4;
      if (smem > 227 * 1024) return;
      CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      float ms = 0;
      for (int rep = 0; rep < 2; rep++) {
        cudaEventRecord(e0);
        kern<<<nsm, T, smem>>>(x, idx, rows_per_stage, stages, row_bytes / 16, nidx, sink);
        cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms, e0, e1);
      }
      double bytes = (double)nsm * stages * rows_per_stage * 128;
      printf("local=%d %-10s T=%4d depth=%d rows/stage=%3d: %.3f ms %7.1f GB/s total %6.1f GB/s/SM (%.1f B/clk)\n", local, name, T, depth, rows_per_stage, ms,
             bytes / ms / 1e6, bytes / ms / 1e6 / nsm, bytes / ms / 1e6 / nsm / 1.9);
    };
    for (int rps : {128, 256}) {
      for (int T : {128, 256, 512, 1024}) { run("8thr/row", k_gather<0, 4>, T, 4, rps); }
      for (int T : {128, 256, 512}) { run("8thr/row", k_gather<0, 2>, T, 2, rps); }
      for (int T : {128, 256}) { run("8thr/row", k_gather<0, 6>, T, 6, rps); }
      for (int T : {32, 64, 128}) { if (T <= rps) run("1thr/row", k_gather<1, 4>, T, 4, rps); }
    }
    CK(cudaFree(idx));
  }
  return 0;
}
