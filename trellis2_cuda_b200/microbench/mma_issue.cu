// Build and run: make -C trellis2_cuda_b200/microbench mma_issue && trellis2_cuda_b200/microbench/mma_issue
// tcgen05.mma issue-rate microbenchmark: clocks per instruction for several (M, N) shapes, K = 16, bf16, operands in smem
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t desc(uint32_t saddr) {
  uint64_t d = 0; d |= (uint64_t)((saddr & 0x3FFFFu) >> 4); d |= (uint64_t)1 << 16; d |= (uint64_t)(1024 >> 4) << 32; d |= (uint64_t)1 << 46; d |= (uint64_t)2 << 61; return d;
}
__global__ void __launch_bounds__(128, 1) k(int M, int N, int iters, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar; __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < 98304 / 4; i += 128) ((uint32_t*)sm)[i] = 0;
  if (threadIdx.x == 0) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar))); asm volatile("fence.mbarrier_init.release.cluster;"); }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads(); asm volatile("tcgen05.fence::after_thread_sync;");
  asm volatile("fence.proxy.async.shared::cta;");
  uint32_t tm = slot;
  uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
  if (threadIdx.x == 0) {
    uint64_t ad = desc(smem_u32(sm)), bd = desc(smem_u32(sm) + 32768);
    long long t0 = clock64();
    for (int i = 0; i < iters; i++) {
      uint32_t acc = i > 0;
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tm + (i & 1) * 256), "l"(ad + 2 * (i & 3)), "l"(bd + 2 * (i & 3)), "r"(idesc), "r"(acc) : "memory");
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    uint32_t ok = 0; long long guard = clock64();
    while (!ok && clock64() - guard < 2000000000ll)
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(&bar)) : "memory");
    long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads();
  if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(512) : "memory");
}
int main() {
  long long* out; cudaMalloc(&out, 8);
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 100352);
  int shapes[][2] = {{128, 256}, {128, 128}, {128, 64}, {128, 32}, {64, 256}, {64, 128}, {64, 64}};
  for (auto& s : shapes) for (int grid : {1, 148}) {
    int iters = 4096; long long h = 0;
    for (int rep = 0; rep < 2; rep++) { k<<<grid, 128, 100352>>>(s[0], s[1], iters, out); cudaError_t e = cudaDeviceSynchronize(); if (e) { printf("err %s\n", cudaGetErrorString(e)); return 1; } }
    cudaMemcpy(&h, out, 8, cudaMemcpyDeviceToHost);
    printf("M=%3d N=%3d grid=%3d: %.1f clk per MMA (ideal at 8192 flop/clk: %.1f)\n", s[0], s[1], grid, (double)h / iters, 2.0 * s[0] * s[1] * 16 / 8192);
  }
  return 0;
}
