// CUDA-core variant of the masked implicit-GEMM sparse conv: fp32 math on fp32 / fp16 / bf16 storage.
//
// This is the path for fp32 features (the tensor cores would drop them to tf32) and for shapes the
// tcgen05 kernel does not take (Ci not a multiple of 64, Co not a multiple of 32).  It computes the
// operator of src/spconv.cu:91-150 (trellis2-cuda): y[i,co] = sum over the tile's taps, ascending, of
// x[nbr[i,v],:] . w[co,v,:], fp32 accumulation, absent neighbours contributing zeros.
// One CTA = 128 rows of a plan tile x 64 output channels; 256 threads, 8x4 outputs each; K in chunks of 16.
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 64, BK = 16, LDA = BM + 4, LDB = BN + 4;

template <class T> __device__ __forceinline__ void load8(const T* p, float* o);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* o) {
  float4 a = __ldg((const float4*)p), b = __ldg((const float4*)p + 1);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float* o) {
  uint4 r = __ldg((const uint4*)p); const __half2* h = (const __half2*)&r;
#pragma unroll
  for (int i = 0; i < 4; i++) { float2 f = __half22float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
  uint4 r = __ldg((const uint4*)p); const __nv_bfloat162* h = (const __nv_bfloat162*)&r;
#pragma unroll
  for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
template <class T> __device__ __forceinline__ void load4(const T* p, float* o) {
#pragma unroll
  for (int i = 0; i < 4; i++) o[i] = to_f<T>(p[i]);
}

template <class T>
__global__ void __launch_bounds__(256) k_conv_simt(const T* __restrict__ x, const T* __restrict__ w, const uint32_t* __restrict__ nbr,
                                                   const int* __restrict__ order, const int* __restrict__ src,
                                                   const PlanTile* __restrict__ tiles, const int* __restrict__ tile_lo,
                                                   const int* __restrict__ tile_hi, EpiDev ep, T* __restrict__ y, int Ci, int Co, int subs, uint32_t n_in, int* status) {
  const int tile_id = *tile_lo + blockIdx.x / subs, sub = blockIdx.x % subs;      // plan tiles of 256 rows are two CTAs
  if (tile_id >= *tile_hi) return;
  __shared__ __align__(16) float As[BK][LDA];
  __shared__ __align__(16) float Bs[BK][LDB];
  __shared__ int s_out[BM];
  __shared__ int s_nrow[BM];
  const PlanTile tile = tiles[tile_id];
  if (sub * BM >= tile.rows) return;
  const int tid = threadIdx.x, co0 = blockIdx.y * BN;
  const i64 wrow0 = (i64)tile.wbase * Co;
  if (tid < BM) {
    int r = sub * BM + tid < tile.rows ? order[tile.start + sub * BM + tid] : -1;
    s_out[tid] = r;
    s_nrow[tid] = r < 0 ? -1 : (src ? (src[r] >> 3) : r);
  }
  __syncthreads();
  const int ty = tid >> 4, tx = tid & 15;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  const int a_row = tid >> 1, a_k0 = (tid & 1) * 8;     // A loader: 128 rows x 2 halves of 8 channels
  const int b_co = tid >> 2, b_k0 = (tid & 3) * 4;      // B loader: 64 channels x 4 quarters of 4 channels
  const int a_nrow = s_nrow[a_row];
  const int b_cog = co0 + b_co;

  for (uint32_t mk = tile.mask; mk; mk &= mk - 1) {
    const int v = __ffs(mk) - 1;
    uint32_t a_src = a_nrow < 0 ? NBR_EMPTY : __ldg(nbr + (i64)a_nrow * 27 + v);
    if (a_src >= n_in && a_src != NBR_EMPTY) { atomicOr(status, 256); a_src = NBR_EMPTY; }   // entry past the end of x: reported, read as absent
    for (int c0 = 0; c0 < Ci; c0 += BK) {
      float av[8], bv[4];
      if (a_src != NBR_EMPTY) load8<T>(x + (i64)a_src * Ci + c0 + a_k0, av);
      else {
#pragma unroll
        for (int i = 0; i < 8; i++) av[i] = 0.f;
      }
      if (b_cog < Co) load4<T>(w + ((wrow0 + b_cog) * 27 + v) * Ci + c0 + b_k0, bv);
      else {
#pragma unroll
        for (int i = 0; i < 4; i++) bv[i] = 0.f;
      }
      __syncthreads();   // previous chunk fully consumed
#pragma unroll
      for (int i = 0; i < 8; i++) As[a_k0 + i][a_row] = av[i];
#pragma unroll
      for (int i = 0; i < 4; i++) Bs[b_k0 + i][b_co] = bv[i];
      __syncthreads();
#pragma unroll
      for (int k = 0; k < BK; k++) {
        float4 a0 = *(const float4*)&As[k][ty * 8], a1 = *(const float4*)&As[k][ty * 8 + 4];
        float4 b = *(const float4*)&Bs[k][tx * 4];
        float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
      }
    }
  }
  // epilogue: every step rounds to the storage dtype, as the unfused kernels of the reference do
  const T* bias = (const T*)ep.bias; const T* res = (const T*)ep.residual; const T* skx = (const T*)ep.skip_x;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int orow = s_out[ty * 8 + i];
    if (orow < 0) continue;
    int sp = 0, ss = 0;
    if (skx) { int s = ep.skip_src[orow]; sp = s >> 3; ss = s & 7; }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int co = co0 + tx * 4 + j;
      if (co >= Co) continue;
      float h = rnd<T>(acc[i][j]);
      if (bias) h = rnd<T>(h + to_f<T>(bias[wrow0 + co]));
      if (ep.act) h = rnd<T>(act_apply(h, ep.act));
      if (res) h = rnd<T>(h + to_f<T>(res[(i64)orow * Co + co]));
      if (skx) h = rnd<T>(h + to_f<T>(skx[(i64)sp * ep.skip_cin + ss * (ep.skip_cin / 8) + co / ep.skip_rep]));
      y[(i64)orow * Co + co] = from_f<T>(h);
    }
  }
}

// ---- LayerNorm -> activation -> residual -> skip over [n,C], one warp per row, fp32 statistics
template <class T>
__global__ void __launch_bounds__(256) k_row_epilogue(const T* x, EpiDev ep, T* y, i64 n, int C) {   // y may alias x
  i64 row = (blockIdx.x * (i64)blockDim.x + threadIdx.x) >> 5; int lane = threadIdx.x & 31;
  if (row >= n) return;
  const T* xr = x + row * C; T* yr = y + row * C;
  const T* bias = (const T*)ep.bias; const T* res = (const T*)ep.residual; const T* skx = (const T*)ep.skip_x;
  float mean = 0.f, rstd = 1.f;
  if (ep.ln) {
    float s = 0.f;
    for (int c = lane; c < C; c += 32) { float v = to_f<T>(xr[c]); if (bias) v = rnd<T>(v + to_f<T>(bias[c])); s += v; }
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    mean = s / (float)C;
    float q = 0.f;
    for (int c = lane; c < C; c += 32) { float v = to_f<T>(xr[c]); if (bias) v = rnd<T>(v + to_f<T>(bias[c])); float d = v - mean; q += d * d; }
#pragma unroll
    for (int o = 16; o; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    rstd = rsqrtf(q / (float)C + ep.eps);
  }
  int sp = 0, ss = 0;
  if (skx) { int s = ep.skip_src[row]; sp = s >> 3; ss = s & 7; }
  for (int c = lane; c < C; c += 32) {
    float h = to_f<T>(xr[c]);
    if (bias) h = rnd<T>(h + to_f<T>(bias[c]));
    if (ep.ln) {
      float v = rstd * (h - mean);
      if (ep.gamma) v = ep.gamma[c] * v;
      if (ep.beta) v = v + ep.beta[c];
      h = rnd<T>(v);
    }
    if (ep.act) h = rnd<T>(act_apply(h, ep.act));
    if (res) h = rnd<T>(h + to_f<T>(res[row * C + c]));
    if (skx) h = rnd<T>(h + to_f<T>(skx[(i64)sp * ep.skip_cin + ss * (ep.skip_cin / 8) + c / ep.skip_rep]));
    yr[c] = from_f<T>(h);
  }
}

template <class T> __device__ __forceinline__ void store8(T* p, const float* v);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* v) {
  *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); *((float4*)p + 1) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__half>(__half* p, const float* v) {
  uint4 o; __half2* h = (__half2*)&o;
#pragma unroll
  for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *(uint4*)p = o;
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* v) {
  uint4 o; __nv_bfloat162* h = (__nv_bfloat162*)&o;
#pragma unroll
  for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *(uint4*)p = o;
}

// The same pass for rows of up to NV * 256 channels, C % 8 == 0: one warp per row, the row read ONCE in pieces of 8
// channels (16-byte loads for the 16-bit types) and held in registers through the statistics and the transform.
template <class T, int NV>
__global__ void __launch_bounds__(256) k_row_epilogue_vec(const T* x, EpiDev ep, T* y, i64 n, int C) {   // y may alias x
  const i64 row = (blockIdx.x * (i64)blockDim.x + threadIdx.x) >> 5; const int lane = threadIdx.x & 31;
  if (row >= n) return;
  const T* xr = x + row * C; T* yr = y + row * C;
  const T* bias = (const T*)ep.bias; const T* res = (const T*)ep.residual; const T* skx = (const T*)ep.skip_x;
  const int nvec = C >> 3;
  float h[NV][8];
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const int vi = lane + 32 * k;
    if (vi < nvec) {
      load8<T>(xr + vi * 8, h[k]);
      if (bias) {
        float b[8]; load8<T>(bias + vi * 8, b);
#pragma unroll
        for (int i = 0; i < 8; i++) h[k][i] = rnd<T>(h[k][i] + b[i]);
      }
    }
  }
  if (ep.ln) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; k++)
      if (lane + 32 * k < nvec) {
#pragma unroll
        for (int i = 0; i < 8; i++) s += h[k][i];
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / (float)C;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; k++)
      if (lane + 32 * k < nvec) {
#pragma unroll
        for (int i = 0; i < 8; i++) { const float d = h[k][i] - mean; q += d * d; }
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = rsqrtf(q / (float)C + ep.eps);
#pragma unroll
    for (int k = 0; k < NV; k++) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        float g[8], be[8];
        if (ep.gamma) { const float4 a = __ldg((const float4*)(ep.gamma + vi * 8)), b = __ldg((const float4*)(ep.gamma + vi * 8) + 1);
                        g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w; }
        if (ep.beta) { const float4 a = __ldg((const float4*)(ep.beta + vi * 8)), b = __ldg((const float4*)(ep.beta + vi * 8) + 1);
                       be[0] = a.x; be[1] = a.y; be[2] = a.z; be[3] = a.w; be[4] = b.x; be[5] = b.y; be[6] = b.z; be[7] = b.w; }
#pragma unroll
        for (int i = 0; i < 8; i++) {
          float v = rstd * (h[k][i] - mean);
          if (ep.gamma) v = g[i] * v;
          if (ep.beta) v = v + be[i];
          h[k][i] = rnd<T>(v);
        }
      }
    }
  }
  int sp = 0, ss = 0;
  if (skx) { const int sv = ep.skip_src[row]; sp = sv >> 3; ss = sv & 7; }
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const int vi = lane + 32 * k;
    if (vi >= nvec) continue;
    if (ep.act) {
#pragma unroll
      for (int i = 0; i < 8; i++) h[k][i] = rnd<T>(act_apply(h[k][i], ep.act));
    }
    if (res) {
      float r[8]; load8<T>(res + row * C + vi * 8, r);
#pragma unroll
      for (int i = 0; i < 8; i++) h[k][i] = rnd<T>(h[k][i] + r[i]);
    }
    if (skx) {
      const T* sx = skx + (i64)sp * ep.skip_cin + ss * (ep.skip_cin / 8);
#pragma unroll
      for (int i = 0; i < 8; i++) h[k][i] = rnd<T>(h[k][i] + to_f<T>(sx[(vi * 8 + i) / ep.skip_rep]));
    }
    store8<T>(yr + vi * 8, h[k]);
  }
}

template <class T>
void row_epilogue_pick(cudaStream_t st, const void* x, const EpiDev& ep, void* y, i64 n, int C) {
  const int grid = cdiv_i(n * 32, 256);
  const bool aligned = (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 && (!ep.residual || (uintptr_t)ep.residual % 16 == 0) &&
                       (!ep.bias || (uintptr_t)ep.bias % 16 == 0) && (!ep.gamma || (uintptr_t)ep.gamma % 16 == 0) && (!ep.beta || (uintptr_t)ep.beta % 16 == 0);
  if (C % 8 == 0 && aligned && C <= 2048) {
    if (C <= 256) k_row_epilogue_vec<T, 1><<<grid, 256, 0, st>>>((const T*)x, ep, (T*)y, n, C);
    else if (C <= 512) k_row_epilogue_vec<T, 2><<<grid, 256, 0, st>>>((const T*)x, ep, (T*)y, n, C);
    else if (C <= 1024) k_row_epilogue_vec<T, 4><<<grid, 256, 0, st>>>((const T*)x, ep, (T*)y, n, C);
    else k_row_epilogue_vec<T, 8><<<grid, 256, 0, st>>>((const T*)x, ep, (T*)y, n, C);
  } else {
    k_row_epilogue<T><<<grid, 256, 0, st>>>((const T*)x, ep, (T*)y, n, C);
  }
}

}  // namespace

int conv_simt_launch(t2sc_ctx* ctx, const t2sc_plan* plan, const void* x, const void* w, const EpiDev& ep, void* y,
                     int dtype, i64 n_in, int Ci, int Co, int part) {
  T2_REQ(ctx, Ci % BK == 0, "Ci=%d", Ci);
  const TilePart tp = tile_part(plan, part);
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  const int subs = plan->tile_rows / BM;
  dim3 grid((unsigned)(plan->max_tiles * subs), (unsigned)cdiv_i(Co, BN));
  if (dtype == T2SC_F32)
    k_conv_simt<float><<<grid, 256, 0, ctx->stream>>>((const float*)x, (const float*)w, plan->nbr, plan->order, plan->src, plan->tiles, tp.lo, tp.hi, ep, (float*)y, Ci, Co, subs, (uint32_t)n_in, ctx->status);
  else if (dtype == T2SC_F16)
    k_conv_simt<__half><<<grid, 256, 0, ctx->stream>>>((const __half*)x, (const __half*)w, plan->nbr, plan->order, plan->src, plan->tiles, tp.lo, tp.hi, ep, (__half*)y, Ci, Co, subs, (uint32_t)n_in, ctx->status);
  else
    k_conv_simt<__nv_bfloat16><<<grid, 256, 0, ctx->stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, plan->nbr, plan->order, plan->src, plan->tiles, tp.lo, tp.hi, ep, (__nv_bfloat16*)y, Ci, Co, subs, (uint32_t)n_in, ctx->status);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

int row_epilogue_launch(t2sc_ctx* ctx, const void* x, const EpiDev& ep, void* y, i64 n, int C, int dtype) {
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  if (dtype == T2SC_F32) row_epilogue_pick<float>(ctx->stream, x, ep, y, n, C);
  else if (dtype == T2SC_F16) row_epilogue_pick<__half>(ctx->stream, x, ep, y, n, C);
  else row_epilogue_pick<__nv_bfloat16>(ctx->stream, x, ep, y, n, C);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}
