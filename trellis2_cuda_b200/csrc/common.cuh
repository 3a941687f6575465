// Shared declarations of the t2sc library: context, error plumbing, storage-dtype helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include "../../include/t2sc.h"

using i64 = int64_t;
static constexpr uint32_t NBR_EMPTY = 0xffffffffu;

struct t2sc_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int num_sms = 148;
  int smem_optin = 0;
  i64 launches = 0;
  char* arena = nullptr;        // scratch arena of the entry points (see Scratch), arena_bytes long; grown to arena_want
  size_t arena_bytes = 0, arena_want = 0;
  int* status = nullptr;        // device word; kernels OR an error code into it when a bounded wait gives up
  cudaEvent_t done = nullptr;   // event the host polls when it waits for the stream (see ctx_wait in api.cu)
  char err[1024] = {0};
};

// One tile of the execution plan: `rows` consecutive entries of order[] starting at `start`, all using
// weight rows [wbase, wbase+Co) and the union tap mask `mask`.
struct PlanTile { int start, rows, wbase; uint32_t mask; };

struct t2sc_plan {
  i64 n_out = 0;                // output rows
  i64 n_rows = 0;               // rows of nbr / gray
  i64 n_in = 0;                 // rows of the feature array the map's entries index (n_rows unless t2sc_plan_set_input_rows said more)
  const uint32_t* nbr = nullptr;  // borrowed
  const int32_t* src = nullptr;   // borrowed (NULL for a submanifold plan)
  int32_t* order = nullptr;     // [n_out] output row handled at each plan position
  uint32_t* tnbr = nullptr;     // [max_tiles][27][tile_rows]: the map in tile order, tap-major, absent = 0x80000000 (what a tile's
                                // CTA copies into shared memory with one bulk copy)
  i64 table_n_in = -1;          // n_in the table was last checked against (-1: not yet)
  PlanTile* tiles = nullptr;    // [max_tiles]
  int* perm = nullptr;          // [max_tiles]: positions -> tile numbers, each part's tiles by falling tap count: the order the
                                // tcgen05 kernel's CTAs take them in, so that every SM gets long and short tiles alike
  bool balanced = false;        // perm is filled (maps sorted as one block); large maps keep plan order for L2 locality
  int* meta = nullptr;          // device [16]: group counts, bounds, stats (one allocation, one memset)
  int* bounds = nullptr;        // = meta + 8, device [3]: {0, first boundary tile, realised tile count}; parts are [b0,b1) and [b1,b2)
  int* ntiles = nullptr;        // = bounds + 2: realised tile count (<= max_tiles)
  bool split = false;           // made by t2sc_plan_create_split: interior tiles first, boundary tiles last
  unsigned long long* stats = nullptr;  // device [2]: computed taps, active taps
  i64 max_tiles = 0;
  int tile_rows = 256;           // 128 or 256
};

int t2sc_fail(t2sc_ctx* ctx, int code, const char* fmt, ...);

#define T2_CUDA(ctx, call)                                                                              \
  do {                                                                                                  \
    cudaError_t e_ = (call);                                                                            \
    if (e_ != cudaSuccess)                                                                              \
      return t2sc_fail((ctx), T2SC_ERR_CUDA, "CUDA %s @ %s:%d: %s", #call, __FILE__, __LINE__, cudaGetErrorString(e_)); \
  } while (0)
#define T2_REQ(ctx, cond, ...)                                                  \
  do {                                                                          \
    if (!(cond)) return t2sc_fail((ctx), T2SC_ERR_ARG, "check failed " #cond ": " __VA_ARGS__); \
  } while (0)
#define T2_LAUNCHED(ctx) do { (ctx)->launches++; T2_CUDA(ctx, cudaGetLastError()); } while (0)

static inline int cdiv_i(i64 a, i64 b) { return (int)((a + b - 1) / b); }
static inline size_t dtype_size(int dt) { return dt == T2SC_F32 ? 4 : (dt == T2SC_U8 ? 1 : 2); }

// scratch from the device's stream-ordered pool (freed on the same stream)
template <class T> static inline cudaError_t t2_alloc(t2sc_ctx* ctx, T** p, size_t count) {
  return cudaMallocAsync((void**)p, (count ? count : 1) * sizeof(T), ctx->stream);
}
static inline void t2_free(t2sc_ctx* ctx, void* p) { if (p) cudaFreeAsync(p, ctx->stream); }
// Scratch of one entry point.  Steady state takes nothing from the memory pool: the context keeps one arena (grown to the
// largest total any call has needed) and a call carves its pieces out of it in order; calls on a context run one after the
// other on its stream, so the next call may overwrite what this one used.  A request the arena cannot hold falls back to
// the stream-ordered pool (returned when the entry point returns, on the error paths too) and raises the size the arena
// is grown to before the next call.
struct Scratch {
  t2sc_ctx* ctx; void* held[16]; int n = 0; size_t used = 0, wanted = 0;
  explicit Scratch(t2sc_ctx* c) : ctx(c) {
    if (c->arena_want > c->arena_bytes) {
      if (c->arena) cudaFreeAsync(c->arena, c->stream);
      c->arena = nullptr; c->arena_bytes = 0;
      if (cudaMallocAsync((void**)&c->arena, c->arena_want, c->stream) == cudaSuccess) c->arena_bytes = c->arena_want;
      else (void)cudaGetLastError();
    }
  }
  Scratch(const Scratch&) = delete;
  Scratch& operator=(const Scratch&) = delete;
  template <class T> cudaError_t get(T** p, size_t count) {
    const size_t bytes = (((count ? count : 1) * sizeof(T)) + 255) & ~(size_t)255;
    wanted += bytes;
    if (used + bytes <= ctx->arena_bytes) { *p = (T*)(ctx->arena + used); used += bytes; return cudaSuccess; }
    cudaError_t e = n < 16 ? cudaMallocAsync((void**)p, bytes, ctx->stream) : cudaErrorMemoryAllocation;
    if (e == cudaSuccess) held[n++] = (void*)*p;
    return e;
  }
  ~Scratch() {
    for (int i = 0; i < n; i++) t2_free(ctx, held[i]);
    if (wanted > ctx->arena_want) ctx->arena_want = wanted;
  }
};

// ---- storage types: load as float, round float to storage and widen back
template <class T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <class T> __device__ __forceinline__ float rnd(float v) { return to_f<T>(from_f<T>(v)); }

__device__ __forceinline__ float act_apply(float v, int act) {
  if (act == T2SC_ACT_SILU) return v / (1.f + expf(-v));
  if (act == T2SC_ACT_GELU_ERF) return v * 0.5f * (1.f + erff(v * 0.70710678118654752440f));
  if (act == T2SC_ACT_GELU_TANH) {
    const float kBeta = 0.79788456080286535588f, kKappa = 0.044715f;
    float x3 = v * v * v, inner = kBeta * (v + kKappa * x3);
    return 0.5f * v * (1.f + tanhf(inner));
  }
  return v;
}

// Device-side epilogue description (a flattened t2sc_epilogue)
struct EpiDev {
  const void* bias; const float* gamma; const float* beta; const void* residual;
  const void* skip_x; const int32_t* skip_src;
  float eps; int ln, act, skip_cin, skip_rep;
};
static inline EpiDev epi_dev(const t2sc_epilogue* e) {
  EpiDev d; memset(&d, 0, sizeof(d));
  if (e) {
    d.bias = e->bias; d.gamma = e->ln_gamma; d.beta = e->ln_beta; d.residual = e->residual;
    d.skip_x = e->skip_x; d.skip_src = e->skip_src; d.eps = e->ln_eps; d.ln = e->ln; d.act = e->act;
    d.skip_cin = e->skip_cin; d.skip_rep = e->skip_rep;
  }
  return d;
}

int plan_table_prepare(t2sc_ctx* ctx, t2sc_plan* plan, i64 n_in);      // plan.cu: table bounds-checked against n_in (once per n_in)
// implemented in the kernel files
// which tiles of a plan a launch covers: pointers to the first tile index and to the index one past the last
struct TilePart { const int* lo; const int* hi; };
static inline TilePart tile_part(const t2sc_plan* p, int part) {
  if (part == T2SC_PART_INTERIOR) return TilePart{p->bounds, p->bounds + 1};
  if (part == T2SC_PART_BOUNDARY) return TilePart{p->bounds + 1, p->bounds + 2};
  return TilePart{p->bounds, p->bounds + 2};
}
int conv_simt_launch(t2sc_ctx* ctx, const t2sc_plan* plan, const void* x, const void* w, const EpiDev& ep, void* y,
                     int dtype, i64 n_in, int Ci, int Co, int part = T2SC_PART_ALL);
bool conv_umma_supported(int dtype, int Ci, int Co, const EpiDev& ep);
bool conv_umma_fuses_ln(int Co);      // can the tcgen05 path hold a whole output row in one accumulator (fused LayerNorm)?
int conv_umma_launch(t2sc_ctx* ctx, const t2sc_plan* plan, const void* x, const void* w, i64 w_rows, const EpiDev& ep, void* y,
                     int dtype, i64 n_in, int Ci, int Co, int part = T2SC_PART_ALL, const void* const* x_peers = nullptr,
                     const int64_t* rows_peers = nullptr, int n_peers = 0, int self_rank = 0, const uint32_t* peer_nbr = nullptr);
int linear_umma_launch(t2sc_ctx* ctx, const void* x, const void* w, const EpiDev& ep, void* y, int dtype, i64 n, int Ci, int Co);
bool conv_umma2_supported(const t2sc_plan* plan, int dtype, int Ci, int Co, const EpiDev& ep);
int conv_umma2_launch(t2sc_ctx* ctx, const t2sc_plan* plan, const void* x, const void* w, i64 w_rows, const EpiDev& ep, void* y,
                      int dtype, i64 n_in, int Ci, int Co, int part = T2SC_PART_ALL);
int row_epilogue_launch(t2sc_ctx* ctx, const void* x, const EpiDev& ep, void* y, i64 n, int C, int dtype);
