// C-ABI entry points that are not kernels themselves: context, errors, conv dispatch, host-buffer call.
#include "common.cuh"
#include <sched.h>

static char g_create_err[512] = {0};

int t2sc_fail(t2sc_ctx* ctx, int code, const char* fmt, ...) {
  char* dst = ctx ? ctx->err : g_create_err;
  size_t cap = ctx ? sizeof(ctx->err) : sizeof(g_create_err);
  va_list a; va_start(a, fmt); vsnprintf(dst, cap, fmt, a); va_end(a);
  return code;
}

extern "C" const char* t2sc_last_error(const t2sc_ctx* ctx) { return ctx ? ctx->err : g_create_err; }
extern "C" int64_t t2sc_launch_count(const t2sc_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int t2sc_ctx_create(int device, void* stream, t2sc_ctx** out) {
  if (!out) return t2sc_fail(nullptr, T2SC_ERR_ARG, "t2sc_ctx_create: out is NULL");
  *out = nullptr;
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0)
    return t2sc_fail(nullptr, T2SC_ERR_CUDA, "t2sc_ctx_create: no CUDA device (%s); this library has no CPU path",
                     cudaGetErrorString(e));
  if (device < 0 || device >= ndev) return t2sc_fail(nullptr, T2SC_ERR_ARG, "t2sc_ctx_create: device %d of %d", device, ndev);
  cudaDeviceProp prop;
  if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess)
    return t2sc_fail(nullptr, T2SC_ERR_CUDA, "t2sc_ctx_create: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return t2sc_fail(nullptr, T2SC_ERR_UNSUPPORTED, "t2sc_ctx_create: device %d is sm_%d%d; this library is built for sm_100a only",
                     device, prop.major, prop.minor);
  t2sc_ctx* c = new t2sc_ctx();
  c->device = device; c->num_sms = prop.multiProcessorCount; c->smem_optin = (int)prop.sharedMemPerBlockOptin;
  if (stream) { c->stream = (cudaStream_t)stream; c->own_stream = false; }
  else {
    if ((e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)) != cudaSuccess) {
      delete c; return t2sc_fail(nullptr, T2SC_ERR_CUDA, "t2sc_ctx_create: %s", cudaGetErrorString(e));
    }
    c->own_stream = true;
  }
  // keep freed scratch in the pool instead of returning it to the driver at every sync (src/core.cu:24-26 does the same)
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
    uint64_t thr = UINT64_MAX; cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thr);
  }
  if ((e = cudaMalloc(&c->status, sizeof(int))) != cudaSuccess || (e = cudaMemset(c->status, 0, sizeof(int))) != cudaSuccess) {
    if (c->own_stream) cudaStreamDestroy(c->stream);
    delete c; return t2sc_fail(nullptr, T2SC_ERR_CUDA, "t2sc_ctx_create: %s", cudaGetErrorString(e));
  }
  *out = c;
  return T2SC_OK;
}

// Waits for the context's stream by polling an event and yielding the core between polls.  cudaStreamSynchronize was
// seen to keep other host threads of the process, each driving its own context, from issuing their calls while it waited
// (three complete host-buffer calls in flight then took as long as three calls one after the other); a blocking-sync
// event cured that but added ~0.4 ms to a single call.  A poll returns at once, so nothing is held between polls.
static cudaError_t ctx_wait(t2sc_ctx* ctx) {
  cudaError_t e;
  if (!ctx->done && (e = cudaEventCreateWithFlags(&ctx->done, cudaEventDisableTiming)) != cudaSuccess) return e;
  if ((e = cudaEventRecord(ctx->done, ctx->stream)) != cudaSuccess) return e;
  while ((e = cudaEventQuery(ctx->done)) == cudaErrorNotReady) sched_yield();
  return e;
}

extern "C" int t2sc_ctx_destroy(t2sc_ctx* ctx) {
  if (!ctx) return T2SC_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->arena) cudaFreeAsync(ctx->arena, ctx->stream);
  cudaStreamSynchronize(ctx->stream);
  cudaFree(ctx->status);
  if (ctx->done) cudaEventDestroy(ctx->done);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return T2SC_OK;
}

extern "C" int t2sc_ctx_sync(t2sc_ctx* ctx) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_CUDA(ctx, ctx_wait(ctx));
  return T2SC_OK;
}

extern "C" int t2sc_device_status(t2sc_ctx* ctx, int* status_host) {
  T2_REQ(ctx, ctx && status_host, "null argument");
  T2_CUDA(ctx, cudaMemcpyAsync(status_host, ctx->status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  T2_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (*status_host) {
    T2_CUDA(ctx, cudaMemsetAsync(ctx->status, 0, sizeof(int), ctx->stream));
    const int waits = *status_host & ~256;        // bits 0..9 bar 8: which role's mbarrier wait, 1024: the peer barrier
    return t2sc_fail(ctx, T2SC_ERR_DEVICE, "%s%s(status word 0x%x); results of the last launches are invalid",
                     waits ? "a device-side wait gave up " : "", (*status_host & 256) ? "a neighbour-map entry pointed past the end of its feature array " : "",
                     *status_host);
  }
  return T2SC_OK;
}

// ------------------------------------------------------------------------------------------ conv dispatch
extern "C" int t2sc_subm_conv(t2sc_ctx* ctx, t2sc_plan* plan, const void* x, const void* w, const t2sc_epilogue* ep,
                              void* y, int dtype, int64_t n_in, int Ci, int Co, int variant) {
  return t2sc_subm_conv_part(ctx, plan, x, w, ep, y, dtype, n_in, Ci, Co, variant, T2SC_PART_ALL);
}

extern "C" int t2sc_subm_conv_part(t2sc_ctx* ctx, t2sc_plan* plan, const void* x, const void* w, const t2sc_epilogue* ep,
                                   void* y, int dtype, int64_t n_in, int Ci, int Co, int variant, int part) {
  T2_REQ(ctx, ctx && plan, "null context or plan");
  T2_REQ(ctx, part == T2SC_PART_ALL || part == T2SC_PART_INTERIOR || part == T2SC_PART_BOUNDARY, "part=%d", part);
  T2_REQ(ctx, dtype == T2SC_F32 || dtype == T2SC_F16 || dtype == T2SC_BF16, "dtype %d", dtype);
  T2_REQ(ctx, Ci > 0 && Co > 0 && Ci % 32 == 0, "spconv shapes Ci=%d Co=%d (Ci must be a multiple of 32)", Ci, Co);
  // the reference requires N == c.N (src/spconv.cu:162); a plan whose map indexes a longer array says so (t2sc_plan_set_input_rows)
  T2_REQ(ctx, n_in == plan->n_in, "spconv shapes: x has %lld rows, the plan's neighbour map is over %lld", (long long)n_in, (long long)plan->n_in);
  if (plan->n_out == 0) return T2SC_OK;
  T2_REQ(ctx, x && w && y, "null tensor");
  T2_REQ(ctx, ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)y % 16 == 0), "x, w, y must be 16-byte aligned");
  T2_REQ(ctx, !ep || (((uintptr_t)ep->bias % 16 == 0) && ((uintptr_t)ep->residual % 16 == 0)), "epilogue bias and residual must be 16-byte aligned");
  EpiDev e = epi_dev(ep);
  if (e.skip_x) T2_REQ(ctx, e.skip_src && e.skip_cin % 8 == 0 && e.skip_rep > 0 && Co == (e.skip_cin / 8) * e.skip_rep,
                       "skip: Co=%d Cin=%d rep=%d", Co, e.skip_cin, e.skip_rep);
  i64 w_rows = plan->src ? 8ll * Co : Co;
  bool umma_ok = conv_umma_supported(dtype, Ci, Co, e);
  if (variant == T2SC_VARIANT_UMMA && !umma_ok)
    return t2sc_fail(ctx, T2SC_ERR_UNSUPPORTED, "tcgen05 variant needs fp16/bf16, Ci %% 64 == 0, Co %% 32 == 0 (Ci=%d Co=%d dtype=%d)", Ci, Co, dtype);
  bool use_umma = variant == T2SC_VARIANT_UMMA || variant == T2SC_VARIANT_UMMA_PAIR || (variant == T2SC_VARIANT_AUTO && umma_ok);
  // LayerNorm needs the whole output row in one accumulator: fused on the tcgen05 path when Co is one of its tile widths
  // (32, 64, 128, 256), else conv + bias first and LayerNorm -> activation -> residual -> skip in a row pass
  bool fuse_all = use_umma && (!e.ln || conv_umma_fuses_ln(Co));
  if (variant == T2SC_VARIANT_UMMA_PAIR) {
    if (!conv_umma2_supported(plan, dtype, Ci, Co, e))
      return t2sc_fail(ctx, T2SC_ERR_UNSUPPORTED, "two-SM tcgen05 variant needs fp16/bf16, a 256-row plan, Ci %% 64 == 0, Co %% 256 == 0 (Ci=%d Co=%d tile_rows=%d)", Ci, Co, plan->tile_rows);
    return conv_umma2_launch(ctx, plan, x, w, w_rows, e, y, dtype, n_in, Ci, Co, part);
  }
  if (fuse_all) return conv_umma_launch(ctx, plan, x, w, w_rows, e, y, dtype, n_in, Ci, Co, part);
  // the row pass below runs over all rows: a part of a plan cannot use it
  T2_REQ(ctx, part == T2SC_PART_ALL || !e.ln, "LayerNorm over Co=%d needs the row pass, which is not available for one part of a plan", Co);
  EpiDev first = e, rest = e;
  if (e.ln) {  // conv + bias now; LN -> act -> residual -> skip in the row pass
    first.ln = 0; first.act = 0; first.residual = nullptr; first.skip_x = nullptr; first.gamma = first.beta = nullptr;
    rest.bias = nullptr;
  }
  int rc = use_umma ? conv_umma_launch(ctx, plan, x, w, w_rows, first, y, dtype, n_in, Ci, Co, part)
                    : conv_simt_launch(ctx, plan, x, w, first, y, dtype, n_in, Ci, Co, part);
  if (rc != T2SC_OK || !e.ln) return rc;
  return row_epilogue_launch(ctx, y, rest, y, plan->n_out, Co, dtype);
}

extern "C" int t2sc_subm_conv_peers(t2sc_ctx* ctx, t2sc_plan* plan, const void* const* x_peers, const int64_t* rows_peers, int n_peers,
                                    int self_rank, const void* w, const t2sc_epilogue* ep, void* y, int dtype, int Ci, int Co) {
  return t2sc_subm_conv_peers_part(ctx, plan, nullptr, x_peers, rows_peers, n_peers, self_rank, w, ep, y, dtype, Ci, Co, T2SC_PART_ALL);
}

extern "C" int t2sc_subm_conv_peers_part(t2sc_ctx* ctx, t2sc_plan* plan, const uint32_t* peer_nbr, const void* const* x_peers,
                                         const int64_t* rows_peers, int n_peers, int self_rank, const void* w, const t2sc_epilogue* ep,
                                         void* y, int dtype, int Ci, int Co, int part) {
  T2_REQ(ctx, ctx && plan, "null context or plan");
  T2_REQ(ctx, part == T2SC_PART_ALL || part == T2SC_PART_INTERIOR || part == T2SC_PART_BOUNDARY, "part=%d", part);
  T2_REQ(ctx, n_peers >= 1 && n_peers <= 8 && x_peers && rows_peers, "n_peers=%d (1..8)", n_peers);
  for (int r = 0; r < n_peers; r++) T2_REQ(ctx, rows_peers[r] >= 0 && rows_peers[r] <= (1ll << 28), "peer %d has %lld rows (at most 2^28)", r, (long long)rows_peers[r]);
  T2_REQ(ctx, self_rank >= 0 && self_rank < n_peers, "self_rank=%d of %d", self_rank, n_peers);
  if (plan->n_out == 0) return T2SC_OK;
  T2_REQ(ctx, w && y, "null tensor");
  for (int r = 0; r < n_peers; r++) T2_REQ(ctx, x_peers[r] && (uintptr_t)x_peers[r] % 16 == 0, "peer array %d is null or not 16-byte aligned", r);
  EpiDev e = epi_dev(ep);
  if (!conv_umma_supported(dtype, Ci, Co, e) || (e.ln && !conv_umma_fuses_ln(Co)) || plan->src)
    return t2sc_fail(ctx, T2SC_ERR_UNSUPPORTED, "peer conv needs a submanifold plan, fp16/bf16, Ci %% 64 == 0, Co %% 32 == 0, LayerNorm only for Co in {32,64,128,256} (Ci=%d Co=%d dtype=%d)", Ci, Co, dtype);
  return conv_umma_launch(ctx, plan, x_peers[self_rank], w, Co, e, y, dtype, rows_peers[self_rank], Ci, Co, part, x_peers, rows_peers, n_peers,
                          self_rank, peer_nbr);
}

// ------------------------------------------------------------------------------------------ dense linear layer on the conv kernel
extern "C" int t2sc_linear(t2sc_ctx* ctx, const void* x, const void* w, const t2sc_epilogue* ep, void* y, int dtype,
                           int64_t n, int Ci, int Co) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && n < (1ll << 31) - 256, "n=%lld", (long long)n);
  T2_REQ(ctx, Ci > 0 && Co > 0, "linear shapes Ci=%d Co=%d", Ci, Co);
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, x && w && y, "null tensor");
  T2_REQ(ctx, ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)y % 16 == 0), "x, w, y must be 16-byte aligned");
  T2_REQ(ctx, !ep || (((uintptr_t)ep->bias % 16 == 0) && ((uintptr_t)ep->residual % 16 == 0)), "epilogue bias and residual must be 16-byte aligned");
  EpiDev e = epi_dev(ep);
  if (!conv_umma_supported(dtype, Ci, Co, e) || e.skip_x)
    return t2sc_fail(ctx, T2SC_ERR_UNSUPPORTED, "t2sc_linear runs on the tcgen05 path only: fp16/bf16, Ci %% 64 == 0, Co %% 32 == 0, no skip (Ci=%d Co=%d dtype=%d)", Ci, Co, dtype);
  if (!e.ln || conv_umma_fuses_ln(Co)) return linear_umma_launch(ctx, x, w, e, y, dtype, n, Ci, Co);
  EpiDev first = e, rest = e;       // LayerNorm over a row wider than one accumulator: GEMM + bias now, the rest in the row pass
  first.ln = 0; first.act = 0; first.residual = nullptr; first.gamma = first.beta = nullptr;
  rest.bias = nullptr;
  int rc = linear_umma_launch(ctx, x, w, first, y, dtype, n, Ci, Co);
  if (rc != T2SC_OK) return rc;
  return row_epilogue_launch(ctx, y, rest, y, n, Co, dtype);
}

// ------------------------------------------------------------------------------------------ barrier over peer-mapped flags
namespace {
struct FlagPtrs { int* p[8]; };
// One thread per rank.  Signal: entry `self` of rank t's array.  Wait: entry t of this rank's own array.
__global__ void k_peer_barrier(FlagPtrs f, int n, int self, int epoch, long long limit_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= n) return;
  __threadfence_system();                 // this GPU's earlier writes are visible to the peers before the flag is
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f.p[t] + self), "r"(epoch) : "memory");
  const int* mine = f.p[self] + t;
  unsigned long long t0, now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v - epoch >= 0) break;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if ((long long)(now - t0) > limit_ns) { atomicOr(status, 1024); break; }     // the peer never arrived: report, do not hang
    __nanosleep(200);
  }
}
}  // namespace

extern "C" int t2sc_peer_barrier(t2sc_ctx* ctx, void* const* flags_peers, int n_peers, int self_rank, int epoch, int timeout_ms) {
  T2_REQ(ctx, ctx && flags_peers, "null context or flags");
  T2_REQ(ctx, n_peers >= 1 && n_peers <= 8 && self_rank >= 0 && self_rank < n_peers, "n_peers=%d self_rank=%d", n_peers, self_rank);
  T2_REQ(ctx, timeout_ms > 0 && timeout_ms <= 60000, "timeout_ms=%d (1..60000)", timeout_ms);
  FlagPtrs f;
  for (int r = 0; r < 8; r++) {
    f.p[r] = r < n_peers ? (int*)flags_peers[r] : nullptr;
    if (r < n_peers) T2_REQ(ctx, f.p[r] && (uintptr_t)f.p[r] % 4 == 0, "flag array %d is null or unaligned", r);
  }
  T2_CUDA(ctx, cudaSetDevice(ctx->device));
  k_peer_barrier<<<1, 32, 0, ctx->stream>>>(f, n_peers, self_rank, epoch, (long long)timeout_ms * 1000000ll, ctx->status);
  T2_LAUNCHED(ctx);
  return T2SC_OK;
}

extern "C" int t2sc_row_epilogue(t2sc_ctx* ctx, const void* x, const t2sc_epilogue* ep, void* y, int64_t n, int C, int dtype) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, dtype == T2SC_F32 || dtype == T2SC_F16 || dtype == T2SC_BF16, "dtype %d", dtype);
  T2_REQ(ctx, n >= 0 && C > 0 && C % 4 == 0, "n=%lld C=%d (C must be a multiple of 4)", (long long)n, C);
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, x && y, "null tensor");
  return row_epilogue_launch(ctx, x, epi_dev(ep), y, n, C, dtype);
}

// ------------------------------------------------------------------------------------------ host-buffer operator
extern "C" int t2sc_subm_conv_host(t2sc_ctx* ctx, const int32_t* coords_host, int64_t n, int W, int H, int D,
                                   const void* x_host, const void* w_host, const void* bias_host, void* y_host,
                                   int dtype, int Ci, int Co) {
  T2_REQ(ctx, ctx != nullptr, "null context");
  T2_REQ(ctx, n >= 0 && n < (1ll << 31), "n=%lld", (long long)n);
  if (n == 0) return T2SC_OK;
  T2_REQ(ctx, coords_host && x_host && w_host && y_host, "null host buffer");
  T2_REQ(ctx, dtype == T2SC_F32 || dtype == T2SC_F16 || dtype == T2SC_BF16, "dtype %d", dtype);
  size_t es = dtype_size(dtype);
  int32_t* coords = nullptr; uint32_t* nbr = nullptr; int32_t* gray = nullptr;
  char *x = nullptr, *w = nullptr, *b = nullptr, *y = nullptr;
  t2sc_plan* plan = nullptr;
  int rc = T2SC_OK;
  auto cleanup = [&]() {
    if (plan) t2sc_plan_destroy(ctx, plan);
    t2_free(ctx, coords); t2_free(ctx, nbr); t2_free(ctx, gray); t2_free(ctx, x); t2_free(ctx, w); t2_free(ctx, b); t2_free(ctx, y);
  };
#define HOST_TRY(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { cleanup(); return t2sc_fail(ctx, T2SC_ERR_CUDA, "CUDA %s: %s", #call, cudaGetErrorString(e_)); } } while (0)
  HOST_TRY(cudaSetDevice(ctx->device));
  HOST_TRY(t2_alloc(ctx, &coords, (size_t)n * 4));
  HOST_TRY(t2_alloc(ctx, &nbr, (size_t)n * 27));
  HOST_TRY(t2_alloc(ctx, &gray, (size_t)n));
  HOST_TRY(t2_alloc(ctx, &x, (size_t)n * Ci * es));
  HOST_TRY(t2_alloc(ctx, &w, (size_t)Co * 27 * Ci * es));
  HOST_TRY(t2_alloc(ctx, &y, (size_t)n * Co * es));
  HOST_TRY(cudaMemcpyAsync(coords, coords_host, (size_t)n * 16, cudaMemcpyHostToDevice, ctx->stream));
  HOST_TRY(cudaMemcpyAsync(x, x_host, (size_t)n * Ci * es, cudaMemcpyHostToDevice, ctx->stream));
  HOST_TRY(cudaMemcpyAsync(w, w_host, (size_t)Co * 27 * Ci * es, cudaMemcpyHostToDevice, ctx->stream));
  if (bias_host) {
    HOST_TRY(t2_alloc(ctx, &b, (size_t)Co * es));
    HOST_TRY(cudaMemcpyAsync(b, bias_host, (size_t)Co * es, cudaMemcpyHostToDevice, ctx->stream));
  }
  if ((rc = t2sc_build_neighbors(ctx, coords, n, W, H, D, nbr, gray, nullptr)) != T2SC_OK) { cleanup(); return rc; }
  if ((rc = t2sc_plan_create(ctx, nbr, gray, n, nullptr, n, 0, 0, &plan)) != T2SC_OK) { cleanup(); return rc; }
  t2sc_epilogue ep; memset(&ep, 0, sizeof(ep)); ep.bias = b;
  if ((rc = t2sc_subm_conv(ctx, plan, x, w, &ep, y, dtype, n, Ci, Co, T2SC_VARIANT_AUTO)) != T2SC_OK) { cleanup(); return rc; }
  HOST_TRY(cudaMemcpyAsync(y_host, y, (size_t)n * Co * es, cudaMemcpyDeviceToHost, ctx->stream));
  HOST_TRY(ctx_wait(ctx));
#undef HOST_TRY
  cleanup();
  int st = 0;
  return t2sc_device_status(ctx, &st);
}
