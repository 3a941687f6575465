/*
 * t2sc — B200 (sm_100a) sparse-convolution operators behind a plain C ABI.
 *
 * Drop-in boundary for the sparse-convolution path of suvadityamuk/trellis2-cuda.  Every entry point
 * names the reference interface it replaces (paths are relative to that project).  All pointers are
 * DEVICE pointers owned by the caller unless a parameter is suffixed `_host`; all work is enqueued on
 * the context's stream; every function returns a status (0 = ok, negative = error) and never throws.
 * After a non-zero return, t2sc_last_error() gives the message (the reference's REQ / CK messages,
 * src/core.h:15-17, surfaced the way apps/t2lib.cu:14-23 surfaces them: code + last-error string).
 *
 * Conventions shared with the reference:
 *   coords   int32 [N,4] = (batch, x, y, z), unique rows, 16-byte aligned      (src/spconv.h:12)
 *   features [N,C] row-major, fp16 / bf16 / fp32 (the reference is fp16-only; dtype is a parameter here)
 *   weights  [Co,27,Ci] = checkpoint weight [Co,3,3,3,Ci] viewed flat, tap v = kx*9 + ky*3 + kz with kx
 *            applied to coords column 1                                           (src/spconv.h:15)
 *   nbr      uint32 [N,27], 0xffffffff = absent; gray int32 [N] 27-bit presence mask (src/spconv.h:8)
 */
#ifndef T2SC_H_
#define T2SC_H_
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct t2sc_ctx t2sc_ctx;
typedef struct t2sc_plan t2sc_plan;

/* dtype codes: same numeric values as the reference's `enum DT` (src/core.h:22) for the float types */
enum { T2SC_F32 = 0, T2SC_F16 = 1, T2SC_BF16 = 2, T2SC_U8 = 5 };
/* activations: the reference's `enum Act` (src/ops.h:11) shifted by one so that 0 means none */
enum { T2SC_ACT_NONE = 0, T2SC_ACT_SILU = 1, T2SC_ACT_GELU_TANH = 2, T2SC_ACT_GELU_ERF = 3 };
/* status codes */
enum { T2SC_OK = 0, T2SC_ERR_ARG = -1, T2SC_ERR_CUDA = -2, T2SC_ERR_UNSUPPORTED = -3, T2SC_ERR_DEVICE = -4 };
/* conv kernel variants (t2sc_subm_conv `variant`): AUTO picks tcgen05 whenever the shape allows it */
enum { T2SC_VARIANT_AUTO = 0, T2SC_VARIANT_SIMT = 1, T2SC_VARIANT_UMMA = 2,
       T2SC_VARIANT_UMMA_PAIR = 3 /* two-SM tcgen05 (cta_group::2): needs a 256-row plan and Co % 256 == 0 */ };

/* ---- context.  Replaces the reference's process-wide stream and allocator (src/core.cu:20-40):
 * one context per device; `stream` is a cudaStream_t (NULL = the context creates its own
 * non-blocking stream).  Scratch (hash table, sort buffers, plans) comes from the device's
 * stream-ordered memory pool, as in the reference. */
int t2sc_ctx_create(int device, void* stream, t2sc_ctx** out);
int t2sc_ctx_destroy(t2sc_ctx* ctx);
int t2sc_ctx_sync(t2sc_ctx* ctx);                      /* replaces dsync(), src/core.cu:29 */
const char* t2sc_last_error(const t2sc_ctx* ctx);      /* ctx may be NULL: error of the last failed create */
int64_t t2sc_launch_count(const t2sc_ctx* ctx);        /* kernels of this library launched so far */
/* syncs; *status_host non-zero (and T2SC_ERR_DEVICE returned) = a bounded device-side wait gave up (bits 0-9 except 8)
 * or a neighbour-map entry pointed outside its feature array (bit 8); the word is cleared by the call */
int t2sc_device_status(t2sc_ctx* ctx, int* status_host);

/* ---- neighbour maps.  Replaces build_neighbors (src/spconv.cu:38-54; kernels :14-36).
 * Writes nbr [n,27], gray [n] and, when `sorted` is not NULL, the reference's row order: the stable
 * ascending argsort of the gray->binary key (src/spconv.cu:34,47-52).  Duplicate coordinates resolve to
 * the lowest row index (the reference leaves it to a race).  n = 0 returns at once. */
int t2sc_build_neighbors(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                         uint32_t* nbr, int32_t* gray, int32_t* sorted);

/* Neighbour rows of the row range [row_lo, row_hi) against the hash of all n rows (global row indices in
 * nbr): the map one rank of a Morton-range partition builds for the rows it owns.  The reference is
 * single-GPU and has no counterpart; semantics per row are those of build_neighbors (src/spconv.cu:22-36). */
int t2sc_build_neighbors_range(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                               int64_t row_lo, int64_t row_hi, uint32_t* nbr, int32_t* gray);

/* Rows of arbitrary coordinates: rows[q] = index of the row of coords [n,4] equal to queries[q] = (b,x,y,z), or 0xffffffff
 * (also for a query outside [0,W)x[0,H)x[0,D) or with a negative batch index).  The lookup the reference's other users
 * of a voxel hash need: vhash_find (src/mesh.cu:7-19), which the dual-grid quad search calls per edge (src/mesh.cu:54-72),
 * and the hash half of the grid-sample neighbour build (src/glb.cu:545-552).  Same table and duplicate rule (lowest row
 * index) as t2sc_build_neighbors; queries int32 [m,4], 16-byte aligned. */
int t2sc_voxel_lookup(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                      const int32_t* queries, int64_t m, uint32_t* rows);

/* Neighbour maps for callers that must not allocate.  (No counterpart in the reference, whose
 * build_neighbors always allocates.)  Same nbr / gray results as t2sc_build_neighbors, but the hash table is
 * a fixed 2 MiB array that is part of the library image, so this call performs no cudaMalloc, cudaFree or
 * pool allocation of any kind; it is meant for hosts that have given the whole device to an arena of their
 * own, or that forbid allocation once start-up is over, where a cudaMalloc can fail or force a device-wide
 * synchronisation.  Limits and rules:
 *   - at most T2SC_STATIC_MAX_ROWS rows; more is refused with T2SC_ERR_UNSUPPORTED and a message;
 *   - no `sorted` output (the reference row order needs sort scratch: use t2sc_build_neighbors for it);
 *   - every GPU that loads the library carries the 2 MiB array until the process exits;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call during start-up, before any stream capture;
 *   - all calls on a device share the one array: it is cleared at the start of each call, and two calls
 *     whose kernels overlap on the GPU (different streams or contexts) corrupt each other - serialise them.
 * The context itself (t2sc_ctx_create) is made at start-up, when allocating is still allowed. */
#define T2SC_STATIC_MAX_ROWS 65536
int t2sc_build_neighbors_static(t2sc_ctx* ctx, const int32_t* coords, int64_t n, int W, int H, int D,
                                uint32_t* nbr, int32_t* gray);

/* Replaces SpConvCache::valid (src/spconv.cu:56-75).  seg [ceil(n/B1)+1] exclusive offsets, list
 * [27*ceil(n/B1)] ascending taps present in each block of B1 consecutive `sorted` rows; *total_host
 * receives seg[nb] (one host sync, as in the reference). */
int t2sc_valid_taps(t2sc_ctx* ctx, const int32_t* gray, const int32_t* sorted, int64_t n, int B1,
                    int32_t* seg, int32_t* list, int64_t* total_host);

/* ---- 2x subdivision maps.  Replaces SDecoder::c2s (src/sdec.cu:45-57; kernels :21-33).
 * `sub` is [n,8]: fp16 logits (kept iff > 0, T2SC_F16), bf16 logits (T2SC_BF16) or uint8 flags (kept iff
 * non-zero, T2SC_U8).  count: off [n+1] exclusive child offsets, *m_host = number of children (one host
 * sync, as in the reference).  emit: child_coords [m,4] and src [m] = parent*8 + slot, (parent,slot)
 * ascending, child = (b, 2x+(s&1), 2y+(s>>1&1), 2z+(s>>2&1)). */
int t2sc_subdivide_count(t2sc_ctx* ctx, const void* sub, int sub_dtype, int64_t n, int32_t* off, int64_t* m_host);
int t2sc_subdivide_emit(t2sc_ctx* ctx, const void* sub, int sub_dtype, const int32_t* coords, const int32_t* off,
                        int64_t n, int32_t* child_coords, int32_t* src);

/* Replaces k_gather_rows (src/sdec.cu:34-37): y[r,:] = x.view(-1,C)[src[r],:]. */
int t2sc_gather_rows(t2sc_ctx* ctx, const void* x, const int32_t* src, int64_t m, int C, int dtype, void* y);
/* Replaces k_add_skip (src/sdec.cu:39-43): h[r,c] += x[src[r]>>3, (src[r]&7)*(Cin/8) + c/rep]. */
int t2sc_add_skip(t2sc_ctx* ctx, void* h, const void* x, const int32_t* src, int64_t m, int Co, int Cin, int rep, int dtype);

/* ---- execution plan for one neighbour map (replaces the scheduling half of SpConvCache: `sorted`
 * and valid(), src/spconv.h:6-11).  Orders the output rows so that rows of one tile share
 * most taps, and records each tile's tap mask.  `src` = NULL plans a submanifold conv over the n_rows
 * rows of nbr/gray; src [m] (from t2sc_subdivide_emit) plans the 2x-subdivision conv: m child rows,
 * each using its parent's neighbour row and the weight rows of its slot.  block_rows > 0 keeps the
 * ordering local to runs of that many caller rows (cache locality on large maps); 0 = library default
 * (one global sort up to 262,144 rows, runs of 65,536 rows above).
  * tile_rows is 128 or 256 (0 = library default 128; 256: two 128-row accumulators share every weight slab).
 * The plan borrows nbr and src: they must outlive it. */
int t2sc_plan_create(t2sc_ctx* ctx, const uint32_t* nbr, const int32_t* gray, int64_t n_rows,
                     const int32_t* src, int64_t m, int64_t block_rows, int tile_rows, t2sc_plan** out);
int t2sc_plan_destroy(t2sc_ctx* ctx, t2sc_plan* plan);
/* Declares that the entries of the plan's neighbour map index a feature array of n_in >= n_rows rows (one rank of a
 * partitioned scene: owned rows first, the halo rows of its peers appended).  Without it n_in == n_rows, which is what
 * the reference requires of subm_conv (REQ N == c.N, src/spconv.cu:162). */
int t2sc_plan_set_input_rows(t2sc_ctx* ctx, t2sc_plan* plan, int64_t n_in);
/* The plan keeps its own copy of the map in tile order (what the tcgen05 kernel reads; later changes to nbr are not seen by
 * it).  Its entries are checked against the rows of the feature array once per n_in: entries at or above n_in are made
 * absent and reported by t2sc_device_status.  The first conv with a given n_in does that; this call does it ahead of time,
 * so that the conv launches nothing but the conv. */
int t2sc_plan_check(t2sc_ctx* ctx, t2sc_plan* plan, int64_t n_in);
/* Plan for one rank of a partitioned scene (no counterpart in the reference, which is single-GPU).  nbr is the rank's
 * LOCAL map over its n_rows owned rows: entries below n_own are owned rows, entries from n_own up are halo rows of its
 * peers appended behind them.  Rows none of whose taps reads a halo row form the interior part of the plan, the others
 * the boundary part; the boundary tiles come last.  The interior part can run (T2SC_PART_INTERIOR) while the halo rows are
 * still on their way, the boundary part (T2SC_PART_BOUNDARY) once they have landed.  Together the two parts write every
 * output row exactly once, with the bits t2sc_subm_conv gives on an unsplit plan. */
int t2sc_plan_create_split(t2sc_ctx* ctx, const uint32_t* nbr, const int32_t* gray, int64_t n_rows, int64_t n_own,
                           int64_t block_rows, int tile_rows, t2sc_plan** out);
enum { T2SC_PART_ALL = 0, T2SC_PART_INTERIOR = 1, T2SC_PART_BOUNDARY = 2 };
/* tiles of the two parts (syncs); a plan not made by t2sc_plan_create_split is all interior */
int t2sc_plan_parts(t2sc_ctx* ctx, t2sc_plan* plan, int64_t* interior_tiles, int64_t* boundary_tiles);
/* tiles, sum over tiles of rows*popcount(tile mask), sum over rows of popcount(row mask) (syncs) */
int t2sc_plan_stats(t2sc_ctx* ctx, t2sc_plan* plan, int64_t* tiles, int64_t* computed_taps, int64_t* active_taps);
/* internal row order of the plan, int32 [m] (for inspection and tests) */
int t2sc_plan_order(t2sc_ctx* ctx, t2sc_plan* plan, int32_t* order_out);

/* ---- fused epilogue, applied in this order with the reference's rounding points:
 * round(acc) -> + bias (storage dtype, rounded; src/spconv.cu:141-143) -> LayerNorm over Co in fp32,
 * rounded (src/ops.cu:17-76) -> activation, rounded (src/ops.cu:79-90) -> + residual, rounded
 * (add_, src/ops.cu:105-113) -> + skip (k_add_skip, src/sdec.cu:39-43). */
typedef struct {
  const void* bias;        /* [Co] (subdivision conv: [8*Co]) in the feature dtype, or NULL; bias and residual 16-byte aligned */
  int ln;                  /* 0 = none, 1 = LayerNorm over the Co output channels */
  const float* ln_gamma;   /* fp32 [Co] or NULL (no affine) */
  const float* ln_beta;    /* fp32 [Co] or NULL */
  float ln_eps;
  int act;                 /* T2SC_ACT_* */
  const void* residual;    /* [n_out,Co] feature dtype or NULL */
  const void* skip_x;      /* subdivision skip: parent features [n_parent, skip_cin] or NULL */
  const int32_t* skip_src; /* [n_out] parent*8+slot */
  int skip_cin, skip_rep;
} t2sc_epilogue;

/* Replaces subm_conv (src/spconv.cu:160-175; kernel :91-150) and, with a subdivision plan, the
 * conv1 -> k_gather_rows pair of SDecoder::up (src/sdec.cu:76-80) computing kept children only.
 * x [n_in,Ci], w [w_rows,27,Ci] (w_rows = Co, or 8*Co for a subdivision plan), y [n_out,Co] in the
 * caller's row order; Ci % 32 == 0 as in the reference.  n_in must equal the rows the plan was made for (the
 * reference's REQ N == c.N, src/spconv.cu:162; see t2sc_plan_set_input_rows).  A map entry that points at or past
 * row n_in is read as an absent neighbour and reported by t2sc_device_status (T2SC_ERR_DEVICE).  ep may be NULL. */
int t2sc_subm_conv(t2sc_ctx* ctx, t2sc_plan* plan, const void* x, const void* w, const t2sc_epilogue* ep,
                   void* y, int dtype, int64_t n_in, int Ci, int Co, int variant);

/* t2sc_subm_conv over one part of a plan (T2SC_PART_*): the rows of the other part are left untouched in y.  n_in is the
 * index space of the plan's map as for t2sc_subm_conv; T2SC_PART_INTERIOR of a split plan reads rows below n_own only, so
 * x may end there (a rank whose boundary tiles gather the halo rows from peer memory never copies them). */
int t2sc_subm_conv_part(t2sc_ctx* ctx, t2sc_plan* plan, const void* x, const void* w, const t2sc_epilogue* ep,
                        void* y, int dtype, int64_t n_in, int Ci, int Co, int variant, int part);

/* The same operator for one rank of a Morton-range partition, reading its inputs straight from its peers' memory: the
 * gather of the conv kernel itself is the halo exchange (no pack kernel, no collective in the data path).  x_peers[r]
 * is rank r's feature array [rows_r, Ci], mapped into this process (CUDA IPC / symmetric memory; x_peers[self_rank] is
 * the local array: taps whose rows are all local, nearly all of them, take the ordinary gather path); rows_peers[r] is
 * the number of rows of that array.  Every present entry of the plan's neighbour map is
 * (owner rank << T2SC_PEER_SHIFT) | (row within the owner's array), 0xffffffff = absent; an entry naming an owner
 * >= n_peers or a row >= rows_peers[owner] is read as absent and reported by t2sc_device_status.  At most 8 peers, at
 * most 2^28 rows per rank.  The caller orders the ranks: a layer may start only when every peer has finished writing
 * the array it reads.  Only the tcgen05 path (fp16 / bf16, Ci % 64 == 0, Co % 32 == 0).  The reference is single-GPU
 * and has no counterpart. */
#define T2SC_PEER_SHIFT 28
int t2sc_subm_conv_peers(t2sc_ctx* ctx, t2sc_plan* plan, const void* const* x_peers, const int64_t* rows_peers, int n_peers,
                         int self_rank, const void* w, const t2sc_epilogue* ep, void* y, int dtype, int Ci, int Co);

/* t2sc_subm_conv_peers over one part of a plan, reading the entries of `peer_nbr` [n_rows,27] (the (owner, row) form
 * of the map the plan was made for; NULL = the plan's own map) instead of the plan's map.  With a split plan made over the
 * local map: t2sc_subm_conv_part(INTERIOR) on the local map, then this call with T2SC_PART_BOUNDARY, so that only the
 * boundary tiles pay for the peer-memory gather. */
int t2sc_subm_conv_peers_part(t2sc_ctx* ctx, t2sc_plan* plan, const uint32_t* peer_nbr, const void* const* x_peers,
                              const int64_t* rows_peers, int n_peers, int self_rank, const void* w, const t2sc_epilogue* ep,
                              void* y, int dtype, int Ci, int Co, int part);

/* Barrier between the ranks of one node through flags in peer-mapped memory, enqueued on the context's stream (no
 * counterpart in the reference).  flags_peers[r] is rank r's flag array (int32, at least n_peers entries, zero before the
 * first use) mapped into this process.  The kernel stores `epoch` into entry self_rank of every rank's array (plain
 * peer stores, release at system scope) and then waits until all entries of its own array have reached `epoch`
 * (epochs must grow by one per call, starting at 1).  The wait is bounded: after timeout_ms it gives up, sets the
 * context's status word (t2sc_device_status -> T2SC_ERR_DEVICE) and the kernel returns, so a peer that has died
 * leaves this GPU usable.  At most 8 ranks. */
int t2sc_peer_barrier(t2sc_ctx* ctx, void* const* flags_peers, int n_peers, int self_rank, int epoch, int timeout_ms);

/* Replaces layer_norm + act_ + add_ (src/ops.cu:17-113) as one pass over [n,C]; any of the three may
 * be disabled (ln = 0, act = 0, residual = NULL).  In place when y == x. */
int t2sc_row_epilogue(t2sc_ctx* ctx, const void* x, const t2sc_epilogue* ep, void* y, int64_t n, int C, int dtype);

/* Replaces linear (src/gemm.cu:25-64, a cuBLAS call in the reference) for the MLP half of the decoder's ConvNeXt block
 * (src/sdec.cu:62-65: Linear C -> 4C, SiLU, Linear 4C -> C, add_), with the ops around it fused: y [n,Co] = epilogue(x [n,Ci] .
 * w [Co,Ci]^T).  It runs on the conv's tcgen05 kernel (one tap whose gather reads the row's own input row) and shares its
 * epilogue: bias, LayerNorm, activation, residual in t2sc_epilogue's order.  fp16 / bf16, Ci % 64 == 0, Co % 32 == 0. */
int t2sc_linear(t2sc_ctx* ctx, const void* x, const void* w, const t2sc_epilogue* ep, void* y, int dtype,
                int64_t n, int Ci, int Co);

/* Whole operator with HOST buffers, as apps/parity.cu:148-167 drives it: copies coords / x / w / bias
 * in, builds the neighbour map, runs the conv, copies y back and synchronises.  bias_host may be NULL. */
int t2sc_subm_conv_host(t2sc_ctx* ctx, const int32_t* coords_host, int64_t n, int W, int H, int D,
                        const void* x_host, const void* w_host, const void* bias_host, void* y_host,
                        int dtype, int Ci, int Co);

#ifdef __cplusplus
}
#endif
#endif /* T2SC_H_ */
