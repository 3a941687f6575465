// Test infrastructure: the binding a maintainer of trellis2-cuda would add to use libt2sc.so.  This translation unit
// REPLACES the reference's src/spconv.cu: it implements the reference's own header src/spconv.h (build_neighbors,
// SpConvCache::valid, spconv_cfg, subm_conv) on the reference's Tensor type by calling the t2sc C ABI.  oracle/Makefile
// compiles it together with the reference's unchanged src/sdec.cu, src/ops.cu, src/gemm.cu, src/core.cu into
// oracle/_ref/libt2ref_dropin.so, so the reference's decoder code runs on this library's kernels.
#include "spconv.h"          // the reference's header (found through -I<reference>/src)
#include "t2sc.h"
#include <algorithm>

static t2sc_ctx* ctx() {     // one context on the reference's global stream (src/core.cu:20-28)
  static t2sc_ctx* c = [] {
    t2sc_ctx* p = nullptr;
    REQ(t2sc_ctx_create(0, stream(), &p) == 0, "%s", t2sc_last_error(nullptr));
    return p;
  }();
  return c;
}
#define T2(call) REQ((call) == 0, "%s", t2sc_last_error(ctx()))       // status code -> the reference's exception

SpConvCache build_neighbors(const Tensor& coords, int W, int H, int D) {
  SpConvCache c; int n = (int)coords.size(0); c.N = n;
  c.nbr = empty({n, 27}, I32); c.gray = empty({n}, I32); c.sorted = empty({n}, I32);
  T2(t2sc_build_neighbors(ctx(), coords.ptr<int32_t>(), n, W, H, D, c.nbr.ptr<uint32_t>(), c.gray.ptr<int32_t>(), c.sorted.ptr<int32_t>()));
  return c;
}

const std::pair<Tensor, Tensor>& SpConvCache::valid(int B1) {
  auto it = vk.find(B1); if (it != vk.end()) return it->second;
  int nb = cdiv(N, B1);
  Tensor seg = empty({nb + 1}, I32), list = empty({std::max(27 * nb, 1)}, I32); int64_t total = 0;
  T2(t2sc_valid_taps(ctx(), gray.ptr<int32_t>(), sorted.ptr<int32_t>(), N, B1, seg.ptr<int32_t>(), list.ptr<int32_t>(), &total));
  return vk.emplace(B1, std::make_pair(list.slice0(0, std::max<int64_t>(total, 1)), seg)).first->second;
}

SpConvCfg spconv_cfg(int, int, int) { return {128, 64, 1}; }

// The schedule lives as long as the cache: it is parked in the cache's own map under a key valid() never uses, inside
// a Tensor whose deleter destroys the plan.
static t2sc_plan* plan_of(SpConvCache& c) {
  auto it = c.vk.find(-1);
  if (it != c.vk.end()) return (t2sc_plan*)it->second.first.p;
  t2sc_plan* p = nullptr;
  T2(t2sc_plan_create(ctx(), c.nbr.ptr<uint32_t>(), c.gray.ptr<int32_t>(), c.N, nullptr, c.N, 0, 0, &p));
  Tensor holder; holder.p = p; holder.dt = U8; holder.sh = {0};
  holder.own = std::shared_ptr<void>((void*)p, [](void* q) { t2sc_plan_destroy(ctx(), (t2sc_plan*)q); });
  c.vk.emplace(-1, std::make_pair(holder, Tensor()));
  return p;
}

Tensor subm_conv(const Tensor& x, const Tensor& w, const Tensor* b, SpConvCache& c) {
  int N = (int)x.size(0), Ci = (int)x.size(1), Co = (int)w.size(0);
  REQ(x.dt == F16 && w.dt == F16 && w.size(1) == 27 && w.size(2) == Ci && Ci % 32 == 0 && N == c.N, "spconv shapes");
  Tensor bb; if (b) bb = b->dt == F16 ? *b : cast(*b, F16);
  t2sc_epilogue ep = {}; ep.bias = b ? bb.p : nullptr;
  Tensor y = empty({N, Co}, F16);
  T2(t2sc_subm_conv(ctx(), plan_of(c), x.p, w.p, &ep, y.p, T2SC_F16, N, Ci, Co, T2SC_VARIANT_AUTO));
  return y;
}
