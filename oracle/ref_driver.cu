// Test infrastructure: a C-ABI harness around the REFERENCE's own CUDA implementation of the path
// (trellis2-cuda src/spconv.cu, src/sdec.cu, src/ops.cu, src/core.cu), compiled from the reference's
// sources where they lie by oracle/Makefile into oracle/_ref/libt2ref.so.  Nothing from those sources
// is copied here; this file only calls their public functions with host buffers so that Python tests
// and the golden-vector generator can run the reference on a GPU box.  Never linked into the product.
#define private public          // SDecoder::c2s is a private member; the harness calls it directly
#include "models.h"
#undef private
#include "sdec.cu"              // the reference's translation unit itself (found through -I): its kernels
                                // k_gather_rows / k_add_skip are launched below, which needs one TU
#include <stdexcept>
#include <string>

static std::string g_err;
#define GUARD(...) try { __VA_ARGS__; return 0; } catch (const std::exception& e) { g_err = e.what(); return -1; }

extern "C" const char* ref_last_error() { return g_err.c_str(); }

// build_neighbors (src/spconv.cu:38-54) + optional valid(B1) (src/spconv.cu:65-75)
extern "C" int ref_build_neighbors(const int* coords, int n, int W, int H, int D, uint32_t* nbr, int* gray, int* sorted,
                                   int B1, int* seg, int* list, int* list_len) {
  GUARD({
    Tensor c = from_host(coords, {n, 4}, I32);
    SpConvCache cache = build_neighbors(c, W, H, D);
    auto a = to_host(cache.nbr); memcpy(nbr, a.data(), a.size());
    auto b = to_host(cache.gray); memcpy(gray, b.data(), b.size());
    auto s = to_host(cache.sorted); memcpy(sorted, s.data(), s.size());
    if (B1 > 0) {
      auto& vk = cache.valid(B1);
      auto sg = to_host(vk.second); memcpy(seg, sg.data(), sg.size());
      int L = ((int*)sg.data())[sg.size() / 4 - 1];
      auto li = to_host(vk.first); memcpy(list, li.data(), (size_t)L * 4);
      *list_len = L;
    }
  })
}

// subm_conv (src/spconv.cu:160-175), fp16 only.  reps > 0 additionally times `reps` calls of the conv
// alone (neighbour map built once) and of build_neighbors alone with cudaEvents, as apps/parity.cu:157-160.
extern "C" int ref_subm_conv(const int* coords, int n, const void* x, const void* w, const void* bias, int Ci, int Co,
                             void* y, int reps, float* conv_ms, float* nbr_ms) {
  GUARD({
    Tensor c = from_host(coords, {n, 4}, I32), xt = from_host(x, {n, Ci}, F16), wt = from_host(w, {Co, 27, Ci}, F16), bt;
    if (bias) bt = from_host(bias, {Co}, F16);
    SpConvCache cache = build_neighbors(c, 4096, 4096, 4096);
    Tensor yt = subm_conv(xt, wt, bias ? &bt : nullptr, cache);
    auto h = to_host(yt); memcpy(y, h.data(), h.size());
    if (reps > 0) {
      Timer tm; dsync(); tm.start();
      for (int i = 0; i < reps; i++) yt = subm_conv(xt, wt, bias ? &bt : nullptr, cache);
      *conv_ms = tm.ms() / reps;
      dsync(); tm.start();
      for (int i = 0; i < reps; i++) { SpConvCache c2 = build_neighbors(c, 4096, 4096, 4096); }
      *nbr_ms = tm.ms() / reps;
    }
  })
}

// SDecoder::c2s (src/sdec.cu:45-57): sub fp16 [n,8] -> child coords / src (capacity 8n), *m children
extern "C" int ref_c2s(const int* coords, int n, const void* sub, int* child_coords, int* src, int* m) {
  GUARD({
    SDecoder dec; SDecoder::Level lv;
    lv.coords = from_host(coords, {n, 4}, I32);
    Tensor st = from_host(sub, {n, 8}, F16);
    SDecoder::Level ch = dec.c2s(lv, st);
    *m = (int)ch.coords.size(0);
    auto a = to_host(ch.coords); memcpy(child_coords, a.data(), a.size());
    auto b = to_host(ch.src); memcpy(src, b.data(), b.size());
  })
}

// conv -> [layer_norm] -> [act_] -> [add_ residual], each a separate reference kernel on fp16 tensors
// (src/ops.cu:17-113); gamma / beta fp32 or NULL; act: 0 none, 1 SiLU, 2 GELU-tanh, 3 GELU-erf
extern "C" int ref_conv_block(const int* coords, int n, const void* x, const void* w, const void* bias, int Ci, int Co,
                              int ln, const float* gamma, const float* beta, float eps, int act, const void* residual, void* y) {
  GUARD({
    Tensor c = from_host(coords, {n, 4}, I32), xt = from_host(x, {n, Ci}, F16), wt = from_host(w, {Co, 27, Ci}, F16), bt, gt, bet;
    if (bias) bt = from_host(bias, {Co}, F16);
    SpConvCache cache = build_neighbors(c, 4096, 4096, 4096);
    Tensor h = subm_conv(xt, wt, bias ? &bt : nullptr, cache);
    if (ln) {
      if (gamma) gt = from_host(gamma, {Co}, F32);
      if (beta) bet = from_host(beta, {Co}, F32);
      h = layer_norm(h, gamma ? &gt : nullptr, beta ? &bet : nullptr, eps);
    }
    if (act) act_(h, act == 1 ? SILU : act == 2 ? GELU_TANH : GELU_ERF);
    if (residual) { Tensor r = from_host(residual, {n, Co}, F16); add_(h, r); }
    auto o = to_host(h); memcpy(y, o.data(), o.size());
  })
}

// The sparse tail of SDecoder::up (src/sdec.cu:76-84) with the subdivision logits given:
// conv1 (Ci -> 8*Cc at parent level) -> c2s -> k_gather_rows -> layer_norm(no affine) -> SiLU ->
// conv2 (Cc -> Cc at child level) -> k_add_skip.  Outputs: hc = gathered conv1 rows [m,Cc], out [m,Cc].
extern "C" int ref_up_tail(const int* coords, int n, const void* x, const void* sub, const void* w1, const void* b1,
                           const void* w2, const void* b2, int Ci, int Cc, void* hc_out, void* out, int* m_out) {
  GUARD({
    SDecoder dec; SDecoder::Level lv;
    lv.coords = from_host(coords, {n, 4}, I32);
    lv.nb = std::make_shared<SpConvCache>(build_neighbors(lv.coords, 4096, 4096, 4096));
    Tensor xt = from_host(x, {n, Ci}, F16), st = from_host(sub, {n, 8}, F16);
    Tensor w1t = from_host(w1, {8 * Cc, 27, Ci}, F16), b1t = from_host(b1, {8 * Cc}, F16);
    Tensor w2t = from_host(w2, {Cc, 27, Cc}, F16), b2t = from_host(b2, {Cc}, F16);
    Tensor h = subm_conv(xt, w1t, &b1t, *lv.nb);
    SDecoder::Level ch = dec.c2s(lv, st);
    i64 m = ch.coords.size(0); *m_out = (int)m;
    Tensor hc = empty({m, Cc}, F16);
    k_gather_rows<<<cdiv(m * Cc, 256), 256, 0, stream()>>>(h.ptr<f16>(), ch.src.ptr<int>(), m, Cc, hc.ptr<f16>());
    auto a = to_host(hc); memcpy(hc_out, a.data(), a.size());
    h = layer_norm(hc, nullptr, nullptr, 1e-6f);
    act_(h, SILU);
    h = subm_conv(h, w2t, &b2t, *ch.nb);
    k_add_skip<<<cdiv(m * Cc, 256), 256, 0, stream()>>>(h.ptr<f16>(), xt.ptr<f16>(), ch.src.ptr<int>(), m, Cc, Ci, Cc / (Ci / 8));
    auto o = to_host(h); memcpy(out, o.data(), o.size());
  })
}
