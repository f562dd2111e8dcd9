// The C ABI: argument checks and conversion of every failure into a return code.  No entry point throws or aborts; none
// falls back to host arithmetic — if the device or a kernel is unusable the call fails with a message.
#include <new>

#include "hb_common.cuh"
#include "hb_kernels.h"

namespace {
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool pdl_on(const hb_ctx* c) { return !(c->flags & HB_FLAG_NO_PDL); }
}  // namespace

#define HB_CTX(ctx) \
  do { if (!(ctx)) return HB_ERR_INVALID; } while (0)
#define HB_PTR(ctx, p) HB_REQUIRE(ctx, (p) != nullptr, HB_ERR_INVALID, "%s: %s is NULL", __func__, #p)
#define HB_ALIGN16(ctx, p) HB_REQUIRE(ctx, hb_aligned((p), 16), HB_ERR_INVALID, "%s: %s must be 16-byte aligned", __func__, #p)

extern "C" {

int hb_create(const hb_config* cfg, hb_ctx** out) {
  if (!out) return HB_ERR_INVALID;
  *out = nullptr;
  hb_ctx* c = new (std::nothrow) hb_ctx();
  if (!c) return HB_ERR_CUDA;
  c->device = cfg ? cfg->device : 0;
  c->max_ctas = cfg ? cfg->max_ctas : 0;
  c->flags = cfg ? cfg->flags : 0;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || c->device < 0 || c->device >= n) { delete c; cudaGetLastError(); return HB_ERR_NO_DEVICE; }
  cudaDeviceProp prop;
  if (cudaSetDevice(c->device) != cudaSuccess || cudaGetDeviceProperties(&prop, c->device) != cudaSuccess) { delete c; cudaGetLastError(); return HB_ERR_NO_DEVICE; }
  if (prop.major != 10) { delete c; return HB_ERR_NO_DEVICE; }          // the kernels are sm_100a only
  c->sm_count = prop.multiProcessorCount;
  c->smem_optin = (int)prop.sharedMemPerBlockOptin;
  if (cudaMalloc(&c->dev_err, 256) != cudaSuccess || cudaMemset(c->dev_err, 0, 256) != cudaSuccess) { delete c; cudaGetLastError(); return HB_ERR_CUDA; }
  {
    const uint32_t polls = cfg && cfg->wait_polls ? cfg->wait_polls : (1u << 24);
    if (cudaMemcpy(c->dev_err + kErrWaitPolls, &polls, 4, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(c->dev_err); delete c; cudaGetLastError(); return HB_ERR_CUDA; }
  }
  int r = hbk_moe_decode_setup(c);
  if (r == HB_OK) r = hbk_nvfp4_setup(c);
  if (r == HB_OK) r = hbk_dense_setup(c);
  if (r == HB_OK) r = hbk_moe_prefill_setup(c);
  if (r != HB_OK) { cudaFree(c->dev_err); delete c; return r; }
  *out = c;
  return HB_OK;
}

void hb_destroy(hb_ctx* ctx) {
  if (!ctx) return;
  if (ctx->dev_err) cudaFree(ctx->dev_err);
  if (ctx->dtc_maps) cudaFree(ctx->dtc_maps);
  if (ctx->prof_ev) {
    for (int i = 0; i < 2 * hb_ctx::kProfMax; ++i) cudaEventDestroy(ctx->prof_ev[i]);
    delete[] ctx->prof_ev;
    delete[] ctx->prof_name;
  }
  delete ctx;
}

int hb_profile_enable(hb_ctx* ctx, int on) {
  HB_CTX(ctx);
  if (on && !ctx->prof_ev) {
    ctx->prof_ev = new (std::nothrow) cudaEvent_t[2 * hb_ctx::kProfMax];
    ctx->prof_name = new (std::nothrow) const char*[hb_ctx::kProfMax];
    if (!ctx->prof_ev || !ctx->prof_name) return hb_fail(ctx, HB_ERR_CUDA, "profile: out of host memory");
    for (int i = 0; i < 2 * hb_ctx::kProfMax; ++i) HB_CUDA(ctx, cudaEventCreate(&ctx->prof_ev[i]));
  }
  ctx->prof_on = on != 0;
  ctx->prof_n = 0;
  return HB_OK;
}

int hb_profile_read(hb_ctx* ctx, hb_kernel_stat* out, int max_out, int* n_out) {
  HB_CTX(ctx); HB_PTR(ctx, out); HB_PTR(ctx, n_out);
  *n_out = 0;
  HB_CUDA(ctx, cudaDeviceSynchronize());
  int n = 0;
  for (int i = 0; i < ctx->prof_n; ++i) {
    float ms = 0.f;
    HB_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->prof_ev[2 * i], ctx->prof_ev[2 * i + 1]));
    int j = 0;
    while (j < n && strncmp(out[j].name, ctx->prof_name[i], sizeof out[j].name - 1) != 0) ++j;
    if (j == n) {
      if (n >= max_out) continue;
      memset(&out[n], 0, sizeof out[n]);
      strncpy(out[n].name, ctx->prof_name[i], sizeof out[n].name - 1);
      ++n;
    }
    out[j].launches++;
    out[j].total_ms += ms;
  }
  ctx->prof_n = 0;
  *n_out = n;
  return HB_OK;
}

const char* hb_last_error(const hb_ctx* ctx) { return ctx ? ctx->err : "null context"; }

const char* hb_status_string(int s) {
  switch (s) {
    case HB_OK: return "ok";
    case HB_ERR_INVALID: return "invalid argument";
    case HB_ERR_UNSUPPORTED: return "unsupported shape";
    case HB_ERR_CUDA: return "CUDA error";
    case HB_ERR_NO_DEVICE: return "no sm_100 device";
    case HB_ERR_WORKSPACE: return "bad workspace";
    case HB_ERR_DEVICE_FLAG: return "device-side bounded wait gave up";
    default: return "unknown status";
  }
}

int hb_sm_count(const hb_ctx* ctx) { return ctx ? ctx->sm_count : 0; }
uint64_t hb_launch_count(const hb_ctx* ctx) { return ctx ? ctx->launches : 0; }

int hb_check_device(hb_ctx* ctx, void* stream) {
  HB_CTX(ctx);
  uint32_t v = 0;
  HB_CUDA(ctx, cudaMemcpyAsync(&v, ctx->dev_err, 4, cudaMemcpyDeviceToHost, as_stream(stream)));
  HB_CUDA(ctx, cudaStreamSynchronize(as_stream(stream)));
  if (v == 0) return HB_OK;
  uint32_t site[2] = {0u, 0u};
  if (v & 0x80000000u) {                                                       // a range check of the debug build: which one, and the value it saw
    HB_CUDA(ctx, cudaMemcpyAsync(site, ctx->dev_err + kErrBoundSite, 8, cudaMemcpyDeviceToHost, as_stream(stream)));
    HB_CUDA(ctx, cudaMemsetAsync(ctx->dev_err + kErrBoundSite, 0, 8, as_stream(stream)));
    HB_CUDA(ctx, cudaStreamSynchronize(as_stream(stream)));
  }
  HB_CUDA(ctx, cudaMemsetAsync(ctx->dev_err, 0, 4, as_stream(stream)));
  if (v & 0x80000000u)
    return hb_fail(ctx, HB_ERR_DEVICE_FLAG, "device error word 0x%x: range check 0x%x failed with value %d (debug build)", v, site[0], (int)site[1]);
  return hb_fail(ctx, HB_ERR_DEVICE_FLAG, "device error word 0x%x (bits 0x1-0x80: a pipeline wait inside a decode or prefill kernel; 0x400-0x2000: the decode layer kernel's tables and grid barrier; "
                 "0x40000: rows of another rank did not arrive; 0x80000: partial sums of another rank did not arrive; 0x400000: an expert record outside the tensor maps' range)", v);
}

int hb_rec_layout_make(int H, int I, hb_rec_layout* L) {
  if (!L || H <= 0 || I <= 0 || (H % 32) || (I % 32)) return HB_ERR_INVALID;
  const uint64_t wgu = (uint64_t)I * H / 2, sgu = (uint64_t)I * H / 16;
  L->w1 = 0; L->s1 = wgu; L->w3 = L->s1 + sgu; L->s3 = L->w3 + wgu; L->w2 = L->s3 + sgu; L->s2 = L->w2 + wgu; L->g = L->s2 + sgu;
  L->total = (L->g + 16 + 4095) / 4096 * 4096;
  return HB_OK;
}

int hb_nvfp4_dequant(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, void* out, void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, w); HB_PTR(ctx, s); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, N > 0 && K > 0 && K % 16 == 0, HB_ERR_UNSUPPORTED, "nvfp4_dequant: N=%d K=%d (K %% 16)", N, K);
  HB_REQUIRE(ctx, hb_aligned(w, 8) && hb_aligned(out, 16), HB_ERR_INVALID, "nvfp4_dequant: w 8-byte, out 16-byte aligned");
  return hbk_nvfp4_dequant(ctx, w, s, g, N, K, out, as_stream(stream));
}

int hb_nvfp4_gemv(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, const void* x, int ldx, int M, float* y, int ldy,
                  void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, w); HB_PTR(ctx, s); HB_PTR(ctx, x); HB_PTR(ctx, y);
  HB_REQUIRE(ctx, M >= 1 && M <= 16, HB_ERR_UNSUPPORTED, "nvfp4_gemv: M=%d outside 1..16", M);
  HB_REQUIRE(ctx, N > 0 && K > 0 && K % 32 == 0, HB_ERR_UNSUPPORTED, "nvfp4_gemv: N=%d K=%d (K %% 32)", N, K);
  HB_REQUIRE(ctx, ldx >= K && ldx % 8 == 0 && ldy >= N, HB_ERR_INVALID, "nvfp4_gemv: ldx=%d (≥K, %% 8) ldy=%d (≥N)", ldx, ldy);
  HB_ALIGN16(ctx, w); HB_ALIGN16(ctx, x);
  HB_REQUIRE(ctx, hb_aligned(s, 2), HB_ERR_INVALID, "nvfp4_gemv: s must be 2-byte aligned");
  return hbk_nvfp4_gemv(ctx, w, s, g, N, K, x, ldx, M, y, ldy, as_stream(stream));
}

int hb_nvfp4_quantize(hb_ctx* ctx, const float* w, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax, void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, w); HB_PTR(ctx, q); HB_PTR(ctx, s); HB_PTR(ctx, g_mul); HB_PTR(ctx, amax);
  HB_REQUIRE(ctx, N > 0 && K > 0 && K % 16 == 0, HB_ERR_UNSUPPORTED, "nvfp4_quantize: N=%d K=%d (K %% 16)", N, K);
  HB_ALIGN16(ctx, w);
  HB_REQUIRE(ctx, hb_aligned(q, 8), HB_ERR_INVALID, "nvfp4_quantize: q must be 8-byte aligned");
  return hbk_nvfp4_quantize(ctx, w, N, K, q, s, g_mul, amax, as_stream(stream));
}

int hb_requant_nvfp4(hb_ctx* ctx, const uint8_t* w_fp8, const float* row_scale, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax, void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, w_fp8); HB_PTR(ctx, row_scale); HB_PTR(ctx, q); HB_PTR(ctx, s); HB_PTR(ctx, g_mul); HB_PTR(ctx, amax);
  HB_REQUIRE(ctx, N > 0 && K > 0 && K % 16 == 0, HB_ERR_UNSUPPORTED, "requant_nvfp4: N=%d K=%d (K %% 16)", N, K);
  HB_REQUIRE(ctx, hb_aligned(w_fp8, 4) && hb_aligned(q, 8), HB_ERR_INVALID, "requant_nvfp4: w_fp8 must be 4-byte aligned, q 8-byte aligned");
  return hbk_requant_nvfp4(ctx, w_fp8, row_scale, N, K, q, s, g_mul, amax, as_stream(stream));
}

int hb_a4_quant(hb_ctx* ctx, const void* x, int ld, int n, int K, uint8_t* q, uint8_t* s, float* g, void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, x); HB_PTR(ctx, q); HB_PTR(ctx, s); HB_PTR(ctx, g);
  HB_REQUIRE(ctx, n > 0 && K > 0 && K % 16 == 0 && ld >= K, HB_ERR_UNSUPPORTED, "a4_quant: n=%d K=%d ld=%d", n, K, ld);
  HB_REQUIRE(ctx, hb_aligned(q, 8), HB_ERR_INVALID, "a4_quant: q must be 8-byte aligned");
  return hbk_a4_quant(ctx, x, ld, n, K, q, s, g, as_stream(stream));
}

int hb_route_softmax_topk(hb_ctx* ctx, const float* logits, int ld, int M, int E, int k, int renorm, int logits_bf16, int32_t* ids, float* w,
                          void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, logits); HB_PTR(ctx, ids); HB_PTR(ctx, w);
  HB_REQUIRE(ctx, M > 0 && E > 0 && E <= HB_MAX_EXPERTS && k >= 1 && k <= 16 && k <= E && ld >= E, HB_ERR_UNSUPPORTED,
             "route_softmax_topk: M=%d E=%d (≤%d) k=%d (1..16) ld=%d", M, E, HB_MAX_EXPERTS, k, ld);
  return hbk_route_softmax_topk(ctx, logits, ld, M, E, k, renorm, logits_bf16, ids, w, as_stream(stream), pdl_on(ctx));
}

int hb_route_sigmoid_topk(hb_ctx* ctx, const float* logits, const float* bias, int M, int E, int k, float scale, int32_t* ids, float* w,
                          void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, logits); HB_PTR(ctx, ids); HB_PTR(ctx, w);
  HB_REQUIRE(ctx, M > 0 && E > 0 && E <= HB_MAX_EXPERTS && k >= 1 && k <= 16 && k <= E, HB_ERR_UNSUPPORTED,
             "route_sigmoid_topk: M=%d E=%d (≤%d) k=%d (1..16)", M, E, HB_MAX_EXPERTS, k);
  return hbk_route_sigmoid_topk(ctx, logits, bias, M, E, k, scale, ids, w, as_stream(stream), pdl_on(ctx));
}

int hb_build_moe_pairs(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                       hb_moe_pair* pairs, void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, ids); HB_PTR(ctx, w); HB_PTR(ctx, rec_tab); HB_PTR(ctx, pairs);
  HB_REQUIRE(ctx, M > 0 && K > 0 && E > 0 && li >= 0, HB_ERR_INVALID, "build_moe_pairs: M=%d K=%d E=%d li=%d", M, K, E, li);
  return hbk_build_pairs(ctx, ids, w, M, K, rec_tab, li, E, pairs, as_stream(stream), pdl_on(ctx));
}

int hb_moe_combine(hb_ctx* ctx, const float* routed, const void* shared, const float* lg, int ld, int col, int M, int H, void* out,
                   void* stream) {
  HB_CTX(ctx); HB_PTR(ctx, routed); HB_PTR(ctx, shared); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, M > 0 && H > 0, HB_ERR_INVALID, "moe_combine: M=%d H=%d", M, H);
  return hbk_moe_combine(ctx, routed, shared, lg, ld, col, M, H, out, as_stream(stream), pdl_on(ctx));
}

static int check_decode_shape(hb_ctx* ctx, const char* fn, long long P, int H, int I, const void* x, const void* ws) {
  HB_REQUIRE(ctx, H > 0 && I > 0 && H % 32 == 0 && I % 32 == 0, HB_ERR_UNSUPPORTED, "%s: H=%d I=%d must be multiples of 32", fn, H, I);
  HB_REQUIRE(ctx, P >= 1 && P <= HB_MAX_PAIRS, HB_ERR_UNSUPPORTED, "%s: %lld pairs outside 1..%d", fn, P, HB_MAX_PAIRS);
  HB_REQUIRE(ctx, ws != nullptr && hb_aligned(ws, 256), HB_ERR_WORKSPACE, "%s: ws NULL or not 256-byte aligned", fn);
  HB_REQUIRE(ctx, hb_aligned(x, 16), HB_ERR_INVALID, "%s: x must be 16-byte aligned", fn);
  return HB_OK;
}

int hb_moe_decode_supported(int H, int I) { return (H > 0 && I > 0 && H % 32 == 0 && I % 32 == 0) ? (hbk_moe_decode_fast(H, I) ? 2 : 1) : 0; }

size_t hb_moe_decode_ws_bytes(int n_pairs, int H, int I) { return hbk_moe_decode_ws_bytes(n_pairs, H, I); }

int hb_moe_decode(hb_ctx* ctx, const hb_moe_pair* pairs, int n_pairs, const void* x, int H, int I, float limit, float* out, void* ws,
                  void* stream) {
  HB_CTX(ctx);
  if (n_pairs == 0) return HB_OK;
  HB_PTR(ctx, pairs); HB_PTR(ctx, x); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, n_pairs > 0, HB_ERR_INVALID, "moe_decode: n_pairs=%d", n_pairs);
  int r = check_decode_shape(ctx, "moe_decode", n_pairs, H, I, x, ws);
  if (r) return r;
  HB_REQUIRE(ctx, hb_aligned(out, 8), HB_ERR_INVALID, "moe_decode: out must be 8-byte aligned");
  hbk_pair_src src; src.pairs = pairs; src.n_pairs = n_pairs;
  hbk_reduce red; red.out_accum = out;
  return hbk_moe_decode_run(ctx, src, x, H, I, limit, red, ws, as_stream(stream));
}

int hb_moe_decode_routed(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                         const void* x, int H, int I, float limit, const hb_pf_combine* cmb, void* ws, void* stream) {
  HB_CTX(ctx);
  if (M == 0) return HB_OK;
  HB_PTR(ctx, ids); HB_PTR(ctx, w); HB_PTR(ctx, rec_tab); HB_PTR(ctx, x); HB_PTR(ctx, cmb); HB_PTR(ctx, cmb->out);
  HB_REQUIRE(ctx, M > 0 && K > 0 && E > 0 && E <= HB_MAX_EXPERTS && li >= 0, HB_ERR_INVALID, "moe_decode_routed: M=%d K=%d E=%d li=%d", M, K, E, li);
  int r = check_decode_shape(ctx, "moe_decode_routed", (long long)M * K, H, I, x, ws);
  if (r) return r;
  hbk_pair_src src; src.ids = ids; src.w = w; src.M = M; src.K = K; src.tab = rec_tab; src.li = li; src.E = E;
  hbk_reduce red; red.shared = cmb->shared; red.lg = cmb->lg; red.ld = cmb->ld; red.col = cmb->col; red.out_bf16 = cmb->out;
  return hbk_moe_decode_run(ctx, src, x, H, I, limit, red, ws, as_stream(stream));
}

int hb_moe_decode_routed_f32(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                             const void* x, int H, int I, float limit, float* out, void* ws, void* stream) {
  HB_CTX(ctx);
  if (M == 0) return HB_OK;
  HB_PTR(ctx, ids); HB_PTR(ctx, w); HB_PTR(ctx, rec_tab); HB_PTR(ctx, x); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, M > 0 && K > 0 && E > 0 && E <= HB_MAX_EXPERTS && li >= 0, HB_ERR_INVALID, "moe_decode_routed_f32: M=%d K=%d E=%d li=%d", M, K, E, li);
  int r = check_decode_shape(ctx, "moe_decode_routed_f32", (long long)M * K, H, I, x, ws);
  if (r) return r;
  hbk_pair_src src; src.ids = ids; src.w = w; src.M = M; src.K = K; src.tab = rec_tab; src.li = li; src.E = E;
  hbk_reduce red; red.out_f32 = out;
  return hbk_moe_decode_run(ctx, src, x, H, I, limit, red, ws, as_stream(stream));
}

int hb_moe_decode_ep_local(hb_ctx* ctx, const int32_t* ids, const float* w, int ld_ids, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                           const void* x, int ldx, int H, int I, float limit, const uint8_t* shared_rec, int sh_row0, int sh_rows, float* routed_out,
                           void* shared_out, void* ws, void* stream) {
  HB_CTX(ctx);
  if (M == 0) return HB_OK;
  HB_PTR(ctx, ids); HB_PTR(ctx, w); HB_PTR(ctx, rec_tab); HB_PTR(ctx, x); HB_PTR(ctx, routed_out);
  HB_REQUIRE(ctx, M > 0 && K > 0 && E > 0 && E <= HB_MAX_EXPERTS && li >= 0 && ld_ids >= K && ldx >= H && ldx % 8 == 0, HB_ERR_INVALID,
             "moe_decode_ep_local: M=%d K=%d E=%d li=%d ld_ids=%d ldx=%d (ldx a multiple of 8)", M, K, E, li, ld_ids, ldx);
  HB_REQUIRE(ctx, !shared_rec || (shared_out && sh_row0 >= 0 && sh_rows >= 0 && sh_row0 + sh_rows <= M), HB_ERR_INVALID,
             "moe_decode_ep_local: shared expert rows [%d, %d) outside the %d rows, or no output for them", sh_row0, sh_row0 + sh_rows, M);
  int r = check_decode_shape(ctx, "moe_decode_ep_local", (long long)M * (K + (shared_rec ? 1 : 0)), H, I, x, ws);
  if (r) return r;
  hbk_pair_src src; src.ids = ids; src.w = w; src.M = M; src.K = K; src.tab = rec_tab; src.li = li; src.E = E;
  src.ld_ids = ld_ids; src.x_ld = ldx; src.shared_rec = shared_rec; src.sh_row0 = sh_row0; src.sh_rows = shared_rec ? sh_rows : 0;
  hbk_reduce red; red.out_f32 = routed_out; red.shared_out = shared_rec ? shared_out : nullptr;
  return hbk_moe_decode_run(ctx, src, x, H, I, limit, red, ws, as_stream(stream));
}

int hb_moe_layer_decode(hb_ctx* ctx, const float* logits, int ld, int M, int E, int K, int renorm, int logits_bf16, const float* bias,
                        float sigmoid_scale, const uint8_t* const* rec_tab, int li, const uint8_t* shared_rec, int gate_col, const void* x,
                        int H, int I, float limit, int32_t* ids_out, float* w_out, void* out, void* ws, void* stream) {
  HB_CTX(ctx);
  if (M == 0) return HB_OK;
  HB_PTR(ctx, logits); HB_PTR(ctx, rec_tab); HB_PTR(ctx, x); HB_PTR(ctx, ids_out); HB_PTR(ctx, w_out); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, M > 0 && K >= 1 && K <= 16 && E > 0 && E <= HB_MAX_EXPERTS && K <= E && ld >= E && li >= 0, HB_ERR_INVALID,
             "moe_layer_decode: M=%d K=%d E=%d ld=%d li=%d", M, K, E, ld, li);
  HB_REQUIRE(ctx, gate_col < ld, HB_ERR_INVALID, "moe_layer_decode: gate_col=%d outside the logits row (ld=%d)", gate_col, ld);
  int r = check_decode_shape(ctx, "moe_layer_decode", (long long)M * (K + 1), H, I, x, ws);
  if (r) return r;
  const bool sigmoid = bias != nullptr || sigmoid_scale != 0.f;
  if (sigmoid) HB_REQUIRE(ctx, ld == E, HB_ERR_INVALID, "moe_layer_decode: the sigmoid router takes dense logits rows (ld == E)");
  // routing runs inside the grouping kernel (one launch for route + sort)
  hbk_pair_src src; src.ids = ids_out; src.w = w_out; src.M = M; src.K = K; src.tab = rec_tab; src.li = li; src.E = E; src.shared_rec = shared_rec;
  src.route = sigmoid ? 2 : 1; src.logits = logits; src.ld = ld; src.renorm = renorm; src.logits_bf16 = logits_bf16; src.bias = bias;
  src.sig_scale = sigmoid_scale != 0.f ? sigmoid_scale : 1.f;
  hbk_reduce red; red.out_bf16 = out;
  if (gate_col >= 0 && shared_rec) { red.lg = logits; red.ld = ld; red.col = gate_col; }
  return hbk_moe_decode_run(ctx, src, x, H, I, limit, red, ws, as_stream(stream));
}

// ---- a whole MoE layer for any number of rows: the dispatcher ----
namespace {
constexpr int kDecodeRows = 64;          // rows ≤ 64: decode operators; more: grouped GEMM (engine/src/qwen/qwen_engine.cpp:825, :873)
struct LayerWs { void* op; const uint8_t** tab1; int32_t* ids1; float* w1; float* sh32; void* sh16; };
size_t layer_carve(void* ws, int M, int K, int E, int H, int I, LayerWs* w) {
  size_t off = 0;
  auto take = [&](size_t b) { void* r = ws ? static_cast<char*>(ws) + off : nullptr; off += hb_align256(b); return r; };
  LayerWs t;
  const bool pf = M > kDecodeRows && hb_moe_prefill_supported(H, I) > 0;
  const int rows = M < kDecodeRows ? M : kDecodeRows;
  t.op = take(pf ? hb_moe_prefill_ws_bytes(M, K, E, H, I) : hb_moe_decode_ws_bytes(rows * (K + 1), H, I));
  t.tab1 = (const uint8_t**)take(256); t.ids1 = (int32_t*)take(pf ? (size_t)M * 4 : 0); t.w1 = (float*)take(pf ? (size_t)M * 4 : 0);
  t.sh32 = (float*)take(pf ? (size_t)M * H * 4 : 0); t.sh16 = take(pf ? (size_t)M * H * 2 : 0);
  if (w) *w = t;
  return off;
}
}  // namespace

size_t hb_moe_layer_ws_bytes(int M, int K, int E, int H, int I) {
  if (M < 1 || K < 1 || E < 1 || hb_moe_decode_supported(H, I) <= 0) return 0;
  return layer_carve(nullptr, M, K, E, H, I, nullptr);
}

int hb_moe_layer(hb_ctx* ctx, const float* logits, int ld, int M, int E, int K, int renorm, int logits_bf16, const float* bias, float sigmoid_scale,
                 const uint8_t* const* rec_tab, int li, const uint8_t* shared_rec, int gate_col, const void* x, int H, int I, float limit,
                 int32_t* ids_out, float* w_out, void* out, void* ws, void* stream) {
  HB_CTX(ctx);
  if (M == 0) return HB_OK;
  HB_PTR(ctx, logits); HB_PTR(ctx, rec_tab); HB_PTR(ctx, x); HB_PTR(ctx, ids_out); HB_PTR(ctx, w_out); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, M > 0 && K >= 1 && K <= 16 && E > 0 && E <= HB_MAX_EXPERTS && K <= E && ld >= E && li >= 0 && gate_col < ld, HB_ERR_INVALID,
             "moe_layer: M=%d K=%d E=%d ld=%d li=%d gate_col=%d", M, K, E, ld, li, gate_col);
  HB_REQUIRE(ctx, ws && hb_aligned(ws, 256), HB_ERR_WORKSPACE, "moe_layer: ws NULL or not 256-byte aligned");
  LayerWs W;
  layer_carve(ws, M, K, E, H, I, &W);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(out);
  if (M <= kDecodeRows || !(ctx->flags & (HB_FLAG_LAYER_A4 | HB_FLAG_PREFILL_A16)) || hb_moe_prefill_supported(H, I) <= 0) {
    // decode operators, 64 rows at a time (one pass when M ≤ 64): per-row results do not depend on the batch.  More rows go to a
    // grouped GEMM only when the context asked for one: HB_FLAG_PREFILL_A16 keeps bf16 activations (the same arithmetic, fp32 sums in
    // the tensor core's order), HB_FLAG_LAYER_A4 quantises the activations (W4A4); with both, hb_moe_prefill keeps bf16 activations
    for (int m0 = 0; m0 < M; m0 += kDecodeRows) {
      const int n = M - m0 < kDecodeRows ? M - m0 : kDecodeRows;
      const int r = hb_moe_layer_decode(ctx, logits + (size_t)m0 * ld, ld, n, E, K, renorm, logits_bf16, bias, sigmoid_scale, rec_tab, li, shared_rec, gate_col,
                                        xb + (size_t)m0 * H, H, I, limit, ids_out + (size_t)m0 * K, w_out + (size_t)m0 * K, ob + (size_t)m0 * H, W.op, stream);
      if (r) return r;
    }
    return HB_OK;
  }
  // grouped GEMM: route → shared expert as a one-expert routing over all rows → routed experts with the fused combine
  const bool sigmoid = bias != nullptr || sigmoid_scale != 0.f;
  if (sigmoid) HB_REQUIRE(ctx, ld == E, HB_ERR_INVALID, "moe_layer: the sigmoid router takes dense logits rows (ld == E)");
  cudaStream_t st = as_stream(stream);
  int r = sigmoid ? hbk_route_sigmoid_topk(ctx, logits, bias, M, E, K, sigmoid_scale != 0.f ? sigmoid_scale : 1.f, ids_out, w_out, st, false)
                  : hbk_route_softmax_topk(ctx, logits, ld, M, E, K, renorm, logits_bf16, ids_out, w_out, st, false);
  if (r) return r;
  hb_pf_combine cmb = {};
  if (shared_rec) {
    if ((r = hbk_layer_prep(ctx, W.tab1, W.ids1, W.w1, M, shared_rec, st))) return r;
    if ((r = hb_moe_prefill(ctx, W.tab1, 0, 1, W.ids1, W.w1, M, 1, x, H, I, limit, W.sh32, W.op, M, stream, nullptr))) return r;
    if ((r = hbk_f32_to_bf16(ctx, W.sh32, W.sh16, (size_t)M * H, st))) return r;      // exact: the values are bf16 already
    cmb.shared = W.sh16; cmb.lg = gate_col >= 0 ? logits : nullptr; cmb.ld = ld; cmb.col = gate_col >= 0 ? gate_col : 0; cmb.out = out;
    return hb_moe_prefill(ctx, rec_tab, li, E, ids_out, w_out, M, K, x, H, I, limit, nullptr, W.op, M, stream, &cmb);
  }
  // no shared expert: out = bf16(routed sum)
  if ((r = hb_moe_prefill(ctx, rec_tab, li, E, ids_out, w_out, M, K, x, H, I, limit, W.sh32, W.op, M, stream, nullptr))) return r;
  return hbk_f32_to_bf16(ctx, W.sh32, out, (size_t)M * H, st);
}

int hb_expert_dequant(hb_ctx* ctx, const uint8_t* rec, int H, int I, void* gu_bf16, void* d_bf16, void* stream) {
  HB_CTX(ctx);
  HB_PTR(ctx, rec); HB_PTR(ctx, gu_bf16); HB_PTR(ctx, d_bf16);
  hb_rec_layout L;
  HB_REQUIRE(ctx, hb_rec_layout_make(H, I, &L) == HB_OK && hb_aligned(rec, 16) && hb_aligned(gu_bf16, 16) && hb_aligned(d_bf16, 16), HB_ERR_INVALID,
             "expert_dequant: H=%d I=%d, or misaligned pointers", H, I);
  const float* g = reinterpret_cast<const float*>(rec + L.g);
  __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(gu_bf16);
  int r = hbk_nvfp4_dequant(ctx, rec + L.w1, rec + L.s1, 0.f, I, H, gu, as_stream(stream), g);
  if (!r) r = hbk_nvfp4_dequant(ctx, rec + L.w3, rec + L.s3, 0.f, I, H, gu + (size_t)I * H, as_stream(stream), g + 1);
  if (!r) r = hbk_nvfp4_dequant(ctx, rec + L.w2, rec + L.s2, 0.f, H, I, d_bf16, as_stream(stream), g + 2);
  return r;
}
int hb_gather_rows(hb_ctx* ctx, const void* x, const int32_t* rows, int R, int H, void* out, void* stream) {
  HB_CTX(ctx);
  if (R == 0) return HB_OK;
  HB_PTR(ctx, x); HB_PTR(ctx, rows); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, R > 0 && H > 0 && H % 8 == 0, HB_ERR_UNSUPPORTED, "gather_rows: R=%d H=%d (H %% 8)", R, H);
  HB_ALIGN16(ctx, x); HB_ALIGN16(ctx, out);
  return hbk_gather_rows(ctx, x, rows, R, H, out, as_stream(stream));
}
int hb_swiglu_rows(hb_ctx* ctx, const void* gu, int R, int I, float limit, void* y, void* stream) {
  HB_CTX(ctx);
  if (R == 0) return HB_OK;
  HB_PTR(ctx, gu); HB_PTR(ctx, y);
  HB_REQUIRE(ctx, R > 0 && I > 0, HB_ERR_INVALID, "swiglu_rows: R=%d I=%d", R, I);
  return hbk_swiglu_rows(ctx, gu, R, I, limit, y, as_stream(stream));
}
int hb_scatter_add_rows(hb_ctx* ctx, const void* e, const int32_t* rows, const float* w, int R, int H, float* out, void* stream) {
  HB_CTX(ctx);
  if (R == 0) return HB_OK;
  HB_PTR(ctx, e); HB_PTR(ctx, rows); HB_PTR(ctx, w); HB_PTR(ctx, out);
  HB_REQUIRE(ctx, R > 0 && H > 0, HB_ERR_INVALID, "scatter_add_rows: R=%d H=%d", R, H);
  return hbk_scatter_add_rows(ctx, e, rows, w, R, H, out, as_stream(stream));
}
int hb_add_f32(hb_ctx* ctx, float* a, const float* b, size_t n, void* stream) {
  HB_CTX(ctx);
  if (n == 0) return HB_OK;
  HB_PTR(ctx, a); HB_PTR(ctx, b);
  return hbk_add_f32(ctx, a, b, n, as_stream(stream));
}


// Rows ≤ 64 go to the decode operators, more to the grouped GEMM — the reference engine's own switch
// (engine/src/qwen/qwen_engine.cpp:825, :873) — provided the shape is one the grouped GEMM takes.
int hb_dispatch_plan(const int32_t* ids, int M, int K, int E, int H, int I, int* counts, hb_plan* plan) {
  if (!ids || !plan || M < 0 || K < 1 || E < 1 || E > HB_MAX_EXPERTS) return HB_ERR_INVALID;
  int local[HB_MAX_EXPERTS];
  int* c = counts ? counts : local;
  for (int e = 0; e < E; ++e) c[e] = 0;
  hb_plan p = {};
  for (long long i = 0; i < (long long)M * K; ++i) {
    const int e = ids[i];
    if (e >= 0 && e < E) { ++c[e]; ++p.pairs; }
  }
  for (int e = 0; e < E; ++e) {
    if (!c[e]) continue;
    ++p.distinct_experts;
    if (c[e] > p.max_rows) p.max_rows = c[e];
    p.decode_groups += (c[e] + 7) / 8;
    p.prefill_tiles += (c[e] + 127) / 128;
  }
  p.tile_fill = p.prefill_tiles ? (double)p.pairs / (128.0 * p.prefill_tiles) : 0.0;
  const bool pf_ok = hb_moe_prefill_supported(H, I) > 0;
  p.regime = (M > 64 && pf_ok) ? 1 : 0;
  if (p.regime == 1) p.ws_bytes = hb_moe_prefill_ws_bytes(M, K, E, H, I);
  else p.ws_bytes = ((long long)M * K <= HB_MAX_PAIRS && hb_moe_decode_supported(H, I) > 0) ? hb_moe_decode_ws_bytes(M * K, H, I) : 0;
  *plan = p;
  return HB_OK;
}

}  // extern "C"
