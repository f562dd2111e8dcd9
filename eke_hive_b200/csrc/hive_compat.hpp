// Drop-in C++ surface: the reference engine's expert-compute free functions (namespaces hive::glm and hive::qwen) implemented
// over the C ABI of libhive_b200.so.  A reference call site keeps its includes' names and argument lists; link with -lhive_b200
// instead of the engine's own CUDA objects.  Failures become exceptions of type hive::b200::Error here (the reference aborts
// through HIVE_CHECK); catch them at the engine's boundary or let them terminate like the abort did.
//
//   hive::glm::ExpertRecLayout, MoePair, moe_decode_ws_bytes, moe_decode,
//   gather_rows, swiglu_rows, scatter_add_rows, add_f32            engine/include/hive/glm/glm_moe.h:13-41
//   hive::glm::Nvfp4Mat, nvfp4_gemv, nvfp4_dequant                 engine/include/hive/glm/nvfp4.h:13-23
//   hive::glm::router_topk                                         engine/include/hive/glm/glm_kernels.h:12-17
//   hive::qwen::fn_moe_decode(_ws_bytes,_supported,_routed)        engine/include/hive/qwen/fn_moe.h:18-31
//   hive::qwen::router_softmax_topk, moe_combine, build_moe_pairs  engine/include/hive/qwen/qwen_kernels.h:51-66
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/hive_b200.h"

namespace hive::b200 {
struct Error : std::runtime_error { int status; Error(int s, const std::string& m) : std::runtime_error(m), status(s) {} };
// One context per device, created on first use (the reference's operators are free functions without a handle).
inline hb_ctx* ctx() {
  static thread_local hb_ctx* c[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!c[dev]) {
    hb_config cfg{dev, 0, 0, 0};
    const int st = hb_create(&cfg, &c[dev]);
    if (st != HB_OK) throw Error(st, std::string("hb_create: ") + hb_status_string(st));
  }
  return c[dev];
}
// A second context per device whose hb_moe_prefill keeps bf16 activations (W4A16, the reference's default prefill arithmetic).
inline hb_ctx* ctx_a16() {
  static thread_local hb_ctx* c[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!c[dev]) {
    hb_config cfg{dev, 0, (int)HB_FLAG_PREFILL_A16, 0};
    const int st = hb_create(&cfg, &c[dev]);
    if (st != HB_OK) throw Error(st, std::string("hb_create: ") + hb_status_string(st));
  }
  return c[dev];
}
inline bool& prefill_a4_flag() { static bool on = false; return on; }   // the reference's default: bf16 activations (fn_moe.h:50-52)
inline void check(int st) { if (st != HB_OK) throw Error(st, hb_last_error(ctx())); }
inline void check_on(hb_ctx* c, int st) { if (st != HB_OK) throw Error(st, hb_last_error(c)); }
}  // namespace hive::b200

namespace hive::glm {
struct ExpertRecLayout {
  size_t w1, s1, w3, s3, w2, s2, g, total;
  static ExpertRecLayout make(int H, int I) {
    hb_rec_layout r;
    if (hb_rec_layout_make(H, I, &r) != HB_OK) throw b200::Error(HB_ERR_INVALID, "ExpertRecLayout::make: bad shape");
    return ExpertRecLayout{(size_t)r.w1, (size_t)r.s1, (size_t)r.w3, (size_t)r.s3, (size_t)r.w2, (size_t)r.s2, (size_t)r.g, (size_t)r.total};
  }
};
struct MoePair { int row; const uint8_t* rec; float w; };
static_assert(sizeof(MoePair) == sizeof(hb_moe_pair), "MoePair ABI");
struct Nvfp4Mat { const uint8_t* w = nullptr; const uint8_t* s = nullptr; float g = 1.f; int N = 0, K = 0; };

inline size_t moe_decode_ws_bytes(int n_pairs, int H, int I) { return hb_moe_decode_ws_bytes(n_pairs, H, I); }
inline void moe_decode(const ExpertRecLayout&, const MoePair* pairs, int n_pairs, const __nv_bfloat16* x, int H, int I, float limit, float* out, void* ws,
                       cudaStream_t st) {
  b200::check(hb_moe_decode(b200::ctx(), reinterpret_cast<const hb_moe_pair*>(pairs), n_pairs, x, H, I, limit, out, ws, st));
}
inline void nvfp4_gemv(const Nvfp4Mat& W, const __nv_bfloat16* x, int ldx, int M, float* y, int ldy, cudaStream_t st) {
  b200::check(hb_nvfp4_gemv(b200::ctx(), W.w, W.s, W.g, W.N, W.K, x, ldx, M, y, ldy, st));
}
inline void nvfp4_dequant(const Nvfp4Mat& W, __nv_bfloat16* out, cudaStream_t st) {
  b200::check(hb_nvfp4_dequant(b200::ctx(), W.w, W.s, W.g, W.N, W.K, out, st));
}
inline void expert_dequant(const ExpertRecLayout&, const uint8_t* rec, int H, int I, __nv_bfloat16* gu, __nv_bfloat16* d, cudaStream_t st) {
  b200::check(hb_expert_dequant(b200::ctx(), rec, H, I, gu, d, st));
}
inline void swiglu_rows(const __nv_bfloat16* gu_out, int R, int I, float limit, __nv_bfloat16* y, cudaStream_t st) {
  b200::check(hb_swiglu_rows(b200::ctx(), gu_out, R, I, limit, y, st));
}
inline void scatter_add_rows(const __nv_bfloat16* e, const int32_t* rows, const float* w, int R, int H, float* out, cudaStream_t st) {
  b200::check(hb_scatter_add_rows(b200::ctx(), e, rows, w, R, H, out, st));
}
inline void gather_rows(const __nv_bfloat16* x, const int32_t* rows, int R, int H, __nv_bfloat16* out, cudaStream_t st) {
  b200::check(hb_gather_rows(b200::ctx(), x, rows, R, H, out, st));
}
inline void add_f32(float* a, const float* b, size_t n, cudaStream_t st) { b200::check(hb_add_f32(b200::ctx(), a, b, n, st)); }
inline void router_topk(const float* logits, const float* bias, int M, int E, int k, float scale, int32_t* ids, float* w, cudaStream_t st) {
  b200::check(hb_route_sigmoid_topk(b200::ctx(), logits, bias, M, E, k, scale, ids, w, st));
}
}  // namespace hive::glm

namespace hive::qwen {
struct FnPfCombine { const __nv_bfloat16* shared; const float* lg; int ld, col; __nv_bfloat16* out; };
struct MoePairDev { int row; const uint8_t* rec; float w; };

inline bool fn_moe_decode_supported(int H, int I) { return hb_moe_decode_supported(H, I) > 0; }
inline size_t fn_moe_decode_ws_bytes(int n_pairs, int H, int I) { return hb_moe_decode_ws_bytes(n_pairs, H, I); }
inline void fn_moe_decode(const glm::ExpertRecLayout&, const glm::MoePair* pairs, int n_pairs, const __nv_bfloat16* x, int H, int I, float* out, void* ws,
                          cudaStream_t st) {
  b200::check(hb_moe_decode(b200::ctx(), reinterpret_cast<const hb_moe_pair*>(pairs), n_pairs, x, H, I, 0.f, out, ws, st));
}
// The hybrid arguments of the reference (add / join / host_tab / pcie_div: CPU and PCIe shares of non-resident experts) have no
// counterpart: on B200 every expert is resident.  Passing any of them is an error rather than a silent difference.
inline void fn_moe_decode_routed(const glm::ExpertRecLayout&, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                                 const __nv_bfloat16* x, int H, int I, const __nv_bfloat16* shared, const float* lg, int ld, int col, __nv_bfloat16* out,
                                 void* ws, cudaStream_t st, const float* add = nullptr, cudaEvent_t join = nullptr,
                                 const uint8_t* const* host_tab = nullptr, int pcie_div = 0) {
  if (add || join || host_tab || pcie_div) throw b200::Error(HB_ERR_UNSUPPORTED, "fn_moe_decode_routed: hybrid CPU/PCIe arguments are not supported");
  hb_pf_combine c{shared, lg, ld, col, out};
  b200::check(hb_moe_decode_routed(b200::ctx(), ids, w, M, K, rec_tab, li, E, x, H, I, 0.f, &c, ws, st));
}
// Prefill (engine/include/hive/qwen/fn_moe.h:46-61).  As in the reference, bf16 activations (W4A16) are the default and
// fn_moe_prefill_set_a4(true) opts in to NVFP4 activations (W4A4, the block-scaled tensor-core grouped GEMM).  The W4A16 form here
// is a kind::f16 tensor-core grouped GEMM over exactly dequantised weight tiles for calls of more than 64 rows, and the decode
// operators below that.
inline bool fn_moe_prefill_supported(int H, int I) { return hb_moe_prefill_supported(H, I) > 0; }
inline bool fn_moe_prefill_a4() { return b200::prefill_a4_flag(); }
inline void fn_moe_prefill_set_a4(bool on) { b200::prefill_a4_flag() = on; }
inline size_t fn_moe_prefill_ws_bytes(int S, int K, int E, int H, int I) { return hb_moe_prefill_ws_bytes(S, K, E, H, I); }
inline void fn_moe_prefill(const glm::ExpertRecLayout&, const uint8_t* const* tab, int li, int E, const int32_t* ids, const float* w, int M, int K,
                           const __nv_bfloat16* x, int H, int I, float* out, void* ws, int S, cudaStream_t st, const FnPfCombine* cmb = nullptr) {
  hb_pf_combine c{};
  if (cmb) c = hb_pf_combine{cmb->shared, cmb->lg, cmb->ld, cmb->col, cmb->out};
  hb_ctx* hc = b200::prefill_a4_flag() ? b200::ctx() : b200::ctx_a16();
  b200::check_on(hc, hb_moe_prefill(hc, tab, li, E, ids, w, M, K, x, H, I, 0.f, out, ws, S, st, cmb ? &c : nullptr));
}
inline void router_softmax_topk(const float* logits, int ld, int M, int E, int k, bool renorm, int32_t* ids, float* w, int32_t* ids_host, float* w_host,
                                cudaStream_t st) {
  b200::check(hb_route_softmax_topk(b200::ctx(), logits, ld, M, E, k, renorm ? 1 : 0, 1, ids, w, st));
  if (ids_host) {  // the reference writes mapped-host copies from the kernel; here they are stream-ordered copies
    cudaMemcpyAsync(ids_host, ids, sizeof(int32_t) * (size_t)M * k, cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(w_host, w, sizeof(float) * (size_t)M * k, cudaMemcpyDeviceToHost, st);
  }
}
inline void moe_combine(const float* routed, const __nv_bfloat16* shared, const float* logits, int ld, int col, int M, int dim, __nv_bfloat16* out,
                        cudaStream_t st) {
  b200::check(hb_moe_combine(b200::ctx(), routed, shared, logits, ld, col, M, dim, out, st));
}
inline void build_moe_pairs(const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E, MoePairDev* pairs,
                            cudaStream_t st) {
  b200::check(hb_build_moe_pairs(b200::ctx(), ids, w, M, K, rec_tab, li, E, reinterpret_cast<hb_moe_pair*>(pairs), st));
}
}  // namespace hive::qwen

// Loading (engine/include/hive/ckpt_quant.h:35-37, engine/src/glm/glm_experts.cpp:216-287).  The reference decodes compressed block
// scales and assembles records on host threads; these run on the device over tensors already uploaded, so the signatures differ:
// device pointers, a stream, and a device status word instead of `false` / an exception.
namespace hive::ckq {
inline size_t csf_decode_ws_bytes(int R, int C) { return hb_csf_ws_bytes(R, C); }
// status: device int32[2] = {HB_CSF_* code, position}; shapes the format rules out throw like every other misuse
inline void csf_decode(const uint8_t* fixed, int64_t fixed_rows, int64_t fixed_cols, const uint32_t* exc, size_t n_exc, int R, int C, uint8_t* out,
                       int32_t* status, void* ws, size_t ws_bytes, cudaStream_t st) {
  b200::check(hb_csf_decode(b200::ctx(), fixed, fixed_rows, fixed_cols, exc, n_exc, R, C, out, status, ws, ws_bytes, st));
}
}  // namespace hive::ckq
namespace hive::glm {
inline size_t records_pack_ws_bytes(int H, int I, int n) { return hb_record_pack_ws_bytes(H, I, n); }
// jobs: device array [n]; status: device int32 [n][3][2]
inline void records_pack(const hb_record_job* jobs, int n, int H, int I, int32_t* status, void* ws, size_t ws_bytes, cudaStream_t st) {
  b200::check(hb_record_pack_batch(b200::ctx(), jobs, n, H, I, status, ws, ws_bytes, st));
}
}  // namespace hive::glm

// Dense decode GEMV of the 27B-style MLP (engine/include/hive/q27/q27_kernels.h:17-64).  GMat here carries the formats this library
// streams: NVFP4 as in the reference, plus the 3-/2-bit group-64 layouts hb_qmat defines.  The workspace the reference keeps
// inside its kernels is explicit: ws ≥ hb_dense_gemv_ws_bytes(fmt, N, K, 1 or 2).
namespace hive::q27 {
struct GMat { hb_qmat m; };
namespace k {
inline size_t gemv_ws_bytes(const GMat& W, int n_mats = 1) { return hb_dense_gemv_ws_bytes(W.m.fmt, W.m.N, W.m.K, n_mats); }
inline void gemv(const GMat& W, const __nv_bfloat16* x, int ldx, int M, __nv_bfloat16* yb, float* yf, int ldy, void* ws, cudaStream_t st) {
  b200::check(hb_dense_gemv(b200::ctx(), &W.m, x, ldx, M, yb, yf, ldy, ws, st));
}
inline void gemv_gu(const GMat& G, const GMat& U, const __nv_bfloat16* x, int ldx, int M, __nv_bfloat16* act, int lda, void* ws, cudaStream_t st) {
  b200::check(hb_dense_gemv_gu(b200::ctx(), &G.m, &U.m, x, ldx, M, act, lda, ws, st));
}
}  // namespace k
}  // namespace hive::q27
